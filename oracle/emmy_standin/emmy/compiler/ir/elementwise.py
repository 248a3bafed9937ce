import math

# Algebraic facts about the scalar operators, as the reference's passes query them.
_IDENTITY = {'add': 0.0, 'multiply': 1.0, 'maximum': -math.inf, 'minimum': math.inf}
_ASSOCIATIVE = frozenset(_IDENTITY)
_SELECTING = frozenset(('maximum', 'minimum'))
# (product, sum) pairs of semirings: the usual one and the two tropical ones
_DISTRIBUTES = frozenset((('multiply', 'add'), ('add', 'maximum'), ('add', 'minimum')))


class ElementwiseImpl:
    __slots__ = ('name',)

    def __init__(self, name):
        if isinstance(name, ElementwiseImpl):
            name = name.name
        if type(name) is not str or not name:
            raise ValueError('ElementwiseImpl takes an operator name')
        object.__setattr__(self, 'name', name)

    def __setattr__(self, key, value):
        raise AttributeError('ElementwiseImpl is immutable')

    def __repr__(self):
        return f'ElementwiseImpl({self.name!r})'

    def __eq__(self, other):
        return isinstance(other, ElementwiseImpl) and other.name == self.name

    def __hash__(self):
        return hash(('ElementwiseImpl', self.name))

    @property
    def identity(self):
        return _IDENTITY.get(self.name)

    @property
    def associative(self):
        return self.name in _ASSOCIATIVE

    @property
    def commutative(self):
        return self.name in _ASSOCIATIVE

    @property
    def selecting(self):
        return self.name in _SELECTING

    @property
    def semiring_product(self):
        return self.name == 'multiply'

    def distributes_over(self, other):
        return (self.name, getattr(other, 'name', other)) in _DISTRIBUTES
