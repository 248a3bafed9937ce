class Dim:
    """A static extent."""
    __slots__ = ('value',)

    def __init__(self, value):
        object.__setattr__(self, 'value', value)

    def __setattr__(self, name, value):
        raise AttributeError('Dim is immutable')

    def as_static(self):
        return self.value

    def __int__(self):
        return int(self.value)

    __index__ = __int__

    def __repr__(self):
        return f'Dim({self.value!r})'

    def __eq__(self, other):
        return isinstance(other, Dim) and other.value == self.value

    def __hash__(self):
        return hash(('Dim', self.value))
