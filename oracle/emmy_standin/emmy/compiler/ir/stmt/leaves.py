from dataclasses import dataclass
from typing import Any

from emmy.compiler.ir.elementwise import ElementwiseImpl
from emmy.compiler.ir.stmt.base import Stmt


def _names(value):
    if value is None:
        return None
    return (value,) if isinstance(value, str) else tuple(value)


def _operator(value):
    return value if isinstance(value, ElementwiseImpl) else ElementwiseImpl(value)


# Real dataclasses, so that dataclasses.replace() works on them; the coercions live in __post_init__.


@dataclass(frozen=True)
class Load(Stmt):
    names: Any = None
    input: Any = None
    index: Any = ()
    dtype: Any = None

    def __init__(self, name=None, input=None, index=(), dtype=None, names=None):
        object.__setattr__(self, 'names', _names(names if names is not None else name))
        object.__setattr__(self, 'input', input)
        object.__setattr__(self, 'index', tuple(index) if isinstance(index, (list, tuple)) else index)
        object.__setattr__(self, 'dtype', dtype)

    @property
    def name(self):
        return self.names[0]


@dataclass(frozen=True)
class Assign(Stmt):
    name: str
    op: Any
    args: Any
    dtype: Any = None

    def __post_init__(self):
        object.__setattr__(self, 'op', _operator(self.op))
        object.__setattr__(self, 'args', _names(self.args))


@dataclass(frozen=True)
class Accum(Stmt):
    name: str
    value: str
    op: Any
    dtype: Any = None
    axes: Any = ()
    base: Any = None

    def __post_init__(self):
        object.__setattr__(self, 'op', _operator(self.op))
        object.__setattr__(self, 'axes', _names(self.axes) or ())


@dataclass(frozen=True)
class Init(Stmt):
    name: str
    identity: Any
    dtype: Any = None


@dataclass(frozen=True)
class Let(Stmt):
    name: str
    value: Any
    dtype: Any = None


@dataclass(frozen=True)
class Write(Stmt):
    output: str
    index: Any
    values: Any
    value_dtype: Any = None
    atomic: bool = False
    swizzle: str = 'NONE'

    def __post_init__(self):
        object.__setattr__(self, 'values', _names(self.values))
        if isinstance(self.index, list):
            object.__setattr__(self, 'index', tuple(self.index))


@dataclass(frozen=True)
class SelectBranch(Stmt):
    value: Any
    select: Any


@dataclass(frozen=True)
class Select(Stmt):
    name: str
    branches: Any
