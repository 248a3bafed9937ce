from dataclasses import dataclass
from typing import Any


def _lift(value):
    if isinstance(value, Expr):
        return value
    if type(value) is int:
        return Literal(value, dtype='int')
    if type(value) is float:
        return Literal(value, dtype='float')
    raise TypeError(f'cannot use {value!r} in an index expression')


class Expr:
    """Index expressions combine with Python's arithmetic operators; == stays structural equality."""

    def _bin(self, op, other, swap=False):
        left, right = (_lift(other), self) if swap else (self, _lift(other))
        return BinaryExpr(op=op, left=left, right=right)

    def __add__(self, other): return self._bin('+', other)
    def __radd__(self, other): return self._bin('+', other, True)
    def __sub__(self, other): return self._bin('-', other)
    def __rsub__(self, other): return self._bin('-', other, True)
    def __mul__(self, other): return self._bin('*', other)
    def __rmul__(self, other): return self._bin('*', other, True)
    def __truediv__(self, other): return self._bin('/', other)
    def __rtruediv__(self, other): return self._bin('/', other, True)
    def __floordiv__(self, other): return self._bin('//', other)
    def __rfloordiv__(self, other): return self._bin('//', other, True)
    def __mod__(self, other): return self._bin('%', other)
    def __rmod__(self, other): return self._bin('%', other, True)
    def __and__(self, other): return self._bin('&', other)
    def __or__(self, other): return self._bin('|', other)
    def __xor__(self, other): return self._bin('^', other)
    def __lshift__(self, other): return self._bin('<<', other)
    def __rshift__(self, other): return self._bin('>>', other)


@dataclass(frozen=True, eq=True)
class Literal(Expr):
    value: Any
    dtype: str = 'int'


@dataclass(frozen=True, eq=True)
class Var(Expr):
    name: str


@dataclass(frozen=True, eq=True)
class Builtin(Expr):
    name: str


@dataclass(frozen=True, eq=True)
class BinaryExpr(Expr):
    op: str
    left: Any
    right: Any


@dataclass(frozen=True, eq=True)
class TernaryExpr(Expr):
    cond: Any
    if_true: Any
    if_false: Any


@dataclass(frozen=True, eq=True)
class CastExpr(Expr):
    expr: Any
    dtype: Any


@dataclass(frozen=True, eq=True)
class FlatIndex(Expr):
    buffer: Any
    index: Any


@dataclass(frozen=True, eq=True)
class FuncCallExpr(Expr):
    name: str
    args: Any = ()
