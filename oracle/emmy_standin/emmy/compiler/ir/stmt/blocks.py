from dataclasses import dataclass
from typing import Any

from emmy.compiler.ir.stmt.base import Stmt
from emmy.compiler.ir.stmt.body import Body


def _body(value):
    return value if isinstance(value, Body) else Body(value)


@dataclass(frozen=True)
class Cond(Stmt):
    cond: Any
    body: Any = ()
    else_body: Any = ()

    def __post_init__(self):
        object.__setattr__(self, 'body', _body(self.body))
        object.__setattr__(self, 'else_body', _body(self.else_body))


# A loop re-initialises the accumulators in its body to their operator's identity on entry unless seed is False
# (the reference's example generators build their reduction loops without naming the flag and rely on that).
@dataclass(frozen=True)
class Loop(Stmt):
    axis: Any
    body: Any = ()
    unroll: bool = False
    seed: bool = True

    def __post_init__(self):
        object.__setattr__(self, 'body', _body(self.body))


@dataclass(frozen=True)
class StridedLoop(Stmt):
    axis: Any
    start: Any
    step: Any
    body: Any = ()
    unroll: bool = False
    end: Any = None
    seed: bool = True

    def __post_init__(self):
        object.__setattr__(self, 'body', _body(self.body))
