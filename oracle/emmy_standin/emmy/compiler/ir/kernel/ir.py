from dataclasses import dataclass
from typing import Any

from emmy.compiler.ir.stmt.base import Stmt
from emmy.compiler.ir.stmt.body import Body


def _body(value):
    return value if isinstance(value, Body) else Body(value)


@dataclass(frozen=True)
class KernelOp:
    body: Any
    name: str
    zero_delegated: Any = ()
    serial: Any = ()

    def __post_init__(self):
        object.__setattr__(self, 'body', _body(self.body))


@dataclass(frozen=True)
class Tile(Stmt):
    axes: Any
    body: Any = ()
    block_threads: Any = None
    aux_threads: int = 0
    raster_axes: Any = None
    raster_group: Any = None
    raster_orient: str = 'm'

    def __post_init__(self):
        object.__setattr__(self, 'axes', tuple(self.axes))
        object.__setattr__(self, 'body', _body(self.body))


@dataclass(frozen=True)
class Smem(Stmt):
    name: str
    extents: Any
    dtype: Any = 'float'
    align: int = 16


@dataclass(frozen=True)
class CpAsyncCopy(Stmt):
    smem: str
    smem_index: Any
    src: str
    src_index: Any
    nbytes: int = 16
    swizzle: str = 'NONE'
    lane_index: Any = None
    lane_rows: Any = None


@dataclass(frozen=True)
class CpAsyncCommit(Stmt):
    pass


@dataclass(frozen=True)
class CpAsyncWait(Stmt):
    group: int = 0


@dataclass(frozen=True)
class Sync(Stmt):
    barrier_id: int = 0
    count: Any = None
    warp: bool = False


@dataclass(frozen=True)
class WarpShuffle(Stmt):
    state: Any
    state_b: Any
    combine_states: Any
    length: int = 32
    dtype: Any = None


@dataclass(frozen=True)
class TreeHalve(Stmt):
    bufs: Any
    state: Any
    state_b: Any
    combine_states: Any
    length: int = 0
    tid_var: Any = None
    inner: Any = None
    barrier_id: int = 0
    barrier_count: Any = None
    dtype: Any = None
