from dataclasses import dataclass
from typing import Any

import numpy as _np


@dataclass(frozen=True)
class DataType:
    name: str
    np: Any
    nbytes: int


@dataclass(frozen=True)
class StructuredType:
    name: str = ''
    fields: Any = ()


F16 = DataType(name='f16', np=_np.dtype('float16'), nbytes=2)
F32 = DataType(name='f32', np=_np.dtype('float32'), nbytes=4)
F64 = DataType(name='f64', np=_np.dtype('float64'), nbytes=8)
I32 = DataType(name='i32', np=_np.dtype('int32'), nbytes=4)
