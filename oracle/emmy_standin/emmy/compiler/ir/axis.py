from dataclasses import dataclass
from typing import Any

from emmy.compiler.dim import Dim  # noqa: F401  (re-exported)


@dataclass(frozen=True)
class Window:
    parent: Any
    base: Any = None
    bound: Any = None
    partition: bool = False


@dataclass(frozen=True)
class Axis:
    name: str
    extent: Any
    window: Any = None
