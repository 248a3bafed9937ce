"""Compile options with the fields and validation of the reference's Options (compiler/options.py:5-28).

Only `contraction_precision` selects between native kernels; `approximate_math` is honoured (the
kernels use the approximate exp/reciprocal forms the reference emits when it is set, which is the
default) and the remaining switches tune code generation in the reference and are accepted,
validated and recorded here so that callers' option objects keep working unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Options:
    approximate_math: bool = True
    contraction_precision: str = 'bf16x3'
    recurrence_staging: bool = True
    reduction_sharing: bool = True
    vector_width: int = 4
    unroll: int = 0
    tree_specialization: bool = True
    coalesced_reductions: bool = True
    warp_willreturn: bool = True
    elementwise_vectorize: bool = True
    register_forwarding: bool = True
    tail_linearize: bool = True

    def __post_init__(self) -> None:
        booleans = ('approximate_math', 'recurrence_staging', 'reduction_sharing', 'tree_specialization',
                    'coalesced_reductions', 'warp_willreturn', 'elementwise_vectorize', 'register_forwarding',
                    'tail_linearize')
        for name in booleans:
            if type(getattr(self, name)) is not bool:
                raise ValueError(f'{name} must be a boolean')
        if type(self.contraction_precision) is not str or self.contraction_precision not in ('f32', 'tf32x3', 'bf16x3'):
            raise ValueError(f'unsupported contraction precision {self.contraction_precision!r}')
        if type(self.vector_width) is not int or self.vector_width not in (1, 2, 4, 8, 16):
            raise ValueError('vector_width must be 1, 2, 4, 8, or 16')
        if type(self.unroll) is not int or not 0 <= self.unroll < 2**31:
            raise ValueError('unroll must be a nonnegative signed 32-bit integer')
