"""Launches the reference's own `matmul_tiled_128` kernel (built by oracle/build_ref.py) on the
current CUDA device. Test infrastructure, not product code: only the tests, the smoke check and the
baseline leg of bench.py use it, to put the reference's kernel and this build's kernels side by side
on one B200.

The kernel is loaded with the CUDA driver API (cuModuleLoadData / cuLaunchKernel through ctypes) into
the context torch has made current, and launched with the geometry of examples/tensor_matmul/meta.json:
grid 8, block 512, 73 728 bytes of dynamic shared memory, arguments in arg_order (right, left, result).
"""
from __future__ import annotations

import ctypes as ct
from pathlib import Path

CUBIN = Path(__file__).resolve().parent / '_ref' / 'matmul_tiled_128_tf32x3.cubin'
GRID, BLOCK, SMEM_BYTES = 8, 512, 73728
_MAX_DYNAMIC_SHARED = 8   # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES


def available() -> bool:
    return CUBIN.is_file()


class ReferenceMatmul:
    """matmul_tiled_128 (tf32x3, 128 x 128 x 128): result = left @ right on three device buffers of 65 536 bytes."""

    def __init__(self) -> None:
        if not available():
            raise RuntimeError(f'{CUBIN} is missing: run `python -m oracle.build_ref` where the reference tree is present')
        self._driver = ct.CDLL('libcuda.so.1')
        self._module, self._function = ct.c_void_p(), ct.c_void_p()
        image = CUBIN.read_bytes()
        self._check(self._driver.cuModuleLoadData(ct.byref(self._module), image), 'cuModuleLoadData')
        self._check(self._driver.cuModuleGetFunction(ct.byref(self._function), self._module, b'matmul_tiled_128'), 'cuModuleGetFunction')
        self._check(self._driver.cuFuncSetAttribute(self._function, _MAX_DYNAMIC_SHARED, SMEM_BYTES), 'cuFuncSetAttribute')

    def _check(self, status: int, call: str) -> None:
        if status != 0:
            name = ct.c_char_p()
            self._driver.cuGetErrorName(status, ct.byref(name))
            raise RuntimeError(f'{call} failed: {name.value.decode() if name.value else status}')

    def launch(self, right: int, left: int, result: int, stream: int) -> None:
        """Enqueues one launch; arguments are device pointers, `stream` a CUstream handle (0 = default)."""
        values = [ct.c_uint64(right), ct.c_uint64(left), ct.c_uint64(result)]
        params = (ct.c_void_p * 3)(*[ct.cast(ct.byref(v), ct.c_void_p) for v in values])
        self._check(self._driver.cuLaunchKernel(self._function, GRID, 1, 1, BLOCK, 1, 1, SMEM_BYTES, ct.c_void_p(stream), params, None),
                    'cuLaunchKernel')

    def close(self) -> None:
        if self._module:
            self._driver.cuModuleUnload(self._module)
            self._module = ct.c_void_p()
