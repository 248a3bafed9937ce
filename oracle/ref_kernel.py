"""Runs the reference's own kernels (built by oracle/build_ref.py) on the current CUDA device.

Test infrastructure, not product code: only the tests, the smoke check and the baseline legs of bench.py use it,
to put the reference's kernels and this build's kernels side by side on one B200 with the same inputs.

A kernel is loaded with the CUDA driver API (cuModuleLoadData / cuLaunchKernel through ctypes) into the context
torch has made current and launched exactly as the reference's runner launches it: the grid, block and dynamic
shared memory of its meta.json launch, one 64-bit device pointer per buffer in `arg_order`
(benchmark.py:205-243 of the reference). `ReferenceKernel(name)` takes any kernel of oracle/_ref/manifest.json;
`ReferenceMatmul` is the kernel assembled from the PTX file the reference committed itself.
"""
from __future__ import annotations

import ctypes as ct
import json
from pathlib import Path

ROOT = Path(__file__).resolve().parent / '_ref'
CUBIN = ROOT / 'matmul_tiled_128_tf32x3.cubin'
MANIFEST = ROOT / 'manifest.json'
GRID, BLOCK, SMEM_BYTES = 8, 512, 73728
_MAX_DYNAMIC_SHARED = 8   # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES


def available() -> bool:
    return CUBIN.is_file()


def manifest() -> dict:
    """name -> launch record of every compiled reference kernel that was built ({} when none was)."""
    if not MANIFEST.is_file():
        return {}
    kernels = json.loads(MANIFEST.read_text()).get('kernels', {})
    return {name: record for name, record in kernels.items() if (ROOT / record['cubin']).is_file()}


class _Module:
    def __init__(self, cubin: Path, entry: str, smem_bytes: int) -> None:
        if not cubin.is_file():
            raise RuntimeError(f'{cubin} is missing: run `python -m oracle.build_ref` where the reference checkout is present')
        self._driver = ct.CDLL('libcuda.so.1')
        self._module, self._function = ct.c_void_p(), ct.c_void_p()
        self._check(self._driver.cuModuleLoadData(ct.byref(self._module), cubin.read_bytes()), 'cuModuleLoadData')
        self._check(self._driver.cuModuleGetFunction(ct.byref(self._function), self._module, entry.encode()), 'cuModuleGetFunction')
        if smem_bytes > 48 * 1024:
            self._check(self._driver.cuFuncSetAttribute(self._function, _MAX_DYNAMIC_SHARED, smem_bytes), 'cuFuncSetAttribute')

    def _check(self, status: int, call: str) -> None:
        if status != 0:
            name = ct.c_char_p()
            self._driver.cuGetErrorName(status, ct.byref(name))
            raise RuntimeError(f'{call} failed: {name.value.decode() if name.value else status}')

    def _launch(self, grid, block, smem_bytes: int, pointers: list[int], stream: int) -> None:
        values = [ct.c_uint64(pointer) for pointer in pointers]
        params = (ct.c_void_p * len(values))(*[ct.cast(ct.byref(v), ct.c_void_p) for v in values])
        self._check(self._driver.cuLaunchKernel(self._function, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem_bytes,
                                                ct.c_void_p(stream), params, None), 'cuLaunchKernel')

    def close(self) -> None:
        if self._module:
            self._driver.cuModuleUnload(self._module)
            self._module = ct.c_void_p()


class ReferenceKernel(_Module):
    """One kernel of the manifest. `record` is its launch: entry, grid, block, smem_bytes, arg_order, args."""

    def __init__(self, name: str) -> None:
        records = manifest()
        if name not in records:
            raise RuntimeError(f'no reference kernel {name!r} in {MANIFEST}')
        self.name, self.record = name, records[name]
        super().__init__(ROOT / self.record['cubin'], self.record['entry'], self.record['smem_bytes'])

    def launch(self, pointers: dict[str, int], stream: int) -> None:
        """Enqueues one launch. `pointers`: device pointer of every buffer by name; `stream`: a CUstream handle.
        Buffers named in `zero_outputs` must be cleared by the caller before each launch, as the reference's runner does."""
        record = self.record
        self._launch(record['grid'], record['block'], record['smem_bytes'], [pointers[name] for name in record['arg_order']], stream)

    def __enter__(self) -> 'ReferenceKernel':
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class ReferenceMatmul(_Module):
    """matmul_tiled_128 (tf32x3, 128 x 128 x 128) from the PTX the reference committed: result = left @ right on three
    device buffers of 65 536 bytes, launched with the geometry of examples/tensor_matmul/meta.json (grid 8, block 512,
    73 728 bytes of dynamic shared memory, arguments right, left, result)."""

    def __init__(self) -> None:
        super().__init__(CUBIN, 'matmul_tiled_128', SMEM_BYTES)

    def launch(self, right: int, left: int, result: int, stream: int) -> None:
        self._launch((GRID, 1, 1), (BLOCK, 1, 1), SMEM_BYTES, [right, left, result], stream)
