"""The allocation-free GEMM entry point against the ordinary one, through the C ABI.

dtn_gemm_x3_static serves callers that cannot allocate device memory (everything on the GPU already
belongs to their own pool, or they cannot tolerate the synchronisation an allocation implies): its
operand planes live in a fixed 32 MiB array inside the library. It must produce exactly what
dtn_gemm_x3 produces with a caller-owned workspace. The file sorts last so that a run that stops at
the first failure has already exercised every other test; it passes alone in a fresh process too.
"""
import ctypes as ct

import numpy as np
import pytest

from deuteron_b200 import native

pytestmark = pytest.mark.gpu

STATIC_LIMIT = 32 << 20


def _uniform(cuda, seed, shape):
    generator = cuda.Generator(device='cuda:0').manual_seed(seed)
    return cuda.rand(shape, device='cuda:0', generator=generator) * 2 - 1


def _with_workspace(cuda, mode, a, b):
    m, k = a.shape
    n = b.shape[1]
    need = ct.c_size_t(0)
    native.call('dtn_gemm_workspace_bytes', mode, m, n, k, ct.byref(need))
    scratch = cuda.empty(need.value + 1024, dtype=cuda.uint8, device='cuda:0')
    aligned = (scratch.data_ptr() + 1023) // 1024 * 1024
    out = cuda.empty((m, n), device='cuda:0')
    native.call('dtn_gemm_x3', mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, k, n, n, aligned, need.value,
                cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    return out


def _static(cuda, mode, a, b, out=None):
    m, k = a.shape
    n = b.shape[1]
    out = cuda.empty((m, n), device='cuda:0') if out is None else out
    native.call('dtn_gemm_x3_static', mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, k, n, n,
                cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    return out


def _static_status(cuda):
    """The status word the static-scratch kernels report into (not the one dtn_device_status reads)."""
    word = ct.c_int(-1)
    native.call('dtn_gemm_x3_static_status', ct.byref(word), cuda.cuda.current_stream().cuda_stream)
    return word.value


@pytest.mark.parametrize('mode', [native.GEMM_MODES['bf16x3'], native.GEMM_MODES['tf32x3']])
def test_static_scratch_gemm_equals_the_workspace_gemm_twice_in_a_row(cuda, mode):
    # two different problems back to back: the second call reuses the array the first one filled
    first = (_uniform(cuda, 7, (512, 384)), _uniform(cuda, 11, (384, 640)))
    second = (_uniform(cuda, 3, (200, 1000)), _uniform(cuda, 5, (1000, 136)))
    # The ordinary entry point picks its single-kernel path for products this small; pin it to the split + tensor-core
    # kernels (128 x 128 tiles), which is what the static-scratch entry point always runs.
    native.call('dtn_gemm_set_variant', 1)
    try:
        for a, b in (first, second, first):
            expected = _with_workspace(cuda, mode, a, b)
            produced = _static(cuda, mode, a, b)
            # same kernels, same operand planes, same order of accumulation: the results are identical
            assert bool(cuda.equal(produced, expected))
            exact = a.double() @ b.double()
            assert float(((produced.double() - exact).abs().max() / exact.abs().max()).item()) < 2e-5
    finally:
        native.call('dtn_gemm_set_variant', 0)
    assert _static_status(cuda) == 0


def test_static_scratch_gemm_at_its_size_limit_and_beyond(cuda):
    mode = native.GEMM_MODES['bf16x3']
    need = ct.c_size_t(0)
    native.call('dtn_gemm_workspace_bytes', mode, 2048, 2048, 2048, ct.byref(need))
    # the operand planes of 2048^3 fill the built-in array exactly; a caller-owned workspace is asked for a little more
    # (the counters of the kernel that splits A beside its products, which this entry point does not use)
    assert STATIC_LIMIT <= need.value <= STATIC_LIMIT + 4096
    a, b = _uniform(cuda, 7, (2048, 2048)), _uniform(cuda, 11, (2048, 2048))
    assert bool(cuda.equal(_static(cuda, mode, a, b), _with_workspace(cuda, mode, a, b)))
    too_big_a, too_big_b = _uniform(cuda, 1, (2048, 2112)), _uniform(cuda, 2, (2112, 2048))
    with pytest.raises(ValueError, match='built-in array holds'):
        _static(cuda, mode, too_big_a, too_big_b)
    with pytest.raises(ValueError, match='mode must be'):
        _static(cuda, native.GEMM_MODES['f32'], a, b)
    # an empty product is a no-op, as for the ordinary entry point
    empty = cuda.empty((0, 2048), device='cuda:0')
    assert _static(cuda, mode, empty, b).shape == (0, 2048)
    # an empty sum (K = 0) zero-fills C, as the ordinary entry point does
    filled = cuda.full((64, 96), 3.0, device='cuda:0')
    _static(cuda, mode, cuda.empty((64, 0), device='cuda:0'), cuda.empty((0, 96), device='cuda:0'), out=filled)
    assert float(filled.abs().max().item()) == 0.0
    assert _static_status(cuda) == 0


def test_static_scratch_gemm_treats_the_scratch_free_variants_as_automatic(cuda):
    # variants 4 and 6 name kernels that use no scratch; the static entry point runs its own path under them and
    # agrees with the ordinary entry point to the mode's tolerance
    mode = native.GEMM_MODES['bf16x3']
    a, b = _uniform(cuda, 7, (640, 512)), _uniform(cuda, 11, (512, 768))
    exact = a.double() @ b.double()
    reference = _static(cuda, mode, a, b)
    for variant in (4, 6):
        native.call('dtn_gemm_set_variant', variant)
        try:
            produced = _static(cuda, mode, a, b)
        finally:
            native.call('dtn_gemm_set_variant', 0)
        assert bool(cuda.equal(produced, reference))
        assert float(((produced.double() - exact).abs().max() / exact.abs().max()).item()) < 2e-5
    assert _static_status(cuda) == 0
