"""The mixed sweep of the largest configurations, on one GPU: GEMMs with M = N = K in
{1024, 2048, 4096, 16384} plus the skinny 16 x 8192 x 8192, attention with 64 query / 8 kv heads,
batch 8, head_dim 128 at sequence lengths {512, 2048, 8192, 16384}; N(0,1) inputs from fixed seeds.

At these sizes a full float64 product on the CPU takes minutes to hours, so the float64 oracle is
evaluated on seeded samples of output rows (computed in float64 on the GPU's own copy of the inputs)
and the remaining checks are size-independent properties.
"""
import math

import numpy as np
import pytest

from deuteron_b200 import ops
from oracle import reference_math as R

pytestmark = pytest.mark.gpu


def normal(cuda, seed, shape, dtype=None, scale=1.0):
    generator = cuda.Generator(device='cuda:0').manual_seed(seed)
    values = cuda.randn(shape, device='cuda:0', generator=generator) * scale
    return values if dtype is None else values.to(dtype)


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
@pytest.mark.parametrize('m,n,k', [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (16, 8192, 8192), (16384, 16384, 16384)])
def test_gemm_sweep(cuda, mode, m, n, k):
    a, b = normal(cuda, 7, (m, k)), normal(cuda, 11, (k, n))
    c = ops.gemm(a, b, mode)
    ops.check_device_status()
    rows = cuda.arange(0, m, max(1, m // 16), device='cuda:0')[:16]
    cols = slice(0, min(n, 4096))
    exact = a[rows].double() @ b[:, cols].double()
    error = float(((c[rows][:, cols].double() - exact).abs().max() / exact.abs().max()).item())
    # error floor of the three-product scheme (2^-16 / 2^-21 per term, sqrt(k) growth) plus one truncated unit per
    # accumulator update (3 * k / k-step updates), the same count the reference's mma.sync loop performs
    steps = 3 * k / (16 if mode == 'bf16x3' else 8)
    assert error <= 2e-5 + steps * 2.0 ** -24, (m, n, k, error)
    # transposition identity on a sampled block: (A B)^T = B^T A^T up to the same bound
    if m <= 4096:
        ct = ops.gemm(b.t().contiguous(), a.t().contiguous(), mode)
        assert float((ct.t() - c).abs().max() / c.abs().max()) <= 2 * (2e-5 + steps * 2.0 ** -24)


@pytest.mark.parametrize('s', [512, 2048, 8192, 16384])
def test_attention_sweep(cuda, s):
    batch, hq, hkv, d = 8, 64, 8, 128
    scale = float(np.float32(1 / math.sqrt(d)))
    q = normal(cuda, 7, (batch, hq, s, d), cuda.float16)
    k = normal(cuda, 8, (batch, hkv, s, d), cuda.float16)
    v = normal(cuda, 9, (batch, hkv, s, d), cuda.float16)
    out = ops.gqa_attention(q, k, v, scale)
    ops.check_device_status()
    rows = [0, 1, s // 3, s - 1]
    for b, h in ((0, 0), (3, 29), (7, 63)):
        exact = R.attention_f64(q[b, h, rows].cpu().numpy(), k[b, h // 8].cpu().numpy().astype(np.float64).T,
                                v[b, h // 8].cpu().numpy(), scale)
        produced = out[b, h, rows].cpu().numpy()
        np.testing.assert_allclose(produced, exact, rtol=1e-3, atol=1e-4)
        # N(0,1) scores are peaked: a few keys carry each row, so the result is not a cancelling mean and the
        # error is compared with max|out|; allowance as in the tensor-core bound of the parity tests
        assert R.max_relative_error(produced, exact) <= 3e-6 + (2 * s / 16) * 2.0 ** -24
    del out
    ones = ops.gqa_attention(q[:1], k[:1], cuda.ones_like(v[:1]), scale)
    assert float((ones - 1).abs().max()) <= 3e-6 + (2 * s / 16) * 2.0 ** -24
