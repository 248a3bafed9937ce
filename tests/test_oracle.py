"""The oracle against the reference's own fixtures and published GPU outputs (CPU only)."""
import hashlib
import math

import numpy as np

from oracle import reference_math as R


def sha(array):
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def test_gemm_f64_matches_reference_expected(golden):
    # examples/tensor_matmul/expected.npz, seeds 7 (left) and 11 (right): tests/test_tensor_copy.py:40-57
    expected = np.load(golden / 'tensor_matmul_expected.npz')['result']
    left, right = R.seeded_normal(7, (128, 128)), R.seeded_normal(11, (128, 128))
    np.testing.assert_allclose(R.gemm_f64(left, right), expected, rtol=1e-12, atol=1e-12)


def test_vector_add_matches_reference_expected(golden, published):
    expected = np.load(golden / 'vector_add_expected.npz')['sum']
    result = R.vector_add(R.seeded_normal(21, (1030,)), R.seeded_normal(22, (1030,)))
    np.testing.assert_array_equal(result, expected)
    assert sha(result) == published['results']['vector_add']['output_sha256']['sum']


def test_f16_conversions_reproduce_published_output_hashes(published):
    # examples/f16_storage.py: 512 values, seed 7; hashes are of the reference's GPU outputs
    half = R.seeded_normal(7, (512,), np.float16)
    single = R.seeded_normal(7, (512,), np.float32)
    results = published['results']
    assert sha(half) == results['copy']['output_sha256']['result']
    assert sha(R.f16_widen_bits(half.view(np.uint16))) == results['widen']['output_sha256']['result']
    assert sha(R.f16_narrow_bits(single)) == results['narrow']['output_sha256']['result']


def test_f16_fused_expressions_reproduce_published_output_hashes(published):
    # examples/f16_storage.py affine (scale 1.5, bias -0.25) and cancellation (y from seed 8)
    x, y = R.seeded_normal(7, (512,), np.float16), R.seeded_normal(8, (512,), np.float16)
    assert sha(R.f16_affine(x)) == published['results']['affine']['output_sha256']['result']
    assert sha(R.f16_cancellation(x, y)) == published['results']['cancellation']['output_sha256']['result']
    # tests/test_f16_storage.py:150-155: the FP32 intermediate keeps the small addend
    big = np.resize(np.array([2048., 4096., 65504., -2048.], dtype=np.float16), 512)
    np.testing.assert_array_equal(R.f16_cancellation(big, np.ones(512, np.float16)), np.ones(512, np.float16))


def test_f16_narrow_bits_equal_numpy_on_every_rounding_boundary():
    points = R.f16_boundary_points()
    assert points.size == 190468
    with np.errstate(over='ignore', invalid='ignore'):
        expected = points.astype(np.float16).view(np.uint16)
    actual = R.f16_narrow_bits(points)
    finite = ~np.isnan(points)
    np.testing.assert_array_equal(actual[finite], expected[finite])
    assert np.all((actual[~finite] & 0x7C00) == 0x7C00) and np.all(actual[~finite] & 0x3FF)


def test_f16_widen_bits_equal_numpy_on_every_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    expected = bits.view(np.float16).astype(np.float32)
    actual = R.f16_widen_bits(bits)
    finite = ~np.isnan(expected)
    np.testing.assert_array_equal(actual[finite].view(np.uint32), expected[finite].view(np.uint32))
    np.testing.assert_array_equal(np.isnan(actual), np.isnan(expected))


def test_f32_contraction_oracle_is_bit_identical_to_the_reference_gpu_output(published):
    # contraction_precision='f32' on the 128^3 example: sequential FP32 FMA over k
    left, right = R.seeded_normal(7, (128, 128)), R.seeded_normal(11, (128, 128))
    result = R.gemm_f32_fma(left, right)
    record = published['results']['tensor_f32']
    assert sha(result) == record['output_sha256']['result']
    error = float(np.max(np.abs(result.astype(np.float64) - R.gemm_f64(left, right))))
    assert error == record['max_absolute_errors']['result']


def test_compensated_contraction_models_sit_at_the_published_error_level(published):
    left, right = R.seeded_normal(7, (128, 128)), R.seeded_normal(11, (128, 128))
    exact = R.gemm_f64(left, right)
    for mode, name in (('bf16x3', 'tensor_bf16x3'), ('tf32x3', 'tensor_tf32x3')):
        reference_error = published['results'][name]['max_absolute_errors']['result']
        floor = float(np.max(np.abs(R.gemm_x3_exact_products(left, right, mode) - exact)))
        model = float(np.max(np.abs(R.gemm_x3_f32_accumulate(left, right, mode) - exact)))
        # an ideal accumulator cannot be worse than the reference's measured run; the FP32 model is within 2x
        assert floor <= reference_error * 1.01
        assert model <= 2 * reference_error


def test_bf16_split_is_rne_and_residual_is_small():
    x = R.seeded_normal(3, (4096,))
    hi, lo = R.bf16_split(x)
    assert np.all((hi.view(np.uint32) & 0xFFFF) == 0) and np.all((lo.view(np.uint32) & 0xFFFF) == 0)
    # ties to even: 1 + 2^-8 is halfway between bf16 neighbours 1 and 1 + 2^-7
    assert R.bf16_round(np.array([1 + 2.0 ** -8], np.float32))[0] == 1.0
    assert R.bf16_round(np.array([1 + 3 * 2.0 ** -8], np.float32))[0] == np.float32(1 + 2.0 ** -6)
    residual = np.abs(x.astype(np.float64) - hi.astype(np.float64) - lo.astype(np.float64))
    assert np.all(residual <= np.abs(x) * 2.0 ** -16)


def test_tf32_round_is_ties_away():
    # 1 + 2^-11 is halfway between tf32 neighbours 1 and 1 + 2^-10: rna rounds away from zero
    assert R.tf32_round_away(np.array([1 + 2.0 ** -11], np.float32))[0] == np.float32(1 + 2.0 ** -10)
    assert R.tf32_round_away(np.array([-(1 + 2.0 ** -11)], np.float32))[0] == np.float32(-(1 + 2.0 ** -10))
    x = R.seeded_normal(5, (4096,))
    hi, lo = R.tf32_split(x)
    assert np.all((hi.view(np.uint32) & 0x1FFF) == 0) and np.all((lo.view(np.uint32) & 0x1FFF) == 0)


def test_attention_oracles_agree_and_match_published_error_level(published):
    # examples/attention.py defaults: rows 3, keys 64, depth 32, seeds 7, 8, 9
    q, kt, v = R.seeded_normal(7, (3, 32)), R.seeded_normal(8, (32, 64)), R.seeded_normal(9, (64, 32))
    scale = float(np.float32(1 / math.sqrt(32)))
    exact = R.attention_f64(q, kt, v)
    model = R.attention_recurrence_f32(q, kt, v, scale)
    reference_error = published['results']['attention']['max_absolute_errors']['out']
    assert np.max(np.abs(model - exact)) <= 2 * reference_error
    # softmax rows sum to one: attention of a constant value matrix returns the constant
    ones = R.attention_f64(q, kt, np.ones_like(v))
    np.testing.assert_allclose(ones, 1.0, rtol=1e-12)


def test_gqa_oracle_maps_query_heads_to_kv_heads():
    q = R.seeded_normal(1, (1, 4, 16, 8), np.float16)
    k = R.seeded_normal(2, (1, 2, 16, 8), np.float16)
    v = R.seeded_normal(3, (1, 2, 16, 8), np.float16)
    out = R.gqa_attention_f64(q, k, v, 0.25)
    for head in range(4):
        expected = R.attention_f64(q[0, head], k[0, head // 2].T, v[0, head // 2], 0.25)
        np.testing.assert_allclose(out[0, head], expected, rtol=1e-13)
    sampled = R.gqa_attention_f64(q, k, v, 0.25, heads=[(0, 3)], rows=[5, 9])
    np.testing.assert_allclose(sampled[0, 3, [5, 9]], out[0, 3, [5, 9]], rtol=1e-13)
    assert np.isnan(sampled[0, 0]).all()


def test_row_reductions():
    x = R.seeded_normal(7, (9, 1000))
    x[2, 5] = np.nan
    assert R.row_max(x)[2] == np.nanmax(x[2])  # NaN-suppressing maxnum
    assert R.row_max(np.full((1, 4), np.nan, np.float32))[0] == -np.inf
    assert R.row_max(np.zeros((2, 0), np.float32)).tolist() == [-np.inf, -np.inf]
    np.testing.assert_allclose(R.row_sum_f64(x[:2]), x[:2].astype(np.float64).sum(axis=1))


def test_row_kernel_oracles():
    x = R.seeded_normal(7, (5, 300)) * np.float32(4.0)
    soft = R.row_softmax_f64(x)
    assert np.allclose(soft.sum(axis=1), 1.0, rtol=0, atol=1e-14) and (soft > 0).all()
    assert np.allclose(R.row_softmax_f64(x + np.float32(2.0)), soft, rtol=1e-5)        # shift invariance (inputs re-rounded)
    assert np.allclose((R.l2_norm_f64(x) ** 2).sum(axis=1), 1.0, rtol=0, atol=1e-13)
    unit = R.rms_norm_f64(x, np.ones(300, dtype=np.float32), 300.0, 0.0)
    assert np.allclose((unit ** 2).mean(axis=1), 1.0, rtol=0, atol=1e-13)
    w = R.seeded_normal(8, (300,))
    assert np.allclose(R.rms_norm_f64(x, w, 300.0, 0.0), unit * w.astype(np.float64)[None, :], rtol=1e-15)
    assert np.allclose(R.row_mean_f64(x), x.astype(np.float64).mean(axis=1), rtol=1e-15)
    assert np.allclose(R.row_mean_f64(x, 150.0), 2.0 * R.row_mean_f64(x), rtol=1e-15)
