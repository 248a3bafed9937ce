"""CPU oracle for the hot path: a NumPy restatement of what the reference's emitted kernels compute.

THIS IS TEST INFRASTRUCTURE. Only the tests, the smoke check and the CPU-baseline leg of the
benchmark may import it; the product (the deuteron_b200 package) never does.

Every function names the reference source (stashuk-olek/deuteron, paths relative to that project)
it restates. The oracle is pinned against the reference's own fixtures: the float64 matrix product
of examples/tensor_matmul/expected.npz, the exact sum of examples/vector_add/expected.npz, the
float64 softmax of examples/attention.py:71-75 and the NumPy conversions that
tests/test_f16_storage.py:119-148 compare the f16 kernels with (see tests/test_oracle.py and
tests/golden/).
"""
from __future__ import annotations

import math

import numpy as np

# --------------------------------------------------------------------------------------------
# Seeded inputs
# --------------------------------------------------------------------------------------------


def seeded_normal(seed: int, shape, dtype=np.float32, scale: float = 1.0) -> np.ndarray:
    """Input convention of benchmark.py:70 (argument_array): default_rng(seed).standard_normal -> dtype."""
    values = np.random.default_rng(seed).standard_normal(shape)
    if scale != 1.0:
        values = values * scale
    return values.astype(dtype)


def seeded_uniform(seed: int, shape) -> np.ndarray:
    """FP32 uniform[-1, 1) inputs of the large-GEMM configurations."""
    return (np.random.default_rng(seed).random(shape, dtype=np.float32) * np.float32(2.0) - np.float32(1.0)).astype(np.float32)


# --------------------------------------------------------------------------------------------
# Operand splits (compiler/codegen/tensor.py:50-64, 104-119)
# --------------------------------------------------------------------------------------------


def bf16_round(x: np.ndarray) -> np.ndarray:
    """cvt.rn.bf16.f32: round an FP32 array to bfloat16 (nearest even), returned as FP32 values.

    TensorEmitter.bf16 (compiler/codegen/tensor.py:55-64) packs two such conversions per register.
    """
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    rounded = np.where(nan, 0x7FFF0000, rounded).astype(np.uint32)
    return rounded.view(np.float32).reshape(np.shape(x))


def bf16_split(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """hi = bf16_rn(v); lo = bf16_rn(v - hi) with the subtraction in FP32.

    packed_store (compiler/codegen/tensor.py:104-119): `restored` is the high part shifted back into
    an FP32 register and the residual is converted by the same cvt.rn.bf16x2.
    """
    x = np.asarray(x, dtype=np.float32)
    hi = bf16_round(x)
    with np.errstate(invalid='ignore'):
        lo = bf16_round((x - hi).astype(np.float32))
    return hi, lo


def tf32_round_away(x: np.ndarray) -> np.ndarray:
    """cvt.rna.tf32.f32 (compiler/codegen/tensor.py:50-53): nearest, ties away from zero, 10-bit mantissa."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    special = (bits & 0x7F800000) == 0x7F800000
    rounded = (bits + 0x1000) & 0xFFFFE000
    rounded = np.where(special, bits, rounded).astype(np.uint32)
    return rounded.view(np.float32).reshape(np.shape(x))


def tf32_split(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """hi = tf32_rna(v); lo = tf32_rna(v - hi) (compiler/codegen/tensor.py:234-243)."""
    x = np.asarray(x, dtype=np.float32)
    hi = tf32_round_away(x)
    with np.errstate(invalid='ignore'):
        lo = tf32_round_away((x - hi).astype(np.float32))
    return hi, lo


# --------------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------------


def gemm_f64(left: np.ndarray, right: np.ndarray) -> np.ndarray:
    """float64 product of the FP32 inputs: the reference's expected.npz (tests/test_tensor_copy.py:40-57)."""
    return np.asarray(left, dtype=np.float64) @ np.asarray(right, dtype=np.float64)


def gemm_x3_exact_products(left: np.ndarray, right: np.ndarray, mode: str) -> np.ndarray:
    """The three products the compensated modes keep, summed without accumulation error.

    _emit_packed / _emit (compiler/codegen/tensor.py:166-190, 234-243) accumulate lo_A*hi_B,
    hi_A*lo_B and hi_A*hi_B and drop lo_A*lo_B. Every product of two bf16 (or tf32) values is exact
    in float64, so this is the result of that arithmetic with an ideal accumulator: the error floor
    that any FP32-accumulating implementation of the scheme (the reference's or ours) sits on.
    """
    split = {'bf16x3': bf16_split, 'tf32x3': tf32_split}[mode]
    a_hi, a_lo = (p.astype(np.float64) for p in split(left))
    b_hi, b_lo = (p.astype(np.float64) for p in split(right))
    return a_lo @ b_hi + a_hi @ b_lo + a_hi @ b_hi


def gemm_x3_f32_accumulate(left: np.ndarray, right: np.ndarray, mode: str, k_step: int | None = None) -> np.ndarray:
    """Same three products accumulated in FP32 per k-step in the reference's order (small cases only).

    Order per k-step: lo*hi, hi*lo, hi*hi (compiler/codegen/tensor.py:169-171, 186-188); k-step 16
    for bf16 (m16n8k16) and 8 for tf32 (m16n8k8). Within one k-step the partial dot product is formed
    in float64 and rounded once to FP32, a model of the tensor core's wide internal adder.
    """
    split = {'bf16x3': bf16_split, 'tf32x3': tf32_split}[mode]
    step = k_step or {'bf16x3': 16, 'tf32x3': 8}[mode]
    a_hi, a_lo = (p.astype(np.float64) for p in split(left))
    b_hi, b_lo = (p.astype(np.float64) for p in split(right))
    acc = np.zeros((left.shape[0], right.shape[1]), dtype=np.float32)
    for k in range(0, left.shape[1], step):
        sl = slice(k, k + step)
        for a, b in ((a_lo, b_hi), (a_hi, b_lo), (a_hi, b_hi)):
            acc = (acc.astype(np.float64) + a[:, sl] @ b[sl, :]).astype(np.float32)
    return acc


def gemm_f32_fma(left: np.ndarray, right: np.ndarray) -> np.ndarray:
    """contraction_precision='f32': sequential FP32 FMA over k (generic lowering, compiler/codegen/lower.py:600-653).

    Small cases only (a Python loop over k). Each step is fma(a, b, acc) with one rounding, modelled in float64.
    """
    left = np.asarray(left, dtype=np.float32)
    right = np.asarray(right, dtype=np.float32)
    acc = np.zeros((left.shape[0], right.shape[1]), dtype=np.float32)
    for k in range(left.shape[1]):
        acc = (acc.astype(np.float64) + left[:, k:k + 1].astype(np.float64) * right[k:k + 1, :].astype(np.float64)).astype(np.float32)
    return acc


def max_relative_error(actual: np.ndarray, exact: np.ndarray) -> float:
    """max|x - ref| / max|ref| against the float64 result: the error metric of the parity bar."""
    exact = np.asarray(exact, dtype=np.float64)
    denominator = float(np.max(np.abs(exact))) if exact.size else 0.0
    if denominator == 0.0:
        return float(np.max(np.abs(np.asarray(actual, dtype=np.float64) - exact))) if exact.size else 0.0
    return float(np.max(np.abs(np.asarray(actual, dtype=np.float64) - exact))) / denominator


# --------------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------------


def attention_f64(q: np.ndarray, kt: np.ndarray, v: np.ndarray, scale: float | None = None) -> np.ndarray:
    """examples/attention.py:71-75: float64 softmax(q @ kt * float32(1/sqrt(depth))) @ v on the stored inputs."""
    q64, kt64, v64 = (np.asarray(a).astype(np.float64) for a in (q, kt, v))
    if scale is None:
        scale = np.float32(1 / math.sqrt(q64.shape[1]))
    scores = q64 @ kt64 * np.float64(scale)
    weights = np.exp(scores - scores.max(axis=1, keepdims=True))
    return (weights / weights.sum(axis=1, keepdims=True)) @ v64


def attention_recurrence_f32(q: np.ndarray, kt: np.ndarray, v: np.ndarray, scale: float) -> np.ndarray:
    """The staged recurrence in FP32 (compiler/passes/recurrence.py:609-706, compiler/codegen/lower.py:264-270).

    scores (FP32 FMA over depth) -> scale -> row max -> w = 2^((s - m) * log2e) -> mass = sum w ->
    out = (sum_k w_k v_k) * (1 / mass). ex2.approx and rcp.approx are modelled by exact exp2 and
    division rounded to FP32 (the hardware approximations are within 2 ulp of these).
    """
    f32 = np.float32
    q, kt, v = (np.asarray(a, dtype=f32) for a in (q, kt, v))
    scores = np.zeros((q.shape[0], kt.shape[1]), dtype=f32)
    for d in range(q.shape[1]):
        scores = (scores.astype(np.float64) + q[:, d:d + 1].astype(np.float64) * kt[d:d + 1, :].astype(np.float64)).astype(f32)
    scores = scores * f32(scale)
    row_max = scores.max(axis=1, keepdims=True)
    weights = np.exp2(((scores - row_max) * f32(math.log2(math.e))).astype(f32)).astype(f32)
    mass = weights.sum(axis=1, keepdims=True, dtype=f32)
    weighted = np.zeros((q.shape[0], v.shape[1]), dtype=f32)
    for k in range(kt.shape[1]):
        weighted = (weighted.astype(np.float64) + weights[:, k:k + 1].astype(np.float64) * v[k:k + 1, :].astype(np.float64)).astype(f32)
    return (weighted * (f32(1.0) / mass)).astype(f32)


def gqa_attention_f64(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, heads=None, rows=None) -> np.ndarray:
    """Grouped-query attention in float64 on the stored (f16 or f32) inputs.

    q[B,Hq,S,D], k/v[B,Hkv,S,D]; query head h uses kv head h // (Hq // Hkv); non-causal. Each head is
    examples/attention.py:71-75 with kt = k[b,h].T. `heads` restricts to a list of (b, hq) pairs and
    `rows` to a list of query rows (the sampled oracle for sizes a CPU cannot finish in full).
    Returns out[B,Hq,S,D] (float64) with untouched entries left as NaN when a subset is requested.
    """
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    ratio = Hq // Hkv
    out = np.full((B, Hq, S, D), np.nan, dtype=np.float64)
    pairs = heads if heads is not None else [(b, h) for b in range(B) for h in range(Hq)]
    row_index = np.arange(S) if rows is None else np.asarray(rows)
    for b, h in pairs:
        kt = k[b, h // ratio].astype(np.float64).T
        out[b, h, row_index] = attention_f64(q[b, h, row_index], kt, v[b, h // ratio], scale)
    return out


# --------------------------------------------------------------------------------------------
# f16 storage (compiler/codegen/lower.py:249-256; tests/test_f16_storage.py:119-148)
# --------------------------------------------------------------------------------------------


def f16_narrow_bits(x: np.ndarray) -> np.ndarray:
    """fptrunc float->half = cvt.rn.f16.f32 written out on the bit patterns.

    Round to nearest even, overflow to +-inf, subnormal results kept, NaN stays NaN. Returns uint16.
    """
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.int64).reshape(-1)
    sign = (bits >> 16) & 0x8000
    magnitude = bits & 0x7FFFFFFF
    exponent = (magnitude >> 23) - 127
    mantissa = (magnitude & 0x7FFFFF) | 0x800000
    is_nan = magnitude > 0x7F800000
    is_inf = magnitude == 0x7F800000
    # shift that maps the 24-bit significand onto the half grid: 13 for normal halves, more for subnormals
    shift = np.clip(np.where(exponent >= -14, 13, 13 + (-14 - exponent)), 13, 40)
    kept = mantissa >> shift
    remainder = mantissa & ((np.int64(1) << shift) - 1)
    half = np.int64(1) << (shift - 1)
    round_up = (remainder > half) | ((remainder == half) & ((kept & 1) == 1))
    kept = kept + round_up
    # normal: kept carries the implicit bit at position 10, so adding (biased exponent - 1) << 10
    # lets a mantissa carry bump the exponent
    normal = ((np.clip(exponent, -14, 200) + 14) << 10) + kept
    value = np.where(exponent >= -14, normal, kept)
    value = np.where(value >= 0x7C00, 0x7C00, value)  # overflow -> inf
    value = np.where(magnitude == 0, 0, value)
    value = np.where(is_inf, 0x7C00, value)
    value = np.where(is_nan, 0x7E00, value)
    return (value | sign).astype(np.uint16).reshape(np.shape(x))


def f16_widen_bits(h: np.ndarray) -> np.ndarray:
    """fpext half->float on the bit patterns (exact). Takes uint16, returns float32."""
    bits = np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32)
    sign = (bits & 0x8000) << 16
    exponent = (bits >> 10) & 0x1F
    mantissa = bits & 0x3FF
    normal = sign | ((exponent + 112) << 23) | (mantissa << 13)
    special = sign | 0x7F800000 | (mantissa << 13)
    # subnormal halves: value = mantissa * 2^-24, exactly representable in FP32
    subnormal = (mantissa.astype(np.float32) * np.float32(2.0 ** -24)).view(np.uint32) | sign
    out = np.where(exponent == 0, subnormal, np.where(exponent == 31, special, normal)).astype(np.uint32)
    return out.view(np.float32).reshape(np.shape(h))


def f16_boundary_points() -> np.ndarray:
    """FP32 points at and next to every rounding boundary between adjacent finite halves, both signs,
    plus the special values; the set of tests/test_f16_storage.py:136-141 (padded to a multiple of 4)."""
    values = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    mid = (values[:-1] + values[1:]) * np.float32(0.5)
    points = np.concatenate((np.nextafter(mid, np.float32(-np.inf)), mid, np.nextafter(mid, np.float32(np.inf))))
    specials = np.array([0.0, -0.0, 65504.0, 65520.0, 65519.996, np.inf, -np.inf, np.nan], dtype=np.float32)
    points = np.concatenate((points, -points, specials)).astype(np.float32)
    return np.pad(points, (0, -points.size % 4))


# --------------------------------------------------------------------------------------------
# Elementwise and reductions
# --------------------------------------------------------------------------------------------


def vector_add(x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """examples/vector_add: exact IEEE FP32 add (meta rtol = atol = 0)."""
    return np.add(np.asarray(x, dtype=np.float32), np.asarray(y, dtype=np.float32), dtype=np.float32)


def row_sum_f64(x: np.ndarray) -> np.ndarray:
    """Row sums in float64: what the reassociated FP32 sums of compiler/codegen/lower.py:293-327, 418-421 approximate."""
    return np.asarray(x, dtype=np.float64).sum(axis=1)


def row_sumsq_f64(x: np.ndarray) -> np.ndarray:
    x64 = np.asarray(x, dtype=np.float64)
    return (x64 * x64).sum(axis=1)


def row_max(x: np.ndarray) -> np.ndarray:
    """NaN-suppressing maximum with identity -inf (llvm.maxnum, compiler/codegen/lower.py:275-278). Exact."""
    x = np.asarray(x, dtype=np.float32)
    if x.shape[1] == 0:
        return np.full(x.shape[0], -np.inf, dtype=np.float32)
    return np.fmax(np.fmax.reduce(x, axis=1), np.float32(-np.inf)).astype(np.float32)


def row_softmax_f64(x: np.ndarray) -> np.ndarray:
    """exp(x - max) / sum(exp(x - max)) per row in float64: what the reference's row-softmax kernel
    (compiler/passes/hybrid_normalizer.py:139-183: maximum, sum of exponentials, reciprocal, product) approximates."""
    x64 = np.asarray(x, dtype=np.float64)
    weights = np.exp(x64 - x64.max(axis=1, keepdims=True))
    return weights / weights.sum(axis=1, keepdims=True)


def rms_norm_f64(x: np.ndarray, weight: np.ndarray, count: float, epsilon: float) -> np.ndarray:
    """x * rsqrt(sum(x^2) / count + epsilon) * weight in float64 (the reference's RMS-norm workload: a sum of squares
    (compiler/transforms.py:62-95), scalar divide / add / rsqrt (compiler/codegen/lower.py:259-289), a forwarded
    consumer loop (compiler/passes/regforward.py:150-269))."""
    x64 = np.asarray(x, dtype=np.float64)
    scale = 1.0 / np.sqrt((x64 * x64).sum(axis=1, keepdims=True) / float(count) + float(epsilon))
    return x64 * scale * np.asarray(weight, dtype=np.float64)[None, :]


def l2_norm_f64(x: np.ndarray) -> np.ndarray:
    """x / sqrt(sum(x^2)) per row in float64 (sqrt followed by reciprocal, fused by compiler/transforms.py:6-9)."""
    x64 = np.asarray(x, dtype=np.float64)
    return x64 / np.sqrt((x64 * x64).sum(axis=1, keepdims=True))


def row_mean_f64(x: np.ndarray, count: float | None = None) -> np.ndarray:
    """sum(x) / count per row in float64 (the count arrives as a one-element buffer in the reference's mean workload)."""
    x64 = np.asarray(x, dtype=np.float64)
    return x64.sum(axis=1) / float(x64.shape[1] if count is None else count)


def row_sum_error_bound(x: np.ndarray) -> np.ndarray:
    """Bound on |fp32 tree sum - exact| per row for any summation order: (n-1) * eps * sum|x|."""
    x64 = np.abs(np.asarray(x, dtype=np.float64))
    return (x.shape[1] - 1) * np.finfo(np.float32).eps * x64.sum(axis=1)


def f16_affine(x: np.ndarray, scale: float = 1.5, bias: float = -0.25) -> np.ndarray:
    """examples/f16_storage.py:79-82: f16(f32(x) * scale + bias), each operator rounded once in FP32."""
    widened = np.asarray(x, dtype=np.float16).astype(np.float32)
    return (widened * np.float32(scale) + np.float32(bias)).astype(np.float32).astype(np.float16)


def f16_cancellation(x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """examples/f16_storage.py:83-84: f16((f32(x) + f32(y)) - f32(x)): the sum is kept in FP32, never rounded to f16."""
    a = np.asarray(x, dtype=np.float16).astype(np.float32)
    b = np.asarray(y, dtype=np.float16).astype(np.float32)
    with np.errstate(over='ignore'):
        return ((a + b) - a).astype(np.float16)
