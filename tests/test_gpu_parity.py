"""Parity of the CUDA path against the oracle and the reference's fixtures, through the C ABI.

Every test here launches kernels of libdeuteron_b200.so (via ctypes) on cuda:0. Bars:
  * bit-exact for vector add, f16 copy / widen / narrow, row max, and the FP32 contraction (whose
    output must hash to the reference's own published GPU output);
  * compensated GEMM: within the reference's rtol = atol = 1e-3 of the float64 product and max error
    no worse than 2x the reference's published error on its 128^3 example; elsewhere no worse than 2x
    the error floor of the three-product scheme plus the FP32 accumulation allowance stated below;
  * attention: the reference's rtol 1e-3 / atol 1e-4 against float64 and max error within 2x its published
    1.10e-7 on its example;
  * FP32 sums: within the order-independent bound (n-1) * eps * sum|x|.
"""
import hashlib
import math

import numpy as np
import pytest

from deuteron_b200 import LocalRunner, Options, compile_kernel, native, ops, schedules
from oracle import reference_math as R

pytestmark = pytest.mark.gpu


def sha(array):
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


@pytest.fixture(scope='module')
def dev(cuda):
    return cuda.device('cuda', 0)


@pytest.fixture(scope='module')
def runner(cuda):
    with LocalRunner(0) as local:
        yield local


def to_device(cuda, array):
    return cuda.from_numpy(np.ascontiguousarray(array)).to('cuda:0')


def run_with_data(runner, graph, meta, values, **timing):
    """tests/test_f16_storage.py:110-117: replace seeded inputs by explicit data, one launch."""
    import copy
    launch = copy.deepcopy(meta['kernels'][0])
    for arg in launch['args']:
        if arg['name'] in values:
            arg.pop('seed', None)
            arg['data'] = values[arg['name']]
    compiled = compile_kernel(graph, meta, arch='sm_100a', opt_level=3)
    timing = timing or {'warmup': 0, 'iters': 1, 'samples': 1}
    return runner.run_kernel(launch, compiled, **timing)['outputs']


# ------------------------------------------------------------------------------------------------
# elementwise and f16 storage
# ------------------------------------------------------------------------------------------------


def test_vector_add_example_is_exact_and_hashes_to_the_reference_output(runner, golden, published):
    graph, meta = schedules.vector_add_example()
    compiled = compile_kernel(graph, meta)
    result = runner.run_kernel(meta['kernels'][0], compiled, warmup=1, iters=3, samples=2)
    produced = result['outputs']['sum']
    np.testing.assert_array_equal(produced, np.load(golden / 'vector_add_expected.npz')['sum'])
    assert sha(produced) == published['results']['vector_add']['output_sha256']['sum']
    assert result['median_us'] > 0 and result['timing_method'] == 'cuda_graph_batch_events'
    # the result record carries the resources of the native kernel, as the reference's carries those of its PTX entry
    assert result['native_kernels'] >= 1 and 8 <= result['registers'] <= 255 and result['static_smem_bytes'] == 0


def test_f16_examples_hash_to_the_reference_outputs(runner, published):
    for kind in ('copy', 'widen', 'narrow', 'affine', 'cancellation'):
        for width in (4, 1):
            graph, meta = schedules.f16_storage_example(kind, width=width)
            compiled = compile_kernel(graph, meta)
            produced = runner.run_kernel(meta['kernels'][0], compiled, warmup=0, iters=1, samples=1)['outputs']['result']
            assert sha(produced) == published['results'][kind]['output_sha256']['result'], kind


def test_explicit_float_compute_avoids_half_intermediate_rounding(runner):
    # tests/test_f16_storage.py:150-155
    graph, meta = schedules.f16_storage_example('cancellation')
    x = np.resize(np.array([2048., 4096., 65504., -2048.], dtype=np.float16), 512)
    y = np.ones(512, dtype=np.float16)
    actual = run_with_data(runner, graph, meta, {'x': x, 'y': y})['result']
    np.testing.assert_array_equal(actual, y)


def test_fused_elementwise_programs_at_size_and_misalignment(runner, cuda):
    # large, odd-sized and offset buffers through the same compile/launch surface
    count = 1_000_004
    for kind, oracle in (('affine', lambda x, y: R.f16_affine(x)), ('cancellation', R.f16_cancellation)):
        for offset in (0, 1):
            if kind == 'cancellation' and offset:
                continue
            graph, meta = schedules.f16_storage_example(kind, count=count, width=4, offset=offset)
            x = R.seeded_normal(3, (count + offset,), np.float16, 30.0)
            y = R.seeded_normal(4, (count,), np.float16, 30.0)
            produced = run_with_data(runner, graph, meta, {'x': x, 'y': y})['result']
            np.testing.assert_array_equal(produced.view(np.uint16), oracle(x[offset:], y).view(np.uint16))
    # a longer chain on f32 buffers: relu(x * y + x) - |y|, then exp
    from deuteron_b200 import native
    n = 70_003
    x, y = R.seeded_normal(1, (n,)), R.seeded_normal(2, (n,))
    dx, dy = to_device(cuda, x), to_device(cuda, y)
    out = cuda.empty(n, device='cuda:0')
    ops_ = native.ELEMENTWISE_OPS
    program = {'ops': [ops_['multiply'], ops_['add'], ops_['relu'], ops_['absolute'], ops_['subtract']],
               'dst': [2, 2, 2, 3, 2], 'a': [0, 2, 2, 1, 2], 'b': [1, 0, 2, 1, 3], 'out_reg': 2, 'out_f16': False, 'n': n,
               'inputs': [{'f16': False, 'scalar': False}, {'f16': False, 'scalar': False}]}
    native.elementwise_program(program, [dx.data_ptr(), dy.data_ptr()], out.data_ptr(), cuda.cuda.current_stream().cuda_stream)
    expected = np.maximum((x * y).astype(np.float32) + x, 0).astype(np.float32) - np.abs(y)
    np.testing.assert_array_equal(out.cpu().numpy(), expected)


def test_pointwise_workloads_are_exact(runner):
    """x * 2 + 1 and relu(x) * y in the reference's launch shapes: one rounding per operator, so NumPy's FP32 result
    is reproduced bit for bit."""
    normal = lambda seed, n: np.random.default_rng(seed).standard_normal(n).astype(np.float32)
    graph, meta = schedules.pointwise_example('affine', 4096)
    got = runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta), warmup=0, iters=1, samples=1)['outputs']['add']
    np.testing.assert_array_equal(got, normal(0, 4096) * np.float32(2.0) + np.float32(1.0))
    graph, meta = schedules.pointwise_example('relu_multiply', 2048)
    got = runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta), warmup=0, iters=1, samples=1)['outputs']['mul']
    np.testing.assert_array_equal(got, np.maximum(normal(0, 2048), np.float32(0.0)) * normal(1, 2048))


PER_PROGRAM_CASES = [
    (schedules.pointwise_example, dict(kind='affine', count=4096)), (schedules.pointwise_example, dict(kind='affine', count=4)),
    (schedules.pointwise_example, dict(kind='affine', count=65536)), (schedules.pointwise_example, dict(kind='relu_multiply', count=2048)),
    (schedules.pointwise_example, dict(kind='relu_multiply', count=1028)), (schedules.pointwise_example, dict(kind='affine', count=4_000_004)),
    (schedules.f16_storage_example, dict(kind='affine', count=512)), (schedules.f16_storage_example, dict(kind='cancellation', count=512)),
    (schedules.f16_storage_example, dict(kind='affine', count=1_000_004)), (schedules.f16_storage_example, dict(kind='cancellation', count=262_144)),
    (schedules.f16_storage_example, dict(kind='affine', count=1000, offset=4)),
    (schedules.rms_norm_example, dict(rows=3000, cols=1024)), (schedules.row_softmax_example, dict(rows=20000, cols=128, block=32)),
    (schedules.l2_norm_example, dict(rows=1001, cols=4096)), (schedules.rms_norm_example, dict(rows=5, cols=8192)),
    (schedules.row_softmax_example, dict(rows=3, cols=16384)), (schedules.l2_norm_example, dict(rows=2, cols=32768)),
    (schedules.rms_norm_example, dict(rows=3, cols=32768)), (schedules.row_softmax_example, dict(rows=2, cols=12288)),
    (schedules.row_softmax_example, dict(rows=64, cols=256)), (schedules.row_softmax_example, dict(rows=3, cols=640)),
    (schedules.row_softmax_example, dict(rows=5, cols=4096)), (schedules.row_softmax_example, dict(rows=2, cols=96, block=32)),
    (schedules.rms_norm_example, dict(rows=64, cols=1024)), (schedules.rms_norm_example, dict(rows=7, cols=3072)),
    (schedules.rms_norm_example, dict(rows=1, cols=512)), (schedules.l2_norm_example, dict(rows=64, cols=512)),
    (schedules.l2_norm_example, dict(rows=1, cols=4096)), (schedules.l2_norm_example, dict(rows=16, cols=1536)),
    (schedules.mean_example, dict(count=4096)), (schedules.mean_example, dict(count=1024)),
    (schedules.row_reduce_example, dict(rows=64, cols=512)), (schedules.row_reduce_example, dict(rows=1, cols=1024)),
    (schedules.row_reduce_example, dict(rows=9, cols=4096, op='max')), (schedules.row_reduce_example, dict(rows=1, cols=65536)),
    (schedules.row_reduce_example, dict(rows=3, cols=20480, op='max')), (schedules.mean_example, dict(count=32768)),
    (schedules.attention_example, dict(rows=128, keys=128, depth=32)), (schedules.attention_example, dict(rows=64, keys=64, depth=64, columns=64)),
    (schedules.attention_example, dict(rows=3, keys=32, depth=5)), (schedules.attention_example, dict(rows=200, keys=256, depth=128, columns=64)),
    (schedules.attention_example, dict(rows=7, keys=96, depth=48, inplace_denominator=True)),
]


@pytest.mark.parametrize('make,settings', PER_PROGRAM_CASES, ids=lambda v: v.__name__ if callable(v) else '-'.join(str(x) for x in v.values()))
def test_per_program_kernels_equal_the_library_kernels(runner, monkeypatch, make, settings):
    """A small elementwise or row program runs a kernel compiled for that one program (jit.py). Its operators are the
    library's operators, so an elementwise program gives the library kernel's bits; a row program adds its row in another
    order (128 threads a row, whatever the row's length), so it is held to the row kernels' tolerance against the
    library kernel and must leave the same special values in the same places. The attention example of a few hundred
    rows runs a kernel unrolled for its shape that keeps the library kernel's order of operations, hence its bits."""
    graph, meta = make(**settings)
    launch = meta['kernels'][0]
    compiled = compile_kernel(graph, meta, arch='sm_100a', opt_level=3)
    assert runner._specialized(compiled.plan) is not None, 'the per-program kernel was not built'
    special = runner.run_kernel(launch, compiled, warmup=1, iters=2, samples=1)
    assert special['registers'] > 0
    monkeypatch.setenv('DTN_JIT', '0')
    plain = compile_kernel(graph, meta, arch='sm_100a', opt_level=3)
    assert runner._specialized(plain.plan) is None
    library = runner.run_kernel(launch, plain, warmup=1, iters=2, samples=1)
    for name, expected in library['outputs'].items():
        got = special['outputs'][name]
        if compiled.plan.kind in ('elementwise_program', 'attention'):   # the library kernel's operations in its order
            assert got.dtype == expected.dtype
            bits = np.uint16 if got.dtype == np.float16 else np.uint32
            np.testing.assert_array_equal(got.view(bits), expected.view(bits))
        else:
            # sums of n values of either sign in two orders differ by about 1e-7 n in the worst case, whatever the sum is
            params = compiled.plan.params
            if compiled.plan.kind == 'row_reduce' and params['op'] != 'max':
                atol = 3e-7 * params['cols']
            else:
                atol = 1e-6 if params.get('per_row') else 1e-7
            np.testing.assert_allclose(got, expected, rtol=1e-5, atol=atol)
            np.testing.assert_array_equal(np.isfinite(got), np.isfinite(expected))


@pytest.mark.parametrize('seed', range(12))
def test_random_programs_give_the_same_bits_on_both_kernels(cuda, seed):
    """Random register programs over every operator of the table, f32 and f16 buffers, scalar and vector inputs: the
    kernel written for the program (jit.py) and the library kernel that takes it as an argument must agree bit for bit
    (they apply the same operators in the same order), NaNs and infinities included. Random row programs likewise,
    within the row kernels' tolerance (the rows are added in another order)."""
    from deuteron_b200 import jit, native
    rng = np.random.default_rng(1000 + seed)
    stream = cuda.cuda.current_stream().cuda_stream
    operators = sorted(set(native.ELEMENTWISE_OPS.values()))
    n = int(rng.choice([4, 1000, 4096, 70_008]))
    inputs = [{'f16': bool(rng.integers(2)), 'scalar': bool(i > 0 and rng.integers(3) == 0)} for i in range(int(rng.integers(1, 4)))]
    count = int(rng.integers(1, 9))
    registers = len(inputs) + 3
    program = {'ops': [int(rng.choice(operators)) for _ in range(count)], 'dst': [int(rng.integers(len(inputs), registers)) for _ in range(count)],
               'a': [], 'b': [], 'inputs': inputs, 'out_f16': bool(rng.integers(2)), 'n': n}
    written = set(range(len(inputs)))
    for step in range(count):   # operands are inputs or registers an earlier step wrote
        program['a'].append(int(rng.choice(sorted(written))))
        program['b'].append(int(rng.choice(sorted(written))))
        written.add(program['dst'][step])
    program['out_reg'] = program['dst'][-1]
    tensors = []
    for spec in inputs:
        values = rng.standard_normal(1 if spec['scalar'] else n).astype(np.float32) * 3
        values[rng.integers(len(values))] = 0.0
        tensors.append(to_device(cuda, values.astype(np.float16) if spec['f16'] else values))
    buffers = {'out': ('out', 0), **{f'in{i}': (f'in{i}', 0) for i in range(len(inputs))}}
    spec = jit.elementwise_source(program, buffers)
    assert spec is not None
    kernel = jit.kernel_for(spec, 0)
    assert kernel is not None, 'NVRTC rejected a generated program'
    out_dtype = cuda.float16 if program['out_f16'] else cuda.float32
    mine, theirs = cuda.empty(n, dtype=out_dtype, device='cuda:0'), cuda.empty(n, dtype=out_dtype, device='cuda:0')
    pointers = {'out': mine.data_ptr(), **{f'in{i}': t.data_ptr() for i, t in enumerate(tensors)}}
    jit.launch(spec, kernel, pointers.__getitem__, stream)
    native.elementwise_program(program, [t.data_ptr() for t in tensors], theirs.data_ptr(), stream)
    bits = np.uint16 if program['out_f16'] else np.uint32
    np.testing.assert_array_equal(mine.cpu().numpy().view(bits), theirs.cpu().numpy().view(bits), err_msg=str(program))
    # a row program: a reduction, two scalar instructions, two elementwise instructions over the same operator table
    rows, cols = int(rng.choice([1, 7, 300])), int(rng.choice([4, 256, 1000, 4096, 12288]))
    unary_safe = [native.ELEMENTWISE_OPS[name] for name in ('add', 'subtract', 'multiply', 'maximum', 'minimum', 'negative', 'absolute', 'relu')]
    row_program = {'reduce': str(rng.choice(['sum', 'sumsq', 'max', 'softmax'])), 'rows': rows, 'cols': cols, 'per_row': False,
                   'inputs': [{'kind': 'columns'}, {'kind': 'immediate', 'value': float(rng.standard_normal())}], 'n_scalar': 2, 'out_reg': 7,
                   'ops': [int(rng.choice(unary_safe)) for _ in range(4)], 'dst': [5, 6, 7, 7], 'a': [0, 5, 2, 7], 'b': [4, 1, 6, 3]}
    x = to_device(cuda, (rng.standard_normal((rows, cols)) * 2).astype(np.float32))
    weights = to_device(cuda, rng.standard_normal(cols).astype(np.float32))
    row_spec = jit.row_source(row_program, {'x': ('x', 0), 'out': ('out', 0), 'in0': ('w', 0), 'in1': ('c', 0)})
    assert row_spec is not None
    row_kernel = jit.kernel_for(row_spec, 0)
    assert row_kernel is not None, 'NVRTC rejected a generated row program'
    mine, theirs = cuda.empty_like(x), cuda.empty_like(x)
    jit.launch(row_spec, row_kernel, {'x': x.data_ptr(), 'out': mine.data_ptr(), 'in0': weights.data_ptr()}.__getitem__, stream)
    native.row_fused(row_program, x.data_ptr(), [weights.data_ptr(), None], theirs.data_ptr(), cols, cols, stream)
    ops.check_device_status()
    got, expected = mine.cpu().numpy(), theirs.cpu().numpy()
    scale = max(1.0, float(np.abs(expected[np.isfinite(expected)]).max(initial=0.0)))
    np.testing.assert_allclose(got, expected, rtol=2e-5, atol=2e-5 * scale * max(1, cols // 256), err_msg=str(row_program))


def test_all_half_bits_copy_exactly_at_scalar_and_vector_widths(runner):
    data = np.arange(65536, dtype=np.uint16).view(np.float16)
    for width in (1, 2, 4):
        graph, meta = schedules.f16_storage_example('copy', count=data.size, width=width)
        actual = run_with_data(runner, graph, meta, {'x': data})['result']
        np.testing.assert_array_equal(actual.view(np.uint16), data.view(np.uint16))


def test_half_widening_is_exact_on_every_pattern(runner):
    data = np.arange(65536, dtype=np.uint16).view(np.float16)
    graph, meta = schedules.f16_storage_example('widen', count=data.size)
    actual = run_with_data(runner, graph, meta, {'x': data})['result']
    expected = R.f16_widen_bits(data.view(np.uint16))
    finite = ~np.isnan(expected)
    np.testing.assert_array_equal(actual[finite].view(np.uint32), expected[finite].view(np.uint32))
    np.testing.assert_array_equal(np.isnan(actual), np.isnan(expected))


def test_round_to_nearest_even_half_boundaries(runner):
    points = R.f16_boundary_points()
    graph, meta = schedules.f16_storage_example('narrow', count=points.size)
    actual = run_with_data(runner, graph, meta, {'x': points})['result']
    expected = R.f16_narrow_bits(points)
    finite = ~np.isnan(points)
    np.testing.assert_array_equal(actual.view(np.uint16)[finite], expected[finite])
    assert np.isnan(actual[~finite]).all()


def test_unaligned_vector_half_access(runner):
    for kind in ('copy', 'narrow'):
        graph, meta = schedules.f16_storage_example(kind, count=512, offset=1)
        data = np.arange(513, dtype=np.float16 if kind == 'copy' else np.float32)
        actual = run_with_data(runner, graph, meta, {'x': data})['result']
        np.testing.assert_array_equal(actual, data[1:].astype(np.float16))


def test_f16_kernels_at_every_relative_misalignment(cuda):
    n = 100_003
    source32 = R.seeded_normal(3, (n + 16,), np.float32, 100.0)
    source16 = source32.astype(np.float16)
    d32, d16 = to_device(cuda, source32), to_device(cuda, source16)
    for a in (0, 1, 3, 8):
        for b in (0, 1, 5):
            out16 = cuda.zeros(n + 16, dtype=cuda.float16, device='cuda:0')
            out32 = cuda.zeros(n + 16, dtype=cuda.float32, device='cuda:0')
            ops.f16_narrow(d32[a:a + n], out16[b:b + n])
            np.testing.assert_array_equal(out16[b:b + n].cpu().numpy().view(np.uint16), R.f16_narrow_bits(source32[a:a + n]))
            ops.f16_widen(d16[a:a + n], out32[b:b + n])
            np.testing.assert_array_equal(out32[b:b + n].cpu().numpy(), source16[a:a + n].astype(np.float32))
            ops.f16_copy(d16[a:a + n], out16[b:b + n])
            np.testing.assert_array_equal(out16[b:b + n].cpu().numpy().view(np.uint16), source16[a:a + n].view(np.uint16))
            assert float(out16[b + n:].abs().sum()) == 0.0 and float(out16[:b].abs().sum()) == 0.0  # no overrun


def test_elementwise_operators_and_empty_input(cuda):
    x, y = R.seeded_normal(1, (70_001,)), R.seeded_normal(2, (70_001,))
    dx, dy = to_device(cuda, x), to_device(cuda, y)
    exact = {'add': x + y, 'subtract': x - y, 'multiply': x * y, 'maximum': np.fmax(x, y), 'minimum': np.fmin(x, y)}
    for op, expected in exact.items():
        np.testing.assert_array_equal(ops.elementwise(op, dx, dy).cpu().numpy(), expected, err_msg=op)
    np.testing.assert_array_equal(ops.elementwise('relu', dx).cpu().numpy(), np.maximum(x, 0))
    np.testing.assert_array_equal(ops.elementwise('negative', dx).cpu().numpy(), -x)
    np.testing.assert_array_equal(ops.elementwise('absolute', dx).cpu().numpy(), np.abs(x))
    np.testing.assert_array_equal(ops.elementwise('copy', dx).cpu().numpy(), x)
    np.testing.assert_allclose(ops.elementwise('exp', dx).cpu().numpy(), np.exp(x.astype(np.float64)), rtol=2e-6)
    np.testing.assert_allclose(ops.elementwise('divide', dx, dy).cpu().numpy(), x.astype(np.float64) / y, rtol=1e-6)
    np.testing.assert_allclose(ops.elementwise('reciprocal', dy).cpu().numpy(), 1 / y.astype(np.float64), rtol=1e-6)
    np.testing.assert_allclose(ops.elementwise('sqrt', ops.elementwise('absolute', dx)).cpu().numpy(), np.sqrt(np.abs(x.astype(np.float64))), rtol=1e-6)
    empty = cuda.empty(0, device='cuda:0')
    assert ops.add(empty, empty).numel() == 0
    with pytest.raises(ValueError):
        ops.add(dx, dy[:-1])
    with pytest.raises(NotImplementedError):
        ops.elementwise('tanh', dx)


def test_vector_add_full_size_is_exact(cuda):
    n = 1 << 28
    generator = cuda.Generator(device='cuda:0').manual_seed(21)
    x = cuda.randn(n, device='cuda:0', generator=generator)
    y = cuda.randn(n, device='cuda:0', generator=generator)
    out = ops.add(x, y)
    reference = x + y   # torch's own IEEE add: the same single rounding
    assert bool(cuda.equal(out, reference))
    # a checksum of checksums independent of torch's add: float64 sums of slices agree to rounding
    assert abs(float(out.double().sum()) - float(x.double().sum() + y.double().sum())) < 1e-2 * math.sqrt(n)


# ------------------------------------------------------------------------------------------------
# row reductions
# ------------------------------------------------------------------------------------------------


@pytest.mark.parametrize('rows,cols', [(64, 512), (300, 4096), (77, 1001), (5, 65539), (1, 65536), (3, 1), (9, 33)])
def test_row_reductions_against_float64(cuda, rows, cols):
    x = R.seeded_normal(7, (rows, cols))
    dx = to_device(cuda, x)
    bound = R.row_sum_error_bound(x) + 1e-30
    assert np.all(np.abs(ops.row_reduce('sum', dx).cpu().numpy() - R.row_sum_f64(x)) <= bound)
    squares = R.row_sumsq_f64(x)   # each square rounds once more than a plain term does
    assert np.all(np.abs(ops.row_reduce('sumsq', dx).cpu().numpy() - squares) <= (cols + 1) * np.finfo(np.float32).eps * squares + 1e-30)
    np.testing.assert_array_equal(ops.row_reduce('max', dx).cpu().numpy(), R.row_max(x))


def test_row_reduction_edge_cases(cuda, runner):
    x = R.seeded_normal(7, (4, 1000))
    x[1, 17] = np.nan
    x[2, :] = np.nan
    x[3, 5] = np.inf
    got = ops.row_reduce('max', to_device(cuda, x)).cpu().numpy()
    np.testing.assert_array_equal(got, R.row_max(x))          # NaN-suppressing, all-NaN row -> -inf
    wide = to_device(cuda, R.seeded_normal(1, (16, 4100)))
    view = wide[:, 4:4 + 4000]                                  # strided rows, 16-byte aligned origin
    np.testing.assert_array_equal(ops.row_reduce('max', view).cpu().numpy(), view.cpu().numpy().max(axis=1))
    view = wide[:, 1:1 + 4000]                                  # unaligned origin: scalar path
    np.testing.assert_array_equal(ops.row_reduce('max', view).cpu().numpy(), view.cpu().numpy().max(axis=1))
    assert ops.row_reduce('sum', cuda.empty((0, 8), device='cuda:0')).numel() == 0
    zero_cols = ops.row_reduce('max', cuda.empty((3, 0), device='cuda:0')).cpu().numpy()
    assert np.all(zero_cols == -np.inf)
    # through the compile/launch surface, in the reference's row-sum launch shape
    for op, oracle in (('sum', R.row_sum_f64), ('max', R.row_max)):
        graph, meta = schedules.row_reduce_example(64, 512, op)
        produced = runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta), warmup=0, iters=1, samples=1)['outputs']['out']
        np.testing.assert_allclose(produced, oracle(R.seeded_normal(7, (64, 512))), rtol=1e-5, atol=1e-4)


def test_row_reductions_full_size(cuda):
    rows, cols = 65536, 4096
    generator = cuda.Generator(device='cuda:0').manual_seed(7)
    x = cuda.randn((rows, cols), device='cuda:0', generator=generator)
    sums, maxima = ops.row_reduce('sum', x), ops.row_reduce('max', x)
    assert bool(cuda.equal(maxima, x.max(dim=1).values))
    exact = x.double().sum(dim=1)
    bound = (cols - 1) * np.finfo(np.float32).eps * x.double().abs().sum(dim=1)
    assert bool(((sums.double() - exact).abs() <= bound).all())
    # sum of the row sums equals the sum of everything (float64, order-free up to rounding)
    assert abs(float(sums.double().sum()) - float(exact.sum())) < 1.0


# ------------------------------------------------------------------------------------------------
# fused row kernels: softmax, RMS norm, L2 norm, mean
# Bars: relative 1e-5 of the float64 result (ex2.approx, rsqrt.approx, rcp.approx and div.approx are each good to
# about 2^-22 and at most three of them are chained), plus an absolute floor for values that underflow in FP32.
# ------------------------------------------------------------------------------------------------

ROW_RTOL = 1e-5


@pytest.fixture(params=['1', '0'], ids=['per-program-kernels', 'library-kernels'])
def row_paths(request, monkeypatch):
    """The row operators run a kernel compiled for the one program where there is one (jit.py) and the library's kernel
    otherwise; `DTN_JIT=0` sends everything to the library. Both are held to the same bars."""
    monkeypatch.setenv('DTN_JIT', request.param)
    return request.param


def test_row_kernels_in_the_reference_launch_shapes(runner):
    run = lambda graph, meta: runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta, arch='sm_100a'), warmup=0, iters=1,
                                                samples=1)['outputs']
    normal = lambda seed, shape: np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
    got = run(*schedules.row_softmax_example())['softmax']
    np.testing.assert_allclose(got, R.row_softmax_f64(normal(0, (64, 256))), rtol=ROW_RTOL, atol=1e-12)
    np.testing.assert_allclose(got.astype(np.float64).sum(axis=1), 1.0, rtol=0, atol=1e-5)
    got = run(*schedules.rms_norm_example())['mul_1']
    np.testing.assert_allclose(got, R.rms_norm_f64(normal(0, (64, 1024)), normal(1, (1024,)), 1024.0, 1e-5), rtol=ROW_RTOL, atol=1e-7)
    got = run(*schedules.l2_norm_example())['div']
    np.testing.assert_allclose(got, R.l2_norm_f64(normal(0, (64, 512))), rtol=ROW_RTOL, atol=1e-9)
    got = run(*schedules.mean_example())['mean']
    x = normal(0, (1, 32768))
    assert abs(float(got[0]) - float(R.row_mean_f64(x)[0])) <= float(R.row_sum_error_bound(x)[0]) / 32768 + 1e-9


@pytest.mark.parametrize('rows,cols', [(64, 256), (5, 1000), (3, 1001), (1, 8192), (2, 8196), (7, 40000), (300, 33), (1, 1), (1100, 512)])
def test_row_kernels_against_float64_at_many_shapes(cuda, rows, cols, row_paths):
    x = R.seeded_normal(7, (rows, cols)) * np.float32(3.0)
    w = R.seeded_normal(8, (cols,))
    dx, dw = to_device(cuda, x), to_device(cuda, w)
    np.testing.assert_allclose(ops.row_softmax(dx).cpu().numpy(), R.row_softmax_f64(x), rtol=ROW_RTOL, atol=1e-12)
    np.testing.assert_allclose(ops.rms_norm(dx, dw, 1e-5).cpu().numpy(), R.rms_norm_f64(x, w, cols, 1e-5), rtol=ROW_RTOL, atol=1e-7)
    np.testing.assert_allclose(ops.l2_norm(dx).cpu().numpy(), R.l2_norm_f64(x), rtol=ROW_RTOL, atol=1e-9)
    bound = R.row_sum_error_bound(x) / cols + 5e-7 * np.abs(R.row_mean_f64(x)) + 1e-12   # div.approx is good to 2 ulp
    assert np.all(np.abs(ops.row_mean(dx).cpu().numpy() - R.row_mean_f64(x)) <= bound)


def test_row_kernel_edge_cases(cuda, row_paths):
    # strided rows and a misaligned origin take the scalar path and give the same values as the aligned path
    base = cuda.randn((16, 1030), device='cuda:0', generator=cuda.Generator(device='cuda:0').manual_seed(3))
    view = base[:, 1:1025]
    dense = view.contiguous()
    for op in (ops.row_softmax, ops.l2_norm):
        np.testing.assert_allclose(op(view).cpu().numpy(), op(dense).cpu().numpy(), rtol=2e-6, atol=1e-12)
    # a row of equal values, a row with one dominant value, large magnitudes (no overflow: the maximum is subtracted first)
    x = np.zeros((3, 512), dtype=np.float32)
    x[0, :] = 5.0
    x[1, 17] = 80.0
    x[2, :] = np.linspace(-3.0e4, 3.0e4, 512, dtype=np.float32)
    got = ops.row_softmax(to_device(cuda, x)).cpu().numpy()
    np.testing.assert_allclose(got, R.row_softmax_f64(x), rtol=ROW_RTOL, atol=1e-30)
    assert np.isfinite(got).all() and got[1, 17] == 1.0
    # a program whose elementwise stage is not a chain takes the interpreter: (x - mean) * (x + mean)
    x = R.seeded_normal(5, (9, 700))
    dx = to_device(cuda, x)
    program = [('divide', 4, 0, 3), ('subtract', 5, 2, 4), ('add', 6, 2, 4), ('multiply', 7, 5, 6)]
    got = ops._row_fused('sum', dx, program, 1, 7, inputs=(700.0,)).cpu().numpy()
    mean = R.row_mean_f64(x)[:, None]
    np.testing.assert_allclose(got, (x - mean) * (x + mean), rtol=1e-5, atol=1e-5)
    # a chain that reads the row element again after its first step: (x - max) * x
    got = ops._row_fused('max', dx, [('subtract', 3, 2, 0), ('multiply', 3, 3, 2)], 0, 3).cpu().numpy()
    np.testing.assert_array_equal(got, (x - x.max(axis=1, keepdims=True)) * x)
    # empty inputs
    assert ops.row_softmax(cuda.empty((0, 8), device='cuda:0')).shape == (0, 8)
    assert ops.row_mean(cuda.empty((0, 8), device='cuda:0')).numel() == 0
    with pytest.raises(ValueError):
        ops.row_softmax(cuda.zeros(4, device='cuda:0'))
    with pytest.raises(ValueError):
        ops.rms_norm(cuda.zeros((4, 8), device='cuda:0'), cuda.zeros(3, device='cuda:0'))


def test_row_kernels_full_size(cuda, row_paths):
    """65536 x 4096 (1 GiB): size-independent properties. Softmax rows sum to one and are invariant under a shift of the
    row; normalised rows have unit norm; the RMS norm with unit weight has mean square one."""
    rows, cols = 65536, 4096
    x = cuda.randn((rows, cols), device='cuda:0', generator=cuda.Generator(device='cuda:0').manual_seed(7))
    out = ops.row_softmax(x)
    assert float((out.double().sum(dim=1) - 1.0).abs().max()) < 1e-5
    reference = cuda.softmax(x[:64].double(), dim=1)
    assert bool(((out[:64].double() - reference).abs() <= ROW_RTOL * reference + 1e-12).all())
    x.add_(100.0)
    shifted = ops.row_softmax(x)
    assert float((shifted - out).abs().max()) < 2e-4 * float(out.max())   # x + 100 rounds the inputs to 2^-17
    x.sub_(100.0)
    del shifted
    ops.l2_norm(x, out=out)
    assert float(((out.double() ** 2).sum(dim=1) - 1.0).abs().max()) < 1e-5
    ops.rms_norm(x, cuda.ones(cols, device='cuda:0'), 0.0, out=out)
    assert float(((out.double() ** 2).mean(dim=1) - 1.0).abs().max()) < 1e-5
    means = ops.row_mean(x)
    assert float((means.double() - x.double().mean(dim=1)).abs().max()) < 1e-5


def test_split_k_contraction_is_the_full_product(runner):
    graph, meta = schedules.split_k_matmul_example()
    result = runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta, arch='sm_100a'), warmup=0, iters=1, samples=2)
    produced = result['outputs']['matmul']
    # the launch resets its output before every launch, as the reference's does; the native kernel overwrites it anyway,
    # so the time without the reset is reported beside the comparable one
    assert result['timing_includes_output_resets'] and 0 < result['kernel_only_us'] <= result['median_us'] * 1.5
    assert result['native_kernels'] == 1 and result['static_smem_bytes'] > 0
    normal = lambda seed, shape: np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
    np.testing.assert_allclose(produced, R.gemm_f64(normal(0, (128, 256)), normal(1, (256, 64))), rtol=1e-3, atol=1e-3)


def test_fp32_split_k_mode_adds_partial_sums_in_a_fixed_order(cuda):
    # few output tiles and a long k: clusters of 8 or 4 CTAs along k (or one CTA when there are tiles enough); FP32
    # accuracy, the same bits on every run, ragged edges
    for m, n, k in ((128, 64, 256), (64, 64, 1024), (100, 70, 333), (32, 32, 64), (512, 512, 128)):
        a, b = to_device(cuda, R.seeded_normal(0, (m, k))), to_device(cuda, R.seeded_normal(1, (k, n)))
        first = ops.gemm(a, b, 'f32_splitk').clone()
        again = ops.gemm(a, b, 'f32_splitk')
        assert bool(cuda.equal(first, again))
        exact = a.double() @ b.double()
        assert float(((first.double() - exact).abs().max() / exact.abs().max()).item()) < 5e-7
        sequential = ops.gemm(a, b, 'f32')
        assert float((first - sequential).abs().max().item()) <= 4e-5 * float(exact.abs().max().item())


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------


def test_tensor_matmul_example_all_modes(runner, golden, published):
    graph, meta = schedules.matmul_example()
    expected = np.load(golden / 'tensor_matmul_expected.npz')['result']
    names = {'bf16x3': 'tensor_bf16x3', 'tf32x3': 'tensor_tf32x3', 'f32': 'tensor_f32'}
    for mode, record in names.items():
        compiled = compile_kernel(graph, meta, arch='sm_100a', opt_level=3, options=Options(contraction_precision=mode))
        produced = runner.run_kernel(meta['kernels'][0], compiled, warmup=1, iters=2, samples=1)['outputs']['result']
        np.testing.assert_allclose(produced, expected, rtol=meta['rtol'], atol=meta['atol'])
        error = float(np.max(np.abs(produced.astype(np.float64) - expected)))
        assert error <= 2 * published['results'][record]['max_absolute_errors']['result'], (mode, error)
    # the FP32 mode accumulates k in the reference's order: identical bits to its published GPU output
    assert sha(produced) == published['results']['tensor_f32']['output_sha256']['result']


@pytest.mark.parametrize('variant', [0, 1, 3, 4, 5, 7])
def test_compensated_modes_hash_to_the_reference_gpu_outputs(cuda, published, variant):
    # Same split, same three products in the same order per k-step, FP32 tensor-core accumulation: every kernel
    # variant reproduces the bits of the reference's own run of its 128^3 example (published SHA-256 and max error).
    left, right = R.seeded_normal(7, (128, 128)), R.seeded_normal(11, (128, 128))
    exact = R.gemm_f64(left, right)
    ops.set_gemm_variant(variant)
    try:
        for mode, record in (('bf16x3', 'tensor_bf16x3'), ('tf32x3', 'tensor_tf32x3')):
            produced = ops.gemm(to_device(cuda, left), to_device(cuda, right), mode).cpu().numpy()
            assert sha(produced) == published['results'][record]['output_sha256']['result'], (mode, variant)
            assert float(np.max(np.abs(produced - exact))) == published['results'][record]['max_absolute_errors']['result']
    finally:
        ops.set_gemm_variant(0)


def test_reference_committed_ir_runs_unchanged(runner, golden, published):
    import json
    graph = json.loads((golden / 'tensor_matmul.ir.json').read_text())
    meta = published['meta']['tensor_matmul']
    compiled = compile_kernel(graph, meta, arch='sm_100a')
    produced = runner.run_kernel(meta['kernels'][0], compiled, warmup=0, iters=1, samples=1)['outputs']['result']
    np.testing.assert_allclose(produced, np.load(golden / 'tensor_matmul_expected.npz')['result'], rtol=1e-3, atol=1e-3)


def test_ir_of_the_reference_example_generators_runs_unchanged(runner, golden):
    """The IR and meta the reference's example scripts build (tests/golden/reference_examples.json), through
    compile_kernel + run_kernel unchanged: attention within the scripts' own tolerance of the float64 expectation
    (examples/attention.py:67), the in-place-denominator variant identical to the plain one
    (tests/test_attention.py:122), f16 kernels bit for bit what NumPy gives (examples/f16_storage.py:79-86)."""
    import json
    from deuteron_b200 import argument_array
    examples = json.loads((golden / 'reference_examples.json').read_text())
    outputs = {}
    for name, case in examples.items():
        launch = case['meta']['kernels'][0]
        produced = runner.run_kernel(launch, compile_kernel(case['graph'], case['meta']), warmup=0, iters=1, samples=1)['outputs']
        values = {arg['name']: argument_array(arg) for arg in launch['args'] if not arg.get('output')}
        if name.startswith('attention'):
            exact = R.attention_f64(values['q'], values['kt'], values['v'])
            np.testing.assert_allclose(produced['out'], exact, rtol=1e-3, atol=1e-4)
            assert R.max_relative_error(produced["out"], exact) < 1e-6   # FP32 recurrence; the bar against the reference kernel itself is in test_reference_kernel.py
            outputs[name] = produced['out']
        else:
            kind = name.split('_')[1]
            x = values['x'].astype(np.float32)
            expected = {'copy': lambda: values['x'], 'widen': lambda: x, 'narrow': lambda: x.astype(np.float16),
                        'affine': lambda: (x * values['scale'][0] + values['bias'][0]).astype(np.float16),
                        'cancellation': lambda: ((x + values['y'].astype(np.float32)) - x).astype(np.float16)}[kind]()
            assert produced['result'].dtype == expected.dtype
            np.testing.assert_array_equal(produced['result'].view(np.uint16 if expected.dtype == np.float16 else np.uint32),
                                          expected.view(np.uint16 if expected.dtype == np.float16 else np.uint32))
    np.testing.assert_array_equal(outputs['attention_128x128x32'], outputs['attention_128x128x32_inplace'])


SHAPES = [(128, 128, 128), (256, 256, 64), (384, 768, 1000), (200, 136, 77), (16, 512, 512), (1, 1, 1), (129, 257, 65),
          (1024, 1024, 1024)]


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
@pytest.mark.parametrize('variant', [1, 2, 3, 4, 5, 7])   # tcgen05 tiles 128x128, 128x256, CTA pair 256x256; single-kernel; 128x64; stream
def test_compensated_gemm_shapes_and_variants(cuda, mode, variant):
    ops.set_gemm_variant(variant)
    try:
        for m, n, k in SHAPES:
            a, b = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
            produced = ops.gemm(to_device(cuda, a), to_device(cuda, b), mode)
            ops.check_device_status()
            exact = R.gemm_f64(a, b)
            floor = R.max_relative_error(R.gemm_x3_exact_products(a, b, mode), exact)
            # FP32 accumulation of 3 * k / (k-step) partial sums in the tensor core, the same count the
            # reference's mma.sync loop performs: allow one truncated unit in the last place per accumulation
            steps = 3 * math.ceil(k / (16 if mode == 'bf16x3' else 8))
            allowance = steps * 2.0 ** -24
            error = R.max_relative_error(produced.cpu().numpy(), exact)
            assert error <= 2 * floor + allowance, (m, n, k, error, floor, allowance)
    finally:
        ops.set_gemm_variant(0)


FUSED_SHAPES = [(128, 128, 128), (256, 256, 64), (384, 768, 1000), (200, 136, 80), (16, 512, 512), (1, 8, 8), (129, 264, 72),
                (1024, 1024, 1024), (2048, 1536, 1280)]


@pytest.mark.parametrize('tile_width', ['64', '128'])
def test_fused_split_gemm_reproduces_the_two_kernel_path(cuda, monkeypatch, published, tile_width):
    # One tcgen05 kernel with the operand split in its producer warps: the same rounded operands, the same three
    # products in the same order, so the output is the two-kernel path's bit for bit -- at every shape it accepts,
    # with row, column and k remainders, at both tile widths -- and the reference's published 128^3 output.
    monkeypatch.setenv('DTN_GEMM_FUSED_BN', tile_width)
    try:
        for m, n, k in FUSED_SHAPES:
            a, b = to_device(cuda, R.seeded_uniform(7, (m, k))), to_device(cuda, R.seeded_uniform(11, (k, n)))
            ops.set_gemm_variant(1)
            expected = ops.gemm(a, b, 'bf16x3').cpu().numpy()
            ops.set_gemm_variant(6)
            produced = ops.gemm(a, b, 'bf16x3').cpu().numpy()
            ops.check_device_status()
            assert np.array_equal(produced, expected), (m, n, k)
        # a column block of a wider matrix, written into a column block of a wider result (leading dimensions > extents)
        a = to_device(cuda, R.seeded_uniform(7, (512, 768)))
        b = to_device(cuda, R.seeded_uniform(11, (768, 1024)))
        c = cuda.zeros((512, 1024), device='cuda:0')
        ops.gemm(a, b[:, 256:640], 'bf16x3', out=c[:, 256:640])
        ops.set_gemm_variant(1)
        assert cuda.equal(c[:, 256:640], ops.gemm(a, b[:, 256:640].contiguous(), 'bf16x3'))
        assert float(c[:, :256].abs().max()) == 0 and float(c[:, 640:].abs().max()) == 0
        ops.set_gemm_variant(6)
        left, right = R.seeded_normal(7, (128, 128)), R.seeded_normal(11, (128, 128))
        produced = ops.gemm(to_device(cuda, left), to_device(cuda, right), 'bf16x3').cpu().numpy()
        assert sha(produced) == published['results']['tensor_bf16x3']['output_sha256']['result']
        # shapes and modes it does not take are refused, not routed elsewhere
        with pytest.raises(Exception, match='fused-split'):
            ops.gemm(to_device(cuda, R.seeded_uniform(7, (64, 77))), to_device(cuda, R.seeded_uniform(11, (77, 64))), 'bf16x3')
        with pytest.raises(Exception, match='fused-split'):
            ops.gemm(to_device(cuda, left), to_device(cuda, right), 'tf32x3')
    finally:
        ops.set_gemm_variant(0)


SKINNY_SHAPES = [(16, 8192, 4096), (1, 4096, 4096), (7, 4100, 2052), (16, 2048 + 36, 1024 + 4), (3, 128, 65536), (16, 65536, 64)]


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
def test_skinny_gemm_streams_b_once(cuda, mode):
    """At most 16 rows: the TMA-fed kernel (every SM takes an equal share of B; partial sums of a column block meet in
    the workspace and are added in a fixed order). Ragged N and K, one row, very long and very short k; the same
    launch twice gives the same bits, whoever arrives last."""
    ops.set_gemm_variant(10)   # the streamed kernel whatever the size
    try:
        _check_skinny_shapes(cuda, mode)
    finally:
        ops.set_gemm_variant(0)


def _check_skinny_shapes(cuda, mode):
    for m, n, k in SKINNY_SHAPES:
        a, b = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
        left, right = to_device(cuda, a), to_device(cuda, b)
        produced = ops.gemm(left, right, mode)
        ops.check_device_status()
        again = ops.gemm(left, right, mode)
        assert cuda.equal(produced, again), (m, n, k)
        exact = R.gemm_f64(a, b)
        floor = R.max_relative_error(R.gemm_x3_exact_products(a, b, mode), exact)
        steps = 3 * math.ceil(k / (16 if mode == 'bf16x3' else 8))
        error = R.max_relative_error(produced.cpu().numpy(), exact)
        assert error <= 2 * floor + steps * 2.0 ** -24, (m, n, k, error, floor)
        # a view with padded leading dimensions and an output that is not 16-byte aligned
        wide = cuda.zeros((k, n + 12), device='cuda:0')
        wide[:, 4:n + 4] = right
        shifted = ops.gemm(left, wide[:, 4:n + 4], mode)
        assert cuda.equal(shifted, produced), (m, n, k)
        # the workspace needs no preparation: all ones, all zeros, what the last launch left, other launches' leftovers
        scratch = cuda.empty(ops.gemm_workspace_bytes(mode, m, n, k) + 2048, dtype=cuda.uint8, device='cuda:0')
        for fill in (0xFF, 0x00, None, None, 0x3C):
            if fill is not None:
                scratch.fill_(fill)
            assert cuda.equal(ops.gemm(left, right, mode, workspace=scratch), produced), (m, n, k, fill)
    # back to back in one CUDA graph (every replay repeats the launch's arrival token)
    m, n, k = 16, 2048, 4096
    left, right = to_device(cuda, R.seeded_uniform(7, (m, k))), to_device(cuda, R.seeded_uniform(11, (k, n)))
    expected = ops.gemm(left, right, mode).clone()
    out = cuda.empty_like(expected)
    scratch = cuda.empty(ops.gemm_workspace_bytes(mode, m, n, k) + 2048, dtype=cuda.uint8, device='cuda:0')
    stream = cuda.cuda.Stream()
    with cuda.cuda.stream(stream):
        ops.gemm(left, right, mode, out=out, workspace=scratch)
        graph = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph, stream=stream):
            for _ in range(8):
                ops.gemm(left, right, mode, out=out, workspace=scratch)
        for _ in range(5):
            out.zero_()
            graph.replay()
            stream.synchronize()
            assert cuda.equal(out, expected)
    ops.check_device_status()


def test_gemm_f32_mode_shapes(cuda):
    for m, n, k in SHAPES[:-1]:
        a, b = R.seeded_normal(7, (m, k)), R.seeded_normal(11, (k, n))
        produced = ops.gemm(to_device(cuda, a), to_device(cuda, b), 'f32').cpu().numpy()
        if m * n * k <= 128 ** 3:
            np.testing.assert_array_equal(produced, R.gemm_f32_fma(a, b))  # sequential FMA over k: bit-exact
        assert R.max_relative_error(produced, R.gemm_f64(a, b)) < 2e-6


def test_gemm_f32_result_does_not_depend_on_the_tile(cuda):
    # The FP32 mode picks 32x32, 64x64 or 128x128 CTA tiles by problem size; every output element is the same sequential
    # FMA chain over k in all three, so a corner of a large product equals the small product of the corner operands, bit
    # for bit. Shapes: 64-wide tiles with and without 16-byte alignment, 128-wide tiles.
    for m, n, k in ((640, 640, 100), (641, 643, 77), (1536, 1536, 64)):
        a, b = to_device(cuda, R.seeded_normal(7, (m, k))), to_device(cuda, R.seeded_normal(11, (k, n)))
        whole = ops.gemm(a, b, 'f32')
        corner = ops.gemm(a[m - 48:].contiguous(), b[:, n - 40:].contiguous(), 'f32')   # 48 x 40: one 32-wide-tile launch
        assert cuda.equal(whole[m - 48:, n - 40:], corner), (m, n, k)
        rows = slice(0, m, 97)
        exact = a[rows].double() @ b.double()
        assert float(((whole[rows].double() - exact).abs().max() / exact.abs().max()).item()) < 2e-6
        np.testing.assert_array_equal(whole[:8, :8].cpu().numpy(), R.gemm_f32_fma(a[:8].cpu().numpy(), b[:, :8].cpu().numpy()))


def test_push_block_copies_one_block_into_every_destination(cuda):
    # The exchange step of the sharded GEMM: a column block of one matrix written into the same place of several other
    # copies (here: buffers of the same GPU; between GPUs the destinations are peer mappings). Bit-exact, nothing
    # outside the block touched, vector and scalar paths, empty extents.
    for rows, cols, offset in ((300, 512, 256), (129, 77, 3), (0, 64, 0), (64, 0, 0)):
        width = 1024
        source = cuda.randn((rows, width), device='cuda:0')
        copies = [cuda.full((rows, width), float(i), device='cuda:0') for i in range(7)]
        ops.push_block(source[:, offset:offset + cols], [c[:, offset:offset + cols] for c in copies])
        for i, c in enumerate(copies):
            assert cuda.equal(c[:, offset:offset + cols], source[:, offset:offset + cols])
            assert bool((c[:, :offset] == i).all()) and bool((c[:, offset + cols:] == i).all())
    with pytest.raises(Exception, match='destinations'):
        ops.push_block(source, [cuda.empty_like(source) for _ in range(8)])
    with pytest.raises(ValueError):
        ops.push_block(source, [cuda.empty((3, 3), device='cuda:0')])


def test_gemm_edge_cases_and_errors(cuda):
    a, b = to_device(cuda, R.seeded_uniform(1, (64, 32))), to_device(cuda, R.seeded_uniform(2, (32, 48)))
    assert ops.gemm(a[:0], b, 'bf16x3').shape == (0, 48)
    assert ops.gemm(a, b[:, :0], 'bf16x3').shape == (64, 0)
    zero_k = ops.gemm(a[:, :0], b[:0], 'bf16x3')
    assert float(zero_k.abs().sum()) == 0.0
    with pytest.raises(ValueError):
        ops.gemm(a, b[:16], 'bf16x3')
    with pytest.raises(ValueError):
        ops.gemm(a, b, 'fp8')
    too_small = cuda.empty(2048, dtype=cuda.uint8, device='cuda:0')
    big_a, big_b = to_device(cuda, R.seeded_uniform(1, (1024, 1024))), to_device(cuda, R.seeded_uniform(2, (1024, 1024)))
    with pytest.raises(ValueError, match='workspace'):
        ops.gemm(big_a, big_b, 'bf16x3', workspace=too_small)
    assert ops.gemm(a, b, 'bf16x3', workspace=too_small).shape == (64, 48)   # tiny products need no workspace
    # special values propagate like the reference's arithmetic (inf stays inf, NaN poisons its row/column)
    special = R.seeded_uniform(3, (128, 64))
    special[5, 7] = np.inf
    special[9, 3] = np.nan
    other = np.abs(R.seeded_uniform(4, (64, 128))) + 0.5
    produced = ops.gemm(to_device(cuda, special), to_device(cuda, other), 'bf16x3').cpu().numpy()
    assert np.isnan(produced[9]).all() and np.isnan(produced[5]).all()   # inf - inf residual is NaN, as in the reference's split
    assert np.isfinite(produced[[0, 1, 2, 3, 4, 6, 7, 8]]).all()
    # the same through every kernel family and both modes, with NaNs of every payload in B as well (tf32's high part is
    # rounded with integer arithmetic that may turn such a NaN into a zero: the residual must still carry it)
    def poisoned(m, n, k, mode, variant):
        left, right = R.seeded_uniform(5, (m, k)), np.abs(R.seeded_uniform(6, (k, n))) + 0.5
        bits = right.view(np.uint32)
        bits[3, 1], bits[5, 2], bits[7, 4] = 0x7FFFFFFF, 0xFFFFFFFF, 0x7FC00000   # NaNs: all-ones payloads, canonical
        left[min(2, m - 1), 6] = np.inf
        ops.set_gemm_variant(variant)
        try:
            out = ops.gemm(to_device(cuda, left), to_device(cuda, right), mode).cpu().numpy()
        finally:
            ops.set_gemm_variant(0)
        ops.check_device_status()
        assert np.isnan(out[:, [1, 2, 4]]).all(), (m, n, k, mode, variant)
        assert np.isnan(out[min(2, m - 1)]).all(), (m, n, k, mode, variant)
        clean_rows = [r for r in range(m) if r != min(2, m - 1)]
        clean_columns = [c for c in range(n) if c not in (1, 2, 4)]
        assert np.isfinite(out[np.ix_(clean_rows, clean_columns)]).all(), (m, n, k, mode, variant)
    for mode in ('bf16x3', 'tf32x3'):
        poisoned(64, 48, 32, mode, 0)         # single-kernel form
        poisoned(16, 4096, 2048, mode, 10)    # streamed form for at most 16 rows
        poisoned(1, 2048, 2048, mode, 10)
        poisoned(512, 512, 256, mode, 1)      # split pass + tcgen05 tiles
        poisoned(2048, 1024, 512, mode, 7)    # stream kernel (split of A inside)


def test_gemm_column_blocks_equal_the_full_product(cuda):
    # the multi-GPU partition: a column block computed in place (leading dimensions kept) is bit-identical
    # (every block here is large enough for the tensor-core path, like the full product)
    from deuteron_b200 import sharding
    a, b = to_device(cuda, R.seeded_uniform(7, (1024, 1024))), to_device(cuda, R.seeded_uniform(11, (1024, 2048)))
    full = ops.gemm(a, b, 'bf16x3').clone()
    for world in (2, 4):
        parts = []
        for rank in range(world):
            local, (begin, end) = sharding.gemm_column_shard(a, b, rank, world)
            parts.append(local.clone())
            assert (begin, end) == sharding.column_blocks(2048, world)[rank]
        assert bool(cuda.equal(cuda.cat(parts, dim=1), full))
    into = cuda.zeros((1024, 2048), device='cuda:0')
    ops.gemm(a, b[:, 512:1024], 'bf16x3', out=into[:, 512:1024])
    assert bool(cuda.equal(into[:, 512:1024], full[:, 512:1024])) and float(into[:, :512].abs().sum()) == 0.0


def test_execute_on_host_buffers_matches_the_resident_path(cuda, runner):
    # small product: one launch; large product: the row-block pipeline (copies overlapped with products)
    for m, n, k in ((128, 128, 128), (4096, 1024, 2048)):
        graph, meta = schedules.matmul_example(m, n, k)
        compiled = compile_kernel(graph, meta, options=Options(contraction_precision='bf16x3'))
        left, right = runner.pinned((m, k), np.float32), runner.pinned((k, n), np.float32)
        left[:], right[:] = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
        result = runner.pinned((m, n), np.float32)
        for _ in range(2):   # the second call reuses the resident device buffers
            result[:] = 0
            produced = runner.execute(compiled, {'left': left, 'right': right}, {'result': result})['result']
            assert produced is result
            resident = ops.gemm(to_device(cuda, left), to_device(cuda, right), 'bf16x3').cpu().numpy()
            np.testing.assert_array_equal(produced, resident)
    unpinned = runner.execute(compiled, {'left': np.array(left), 'right': np.array(right)})['result']
    np.testing.assert_array_equal(unpinned, resident)
    graph, meta = schedules.vector_add_example(4096)
    x, y = R.seeded_normal(1, (4096,)), R.seeded_normal(2, (4096,))
    produced = runner.execute(compile_kernel(graph, meta), {'lhs': x, 'rhs': y})['sum']
    np.testing.assert_array_equal(produced, x + y)
    with pytest.raises(ValueError):
        runner.execute(compile_kernel(graph, meta), {'lhs': x[:-1], 'rhs': y})


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
@pytest.mark.parametrize('m,n,k', [(8192, 1024, 512), (8192, 2048, 256), (4096, 4096, 320), (8192, 1000, 200), (2300, 4100, 130),
                                   (8192, 8192, 192)])
def test_stream_kernel_equals_the_plain_tiles_bit_for_bit(cuda, mode, m, n, k):
    # cut bands of unequal widths (first three shapes: a table of tiles; ragged edges; the plain walk) and the split of
    # A inside the kernel change no bit of any output element
    a, b = to_device(cuda, R.seeded_uniform(7, (m, k))), to_device(cuda, R.seeded_uniform(11, (k, n)))
    ops.set_gemm_variant(1)
    try:
        plain = ops.gemm(a, b, mode).clone()
        ops.set_gemm_variant(7)
        streamed = ops.gemm(a, b, mode).clone()
        again = ops.gemm(a, b, mode)                            # counters and flags are cleared by every call
        kept_a = ops.gemm(a, b, mode, out=cuda.empty_like(plain), phase=3 | 4)   # A planes of the call before, B split again
        kept_b = ops.gemm(a, b, mode, out=cuda.empty_like(plain), phase=3 | 8)   # A split in the kernel, B planes kept
        only_products = ops.gemm(a, b, mode, out=cuda.empty_like(plain), phase=2)
    finally:
        ops.set_gemm_variant(0)
    ops.check_device_status()
    for produced in (streamed, again, kept_a, kept_b, only_products):
        assert bool(cuda.equal(produced, plain))
    automatic = ops.gemm(a, b, mode)
    ops.check_device_status()
    assert bool(cuda.equal(automatic, plain))


def test_execute_feeding_b_by_column_blocks_changes_no_bit(cuda, runner, monkeypatch):
    # the host-fed pipeline with B cut into column blocks (first block, A by row blocks, the other blocks against all
    # of A; strided copies both ways) and with the default (B whole, the last row block cut small)
    m, n, k = 4096, 2048, 2048
    graph, meta = schedules.matmul_example(m, n, k)
    compiled = compile_kernel(graph, meta, options=Options(contraction_precision='bf16x3'))
    left, right = runner.pinned((m, k), np.float32), runner.pinned((k, n), np.float32)
    left[:], right[:] = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
    resident = ops.gemm(to_device(cuda, left), to_device(cuda, right), 'bf16x3').cpu().numpy()
    for columns in (None, '1024,512,256,256', '768,1280'):
        if columns is None:
            monkeypatch.delenv('DTN_E2E_COLUMNS', raising=False)
        else:
            monkeypatch.setenv('DTN_E2E_COLUMNS', columns)
        result = runner.pinned((m, n), np.float32)
        result[:] = float('nan')
        produced = runner.execute(compiled, {'left': left, 'right': right}, {'result': result})['result']
        np.testing.assert_array_equal(produced, resident)


def test_execute_with_a_tall_left_operand_and_a_narrow_right_one(cuda, runner):
    # 8 row blocks of 1024 x 128 x 1024: each block alone is small enough for the single-kernel GEMM, which writes no
    # operand planes; the pipeline must still split B before the first block and multiply every block by those planes
    m, n, k = 8192, 128, 1024
    graph, meta = schedules.matmul_example(m, n, k)
    compiled = compile_kernel(graph, meta, options=Options(contraction_precision='bf16x3'))
    left, right = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
    poison = cuda.full((64 << 20,), float('nan'), device='cuda:0')   # whatever scratch comes next does not start clean
    del poison
    produced = runner.execute(compiled, {'left': left, 'right': right})['result']
    exact = left.astype(np.float64) @ right.astype(np.float64)
    assert R.max_relative_error(produced, exact) < 2e-5
    ops.set_gemm_variant(1)
    try:
        resident = ops.gemm(to_device(cuda, left), to_device(cuda, right), 'bf16x3').cpu().numpy()
    finally:
        ops.set_gemm_variant(0)
    np.testing.assert_array_equal(produced, resident)


def test_host_fed_sharded_product_on_one_rank_matches_the_resident_path(cuda, runner):
    # sharding.ShardedHostProduct with a world of one: the same walk as on several GPUs (B split once, row blocks of A
    # copied in, multiplied and copied out on four streams) without the exchange; the N-rank form runs over gloo in
    # tests/test_sharding_cpu.py and over NCCL in bench.py --gpus N
    from deuteron_b200 import sharding
    m, n, k = 4096, 1280, 1024
    compiled = compile_kernel(*schedules.matmul_example(m, n, k), options=Options(contraction_precision='bf16x3'))
    product = sharding.ShardedHostProduct(compiled, 0, 1, 'cuda:0', row_blocks=3)
    left, right = runner.pinned((m, k), np.float32), runner.pinned((k, n), np.float32)
    left[:], right[:] = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
    assert product.columns == (0, n) and product.owned_row_count == m and product.host_bytes() == (4 * (m * k + k * n), 4 * m * n)
    out = runner.pinned((m, n), np.float32)
    for _ in range(2):
        out[:] = 0
        assert product.execute(product.pack_rows(left), right, out) is out
        ops.set_gemm_variant(1)
        try:
            resident = ops.gemm(to_device(cuda, left), to_device(cuda, right), 'bf16x3').cpu().numpy()
        finally:
            ops.set_gemm_variant(0)
        np.testing.assert_array_equal(out, resident)
    ops.check_device_status()
    with pytest.raises(ValueError):
        product.execute(left[:-1], right, out)


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
@pytest.mark.parametrize('m,blocks', [(1536, 4), (2560, 4), (1000, 3)])
def test_row_blocks_of_unequal_heights_share_one_split_of_b(cuda, mode, m, blocks):
    # the walk of sharding.GatheredProduct: B split once (1|4), then every row block with 3|8 and the same workspace
    from deuteron_b200 import sharding
    n, k = 768, 640
    a, b = to_device(cuda, R.seeded_uniform(7, (m, k))), to_device(cuda, R.seeded_uniform(11, (k, n)))
    rows = sharding.row_blocks_for_overlap(m, blocks)
    assert len({r1 - r0 for r0, r1 in rows}) > 1 or m == 1000
    tallest = max(r1 - r0 for r0, r1 in rows)
    planes = cuda.full((ops.gemm_workspace_bytes(mode, tallest, n, k) + 1024,), 0xFF, dtype=cuda.uint8, device='cuda:0')
    out = cuda.zeros((m, n), device='cuda:0')
    r0, r1 = rows[0]
    ops.gemm(a[r0:r1], b, mode, out=out[r0:r1], workspace=planes, phase=1 | 4)
    for r0, r1 in rows:
        ops.gemm(a[r0:r1], b, mode, out=out[r0:r1], workspace=planes, phase=3 | 8)
    ops.set_gemm_variant(1)
    try:
        whole = ops.gemm(a, b, mode)
    finally:
        ops.set_gemm_variant(0)
    ops.check_device_status()
    assert bool(cuda.equal(out, whole))


@pytest.mark.parametrize('mode', ['bf16x3', 'tf32x3'])
def test_gemm_8192_properties(cuda, mode):
    n = 8192
    generator = cuda.Generator(device='cuda:0').manual_seed(7)
    a = cuda.rand((n, n), device='cuda:0', generator=generator) * 2 - 1
    b = cuda.rand((n, n), device='cuda:0', generator=generator) * 2 - 1
    c = ops.gemm(a, b, mode).clone()
    ops.check_device_status()
    rows = cuda.arange(0, n, n // 64, device='cuda:0')
    exact = a[rows].double() @ b.double()
    error = float(((c[rows].double() - exact).abs().max() / exact.abs().max()).item())
    steps = 3 * n // (16 if mode == 'bf16x3' else 8)
    assert error <= 1e-5 + steps * 2.0 ** -24, error
    # scaling an operand by a power of two commutes exactly with both splits and with every accumulation
    scaled = ops.gemm(a * 4.0, b * 0.5, mode)
    assert bool(cuda.equal(scaled, c * 2.0))
    # deterministic: a second run gives the same bits
    assert bool(cuda.equal(ops.gemm(a, b, mode), c))
    # identity on the right returns the compensated reconstruction hi + lo of A (exact to 2^-16 / 2^-21)
    eye = cuda.eye(n, device='cuda:0')
    back = ops.gemm(a[:256], eye, mode)
    assert float((back - a[:256]).abs().max()) <= (2.0 ** -16 if mode == 'bf16x3' else 2.0 ** -20)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------


def test_attention_example_error_level(runner, published):
    graph, meta = schedules.attention_example()
    compiled = compile_kernel(graph, meta)
    produced = runner.run_kernel(meta['kernels'][0], compiled, warmup=0, iters=1, samples=1)['outputs']['out']
    q, kt, v = R.seeded_normal(7, (3, 32)), R.seeded_normal(8, (32, 64)), R.seeded_normal(9, (64, 32))
    exact = R.attention_f64(q, kt, v)
    np.testing.assert_allclose(produced, exact, rtol=meta['rtol'], atol=meta['atol'])
    assert float(np.max(np.abs(produced - exact))) <= 2 * published['results']['attention']['max_absolute_errors']['out']


def test_all_key_groups_and_inplace_denominator(runner):
    # tests/test_attention.py:106-122
    for keys in range(32, 257, 32):
        outputs = []
        rows, depth, seed = 1 + keys // 32, 32 if keys % 64 else 64, keys + 7
        q, kt, v = R.seeded_normal(seed, (rows, depth)), R.seeded_normal(seed + 1, (depth, keys)), R.seeded_normal(seed + 2, (keys, 32))
        exact = R.attention_f64(q, kt, v)
        for alias in (False, True):
            graph, meta = schedules.attention_example(rows=rows, keys=keys, depth=depth, inplace_denominator=alias, seed=seed)
            produced = runner.run_kernel(meta['kernels'][0], compile_kernel(graph, meta), warmup=0, iters=1, samples=1)['outputs']['out']
            np.testing.assert_allclose(produced, exact, rtol=1e-3, atol=1e-4)
            outputs.append(produced)
        np.testing.assert_array_equal(outputs[0], outputs[1])


def test_attention_beyond_one_stage_and_wide_values(cuda):
    for rows, keys, depth, cols in ((5, 600, 48, 40), (2, 1000, 128, 128), (1, 1, 8, 3), (7, 257, 16, 256)):
        q, kt, v = R.seeded_normal(7, (rows, depth)), R.seeded_normal(8, (depth, keys)), R.seeded_normal(9, (keys, cols))
        scale = float(np.float32(1 / math.sqrt(depth)))
        produced = ops.attention(to_device(cuda, q), to_device(cuda, kt), to_device(cuda, v), scale).cpu().numpy()
        np.testing.assert_allclose(produced, R.attention_f64(q, kt, v), rtol=1e-3, atol=1e-4)
    with pytest.raises(NotImplementedError):
        ops.attention(to_device(cuda, q), to_device(cuda, kt), to_device(cuda, np.zeros((257, 300), np.float32)), 1.0)


# sequence lengths that are no multiple of the 256-query items, of the 128-key steps, or of anything (257: one key in
# the last step; 385: a query tile with one row; 1000; 1153 = 9 * 128 + 1)
GQA_CASES = [(1, 4, 2, 128, 128), (2, 4, 2, 300, 128), (1, 8, 8, 512, 128), (1, 2, 1, 64, 64), (1, 4, 1, 1000, 128),
             (1, 1, 1, 256, 128), (2, 4, 1, 1024, 128), (1, 8, 2, 768, 128), (2, 4, 2, 257, 128), (1, 4, 4, 385, 128),
             (2, 2, 1, 1153, 128)]


def gqa_error_bound(keys, tensor_core):
    """Max error relative to max|out|. FP32 kernel: rounding of ~keys FMAs (measured 1.1e-6 .. 1.5e-6).
    Tensor-core kernel: the probabilities carry 22 bits and the accumulator in tensor memory is updated
    2 * keys / 16 times, each update truncating to FP32 (at most 2^-24 of the running magnitude per update
    on average)."""
    return 3e-6 + (2 * keys / 16) * 2.0 ** -24 if tensor_core else 3e-6


@pytest.mark.parametrize('variant', [0, 1, 3, 7])   # automatic, all-FP32, tensor core with two warpgroups per tile (scores read twice / kept)
@pytest.mark.parametrize('storage', [np.float16, np.float32])
def test_gqa_attention_against_float64(cuda, storage, variant):
    ops.set_gqa_variant(variant)
    try:
        for batch, hq, hkv, s, d in GQA_CASES:
            ragged_ok = storage == np.float16 and d == 128 and s >= 256   # the kept-score form masks keys and clips rows
            eligible = ragged_ok if variant in (0, 7) else (ragged_ok and s % 256 == 0)
            if variant in (3, 7) and not eligible:
                continue
            scale = float(np.float32(1 / math.sqrt(d)))
            q = R.seeded_normal(7, (batch, hq, s, d), storage, scale)
            k = R.seeded_normal(8, (batch, hkv, s, d), storage, scale)
            v = R.seeded_normal(9, (batch, hkv, s, d), storage, scale)
            produced = ops.gqa_attention(to_device(cuda, q), to_device(cuda, k), to_device(cuda, v), scale).cpu().numpy()
            ops.check_device_status()
            exact = R.gqa_attention_f64(q, k, v, scale)
            np.testing.assert_allclose(produced, exact, rtol=1e-3, atol=1e-4)
            tensor_core = variant != 1 and eligible
            assert R.max_relative_error(produced, exact) <= gqa_error_bound(s, tensor_core), (batch, hq, hkv, s, d)
    finally:
        ops.set_gqa_variant(0)


def test_gqa_through_the_compile_and_launch_surface(cuda, runner):
    # scheduled IR with [batch, head, position, depth] buffers -> the native grouped-query kernels
    for storage, s, d in (('f16', 512, 128), ('f32', 300, 64)):
        graph, meta = schedules.gqa_attention_example(2, 4, 2, s, d, storage)
        compiled = compile_kernel(graph, meta, arch='sm_100a')
        assert compiled.plan.kind == 'gqa'
        scale = float(np.float32(1 / math.sqrt(d)))
        dtype = np.float16 if storage == 'f16' else np.float32
        q, k, v = (R.seeded_normal(7 + i, shape, dtype) for i, shape in enumerate(((2, 4, s, d), (2, 2, s, d), (2, 2, s, d))))
        result = runner.run_kernel(meta['kernels'][0], compiled, warmup=1, iters=2, samples=1)
        exact = R.gqa_attention_f64(q, k, v, scale)
        np.testing.assert_allclose(result['outputs']['out'], exact, rtol=meta['rtol'], atol=meta['atol'])
        assert R.max_relative_error(result['outputs']['out'], exact) <= gqa_error_bound(s, storage == 'f16')
        hosted = runner.execute(compiled, {'q': q, 'k': k, 'v': v})['out']
        np.testing.assert_array_equal(hosted, result['outputs']['out'])


def test_gqa_cta_pair_kernel_equals_the_one_cta_kernel(cuda):
    """The CTA-pair kernel (one 256-row instruction per product, each CTA holding half of every K and V tile) runs the
    same softmax code on the same products: its output is bit-identical to the one-CTA kernel's, for both warpgroup
    splits, on whole launches and on group ranges; shapes it does not cover are refused."""
    generator = cuda.Generator(device='cuda:0').manual_seed(5)
    batch, hq, hkv, s, d = 2, 6, 2, 1536, 128
    q = (cuda.randn((batch, hq, s, d), device='cuda:0', generator=generator) / d ** 0.5).half()
    k = (cuda.randn((batch, hkv, s, d), device='cuda:0', generator=generator) / d ** 0.5).half()
    v = (cuda.randn((batch, hkv, s, d), device='cuda:0', generator=generator) / d ** 0.5).half()
    try:
        results = {}
        for variant in (2, 3, 4, 5):
            ops.set_gqa_variant(variant)
            results[variant] = ops.gqa_attention(q, k, v, d ** -0.5).clone()
            ops.check_device_status()
        assert bool(cuda.equal(results[4], results[2])) and bool(cuda.equal(results[5], results[3]))
        # all sixteen softmax warps on one tile at a time: the same products, row sums added in another order
        ops.set_gqa_variant(6)
        alternating = ops.gqa_attention(q, k, v, d ** -0.5)
        ops.check_device_status()
        assert float((alternating - results[3]).abs().max()) <= 5e-6 * float(results[3].abs().max())
        ops.set_gqa_variant(5)
        partial = cuda.zeros_like(results[5])
        ops.gqa_attention(q, k, v, d ** -0.5, out=partial, groups=(1, 3))
        per_group = hq // hkv
        flat, whole = partial.view(batch * hkv, per_group, s, d), results[5].view(batch * hkv, per_group, s, d)
        assert bool(cuda.equal(flat[1:3], whole[1:3])) and float(flat[0].abs().sum()) == 0.0 and float(flat[3].abs().sum()) == 0.0
        with pytest.raises(NotImplementedError, match='multiple of 512'):
            ops.gqa_attention(q[:, :, :768].contiguous(), k[:, :, :768].contiguous(), v[:, :, :768].contiguous(), d ** -0.5)
    finally:
        ops.set_gqa_variant(0)


def test_gqa_group_ranges_partition_the_output(cuda):
    from deuteron_b200 import sharding
    batch, hq, hkv, s, d = 2, 8, 2, 256, 128
    scale = float(np.float32(1 / math.sqrt(d)))
    q = to_device(cuda, R.seeded_normal(7, (batch, hq, s, d), np.float16, scale))
    k = to_device(cuda, R.seeded_normal(8, (batch, hkv, s, d), np.float16, scale))
    v = to_device(cuda, R.seeded_normal(9, (batch, hkv, s, d), np.float16, scale))
    full = ops.gqa_attention(q, k, v, scale).clone()
    for world in (2, 4):
        assembled = cuda.full_like(full, float('nan'))
        for rank in range(world):
            sharding.gqa_group_shard(q, k, v, scale, rank, world, out=assembled)
        assert bool(cuda.equal(assembled, full))
    assert ops.gqa_attention(q, k, v, scale, groups=(1, 1)) is not None
    with pytest.raises(ValueError):
        ops.gqa_attention(q, k, v, scale, groups=(0, 5))
    with pytest.raises(ValueError):
        ops.gqa_attention(q, k[:, :1].repeat(1, 3, 1, 1), v[:, :1].repeat(1, 3, 1, 1), scale)


def test_gqa_full_size_properties(cuda):
    # batch 4, 32 query / 8 kv heads, head_dim 128, 4096 keys: sampled rows against float64, plus softmax identities
    batch, hq, hkv, s, d = 4, 32, 8, 4096, 128
    scale = float(np.float32(1 / math.sqrt(d)))
    generator = cuda.Generator(device='cuda:0').manual_seed(7)
    q = (cuda.randn((batch, hq, s, d), device='cuda:0', generator=generator) * scale).half()
    k = (cuda.randn((batch, hkv, s, d), device='cuda:0', generator=generator) * scale).half()
    v = (cuda.randn((batch, hkv, s, d), device='cuda:0', generator=generator) * scale).half()
    out = ops.gqa_attention(q, k, v, scale)
    ops.check_device_status()
    rows = [0, 1, 777, 2048, 4095]
    for b, h in ((0, 0), (1, 13), (3, 31)):
        exact = R.attention_f64(q[b, h, rows].cpu().numpy(), k[b, h // 4].cpu().numpy().astype(np.float64).T, v[b, h // 4].cpu().numpy(), scale)
        produced = out[b, h, rows].cpu().numpy()
        np.testing.assert_allclose(produced, exact, rtol=1e-3, atol=1e-4)
        # the outputs are means of 4096 small values of either sign (|out| ~ |v| / 64): bound the error by the
        # accumulated magnitude max|v| rather than by the cancelled result
        assert float(np.max(np.abs(produced - exact))) <= gqa_error_bound(s, True) * float(v.abs().max())
    # rows of the softmax sum to one: constant values come back unchanged
    ones = ops.gqa_attention(q, k, cuda.ones_like(v), scale)
    # (every update of the tensor-memory accumulator truncates, so a sum of equal-signed terms is biased low by up
    # to 2^-24 per update; the all-FP32 kernel stays within 2e-6 here)
    assert float((ones - 1).abs().max()) <= gqa_error_bound(s, True)
    # outputs are convex combinations of the values
    assert float(out.max()) <= float(v.float().max()) + 1e-6 and float(out.min()) >= float(v.float().min()) - 1e-6


def test_native_errors_are_python_exceptions(cuda):
    with pytest.raises(ValueError):
        native.call('dtn_row_reduce_f32', 9, 1, 1, 1, 1, 1, None)
    with pytest.raises(ValueError):
        ops.row_reduce('sum', cuda.zeros(4, device='cuda:0'))
    with pytest.raises(ValueError):
        ops.add(cuda.zeros(4), cuda.zeros(4))
    assert native.device_status(0) == 0


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(cuda):
    # Failure detection without a fault: a kernel waits about a millisecond on a barrier nothing completes,
    # records a status code and returns; the host sees it as DeviceWaitError, the word is cleared, and the
    # next kernel on the same context runs normally.
    stream = cuda.cuda.current_stream().cuda_stream
    assert native.device_status(stream) == 0
    native.call('dtn_selftest_wait_timeout', 2_000_000, stream)
    with pytest.raises(native.DeviceWaitError, match='self-test'):
        native.raise_on_device_status(stream)
    assert native.device_status(stream) == 0
    a, b = to_device(cuda, R.seeded_uniform(7, (256, 256))), to_device(cuda, R.seeded_uniform(11, (256, 256)))
    ops.set_gemm_variant(1)
    try:
        produced = ops.gemm(a, b, 'bf16x3')
        ops.check_device_status()
    finally:
        ops.set_gemm_variant(0)
    assert R.max_relative_error(produced.cpu().numpy(), R.gemm_f64(a.cpu().numpy(), b.cpu().numpy())) < 1e-5
    with pytest.raises(ValueError):
        native.call('dtn_selftest_wait_timeout', 0, stream)
