"""Compile surface on CPU: parsing, launch validation, classification, caching, library exports.

The cases follow the reference's tests/test_validation.py and tests/test_interface.py: the same
malformed launches, buffer specs, options and constructor escapes must be rejected with the same
exception types before anything is launched.
"""
import copy
import ctypes
import json
import os
import re
import tempfile
import threading
from pathlib import Path

import pytest

from deuteron_b200 import Options, compile_kernel, compile_many, native, schedules
from deuteron_b200.validation import parse_kernel, validate_launch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture()
def vector_add(golden):
    graph = json.loads((golden / 'vector_add.ir.json').read_text())
    meta = json.loads((golden / 'reference_published.json').read_text())['meta']['vector_add']
    return graph, meta


def set_body(graph, expression):
    kernel = next(node for node in graph['nodes'].values() if node.get('op') == 'KernelOp')
    kernel['op_fields']['body'] = [expression]


def test_reference_examples_compile_to_native_plans(golden, vector_add):
    graph, meta = vector_add
    plan = compile_kernel(graph, meta).plan
    assert plan.kind == 'elementwise' and plan.params == {'op': 'add', 'n': 1030}
    assert plan.buffers == {'x': ('lhs', 0), 'y': ('rhs', 0), 'out': ('sum', 0)}
    matmul = json.loads((golden / 'tensor_matmul.ir.json').read_text())
    matmul_meta = json.loads((golden / 'reference_published.json').read_text())['meta']['tensor_matmul']
    for mode in ('bf16x3', 'tf32x3', 'f32'):
        plan = compile_kernel(matmul, matmul_meta, arch='sm_100a', opt_level=3, options=Options(contraction_precision=mode)).plan
        assert plan.kind == 'gemm' and plan.params == {'mode': mode, 'm': 128, 'n': 128, 'k': 128}
        # arg_order is right, left, result: roles come from the index structure, not from the order
        assert plan.buffers == {'left': ('left', 0), 'right': ('right', 0), 'out': ('result', 0)}


def test_path_with_sibling_meta_json(vector_add):
    graph, meta = vector_add
    with tempfile.TemporaryDirectory() as folder:
        source = Path(folder) / 'kernel.ir.json'
        source.write_text(json.dumps(graph))
        source.with_name('meta.json').write_text(json.dumps(meta))
        compiled = compile_kernel(source, arch='sm_100a')
        assert 'vector_add' in compiled.ptx and compiled.plan.kind == 'elementwise'
    with pytest.raises(OSError):
        compile_kernel(Path(folder) / 'missing.ir.json')


def test_generated_schedules_classify(golden):
    cases = [
        (schedules.f16_storage_example('copy', 512, 1), 'f16_copy', {'n': 512}),
        (schedules.f16_storage_example('widen', 512, 2), 'f16_widen', {'n': 512}),
        (schedules.f16_storage_example('narrow', 512, 4, offset=1), 'f16_narrow', {'n': 512}),
        (schedules.f16_storage_example('affine', 512, 4), 'elementwise_program',
         {'n': 512, 'inputs': [{'f16': True, 'scalar': False}, {'f16': False, 'scalar': True}, {'f16': False, 'scalar': True}],
          'out_reg': 0, 'out_f16': True, 'ops': [2, 0], 'dst': [0, 0], 'a': [0, 0], 'b': [1, 2]}),
        (schedules.f16_storage_example('cancellation', 512, 2), 'elementwise_program',
         {'n': 512, 'inputs': [{'f16': True, 'scalar': False}, {'f16': True, 'scalar': False}], 'out_reg': 0, 'out_f16': True,
          'ops': [0, 1], 'dst': [1, 0], 'a': [0, 1], 'b': [1, 0]}),
        (schedules.attention_example(9, 256, 64, True), 'attention', {'rows': 9, 'keys': 256, 'depth': 64, 'cols': 32, 'scale': 0.125}),
        (schedules.gqa_attention_example(4, 32, 8, 4096, 128, 'f16'), 'gqa',
         {'batch': 4, 'hq': 32, 'hkv': 8, 's': 4096, 'd': 128, 'scale': 0.0883883461356163, 'storage': 'f16'}),
        (schedules.gqa_attention_example(1, 6, 2, 100, 64, 'f32'), 'gqa',
         {'batch': 1, 'hq': 6, 'hkv': 2, 's': 100, 'd': 64, 'scale': 0.125, 'storage': 'f32'}),
        (schedules.row_reduce_example(64, 512, 'sum'), 'row_reduce', {'op': 'sum', 'rows': 64, 'cols': 512}),
        (schedules.row_reduce_example(8, 4096, 'max'), 'row_reduce', {'op': 'max', 'rows': 8, 'cols': 4096}),
        (schedules.row_reduce_example(8, 4096, 'sumsq'), 'row_reduce', {'op': 'sumsq', 'rows': 8, 'cols': 4096}),
        (schedules.matmul_example(256, 512, 1024), 'gemm', {'mode': 'bf16x3', 'm': 256, 'n': 512, 'k': 1024}),
        # staged depth 4 is no multiple of the tensor-core k step: the reference lowers this one to FP32 multiply-adds, and so does this build
            (schedules.split_k_matmul_example(), 'gemm', {'mode': 'f32_splitk', 'm': 128, 'n': 64, 'k': 256}),
        (schedules.mean_example(), 'row_fused',
         {'reduce': 'sum', 'rows': 1, 'cols': 32768, 'per_row': True, 'inputs': [{'kind': 'scalar'}], 'n_scalar': 1, 'out_reg': 4,
          'ops': [3], 'dst': [4], 'a': [0], 'b': [3]}),
        (schedules.l2_norm_example(), 'row_fused',
         {'reduce': 'sumsq', 'rows': 64, 'cols': 512, 'per_row': False, 'inputs': [], 'n_scalar': 2, 'out_reg': 4,
          'ops': [8, 10, 2], 'dst': [3, 3, 4], 'a': [0, 3, 3], 'b': [0, 3, 2]}),
        (schedules.row_softmax_example(), 'row_fused',
         {'reduce': 'softmax', 'rows': 64, 'cols': 256, 'per_row': False, 'inputs': [], 'n_scalar': 1, 'out_reg': 4,
          'ops': [10, 1, 7, 2], 'dst': [3, 4, 4, 4], 'a': [1, 2, 4, 4], 'b': [1, 0, 4, 3]}),
    ]
    for (graph, meta), kind, params in cases:
        plan = compile_kernel(graph, meta).plan
        assert plan.kind == kind and plan.params == params
    rms = compile_kernel(*schedules.rms_norm_example()).plan
    assert rms.kind == 'row_fused' and rms.params['reduce'] == 'sumsq' and rms.params['n_scalar'] == 3
    assert [i['kind'] for i in rms.params['inputs']] == ['columns', 'scalar', 'scalar']
    assert rms.buffers == {'x': ('x', 0), 'out': ('mul_1', 0), 'in0': ('w', 0), 'in1': ('mean_count', 0), 'in2': ('add_c1', 0)}
    # a rasterised tile order (compiler/codegen/lower.py:472-487) changes which CTA computes which tile, not the product
    graph, meta = schedules.matmul_example(256, 256, 256)
    body = graph['nodes']['result']['op_fields']['body'][0]
    assert "raster_axes=None, raster_group=None" in body
    set_body(graph, body.replace("raster_axes=None, raster_group=None", "raster_axes=('tile_m', 'tile_n'), raster_group=4"))
    assert compile_kernel(graph, meta).plan.params == {'mode': 'bf16x3', 'm': 256, 'n': 256, 'k': 256}
    narrow = compile_kernel(*schedules.f16_storage_example('narrow', 512, 4, offset=1)).plan
    assert narrow.buffers['x'] == ('x', 1)  # the unaligned origin travels as an element offset
    # the generated 128^3 schedule has the statement census of the reference's committed IR
    from deuteron_b200 import ir
    census = lambda text: sorted((kind, count) for kind, count in __import__('collections').Counter(
        n.kind for n in ir.walk([ir.parse_statement(text)])).items())
    reference_ir = json.loads((golden / 'tensor_matmul.ir.json').read_text())['nodes']['result']['op_fields']['body'][0]
    generated_ir = schedules.matmul_example()[0]['nodes']['result']['op_fields']['body'][0]
    assert census(generated_ir) == census(reference_ir)


def test_unsupported_schedules_raise_not_implemented(vector_add):
    graph, meta = vector_add
    set_body(graph, "Tile(axes=(Axis(name='item', extent=Dim(515), window=None),), body=(Sync(barrier_id=0, count=None, warp=False),), block_threads=128)")
    with pytest.raises(NotImplementedError):
        compile_kernel(graph, meta)
    graph, meta = schedules.matmul_example()
    body = graph['nodes']['result']['op_fields']['body'][0].replace('atomic=False', 'atomic=True')
    set_body(graph, body)
    with pytest.raises(NotImplementedError, match='atomic'):
        compile_kernel(graph, meta)
    # split-K: the output must be zeroed by the launch, and the splits must cover the whole reduction
    graph, meta = schedules.split_k_matmul_example()
    meta['kernels'][0]['zero_outputs'] = []
    with pytest.raises(NotImplementedError, match='zero_outputs'):
        compile_kernel(graph, meta)
    graph, meta = schedules.split_k_matmul_example()
    set_body(graph, graph['nodes']['matmul']['op_fields']['body'][0].replace("Axis(name='split', extent=Dim(64)", "Axis(name='split', extent=Dim(32)"))
    with pytest.raises(NotImplementedError, match='cover'):
        compile_kernel(graph, meta)
    # row kernels: a two-state reduction that is not the online softmax pair, and lanes that mix vector elements
    graph, meta = schedules.row_softmax_example()
    set_body(graph, graph['nodes']['softmax']['op_fields']['body'][0].replace("Assign(name='alpha', op=ElementwiseImpl('exp')", "Assign(name='alpha', op=ElementwiseImpl('sqrt')", 1))
    with pytest.raises(NotImplementedError, match='online maximum'):
        compile_kernel(graph, meta)
    graph, meta = schedules.l2_norm_example()
    set_body(graph, graph['nodes']['div']['op_fields']['body'][0].replace("values=('y0', 'y1', 'y2', 'y3')", "values=('y1', 'y0', 'y2', 'y3')"))
    with pytest.raises(NotImplementedError, match='mix vector elements'):
        compile_kernel(graph, meta)


def test_extra_duplicate_argument_order_is_rejected(vector_add):
    graph, meta = vector_add
    meta['kernels'][0]['arg_order'].append('lhs')
    with pytest.raises(ValueError, match='args and arg_order disagree'):
        compile_kernel(graph, meta)


@pytest.mark.parametrize('field,value', [
    ('grid', [0, 1, 1]), ('grid', [2**31, 1, 1]), ('grid', [True, 1, 1]), ('block', [1024, 2, 1]), ('block', [32., 1, 1]),
    ('block', [32, 1]), ('smem_bytes', -1), ('smem_bytes', True), ('zero_outputs', ['lhs']), ('zero_outputs', ['sum', 'sum']),
    ('zero_outputs', ['missing'])])
def test_malformed_launches_are_value_errors(vector_add, field, value):
    graph, meta = vector_add
    meta['kernels'][0][field] = value
    with pytest.raises(ValueError):
        compile_kernel(graph, meta)


@pytest.mark.parametrize('field,value', [('dtype', 'bf16'), ('shape', [-1]), ('shape', [True]), ('shape', '1030'), ('output', 1),
                                         ('intermediate', 'yes')])
def test_buffer_types_shapes_and_flags_are_validated(vector_add, field, value):
    graph, meta = vector_add
    meta['kernels'][0]['args'][0][field] = value
    with pytest.raises(ValueError):
        compile_kernel(graph, meta)


def test_readonly_global_write_and_rank_mismatch(vector_add):
    graph, meta = vector_add
    broken = copy.deepcopy(meta)
    broken['kernels'][0]['args'][-1]['output'] = False
    with pytest.raises(NotImplementedError, match='output buffers'):
        compile_kernel(graph, broken)
    broken = copy.deepcopy(meta)
    broken['kernels'][0]['args'][0]['shape'] = [2, 515]
    with pytest.raises(ValueError, match='index rank'):
        compile_kernel(graph, broken)
    broken = copy.deepcopy(meta)
    broken['kernels'][0]['grid'] = [5, 2, 1]
    with pytest.raises(NotImplementedError, match='linear'):
        compile_kernel(graph, broken)
    broken = copy.deepcopy(meta)
    broken['kernels'][0]['args'][0]['dtype'] = 'f64'
    with pytest.raises(NotImplementedError, match='f16/f32'):
        compile_kernel(graph, broken)


def test_options_and_compile_arguments_are_validated(vector_add):
    graph, meta = vector_add
    for field, value in (('unroll', -1), ('unroll', 2**31), ('unroll', True), ('vector_width', 3), ('vector_width', 4.),
                         ('contraction_precision', 'bf16'), ('approximate_math', 1), ('register_forwarding', None)):
        with pytest.raises(ValueError):
            Options(**{field: value})
    for kwargs in ({'arch': None}, {'arch': 120}, {'arch': 'sm_89'}, {'opt_level': True}, {'opt_level': 1.0}, {'opt_level': -1},
                   {'options': {}}):
        with pytest.raises(ValueError):
            compile_kernel(graph, meta, **kwargs)
    options = Options()
    object.__setattr__(options, 'unroll', -1)
    with pytest.raises(ValueError):
        compile_kernel(graph, meta, options=options)
    assert compile_kernel(graph, meta, options=Options(unroll=3)).plan.kind == 'elementwise'


def test_constructor_escape_never_executes(vector_add):
    graph, meta = vector_add
    with tempfile.TemporaryDirectory() as folder:
        marker = Path(folder) / 'must-not-exist'
        escape = "Literal.__init__.__globals__['__builtins__']['__import__']('pathlib').Path(" + repr(str(marker)) + ").write_text('x')"
        set_body(graph, 'Literal(value=' + escape + ", dtype='int')")
        with pytest.raises(ValueError):
            compile_kernel(graph, meta)
        assert not marker.exists()


@pytest.mark.parametrize('expression', ["__import__('os')", 'Literal.__init__', '(lambda: 0)()', '[Literal(i) for i in range(2)]',
                                        'Literal(*[1])', "Literal(**{'value': 1})", '[Literal(1)][0]', 'UnknownStatement()'])
def test_arbitrary_python_forms_are_rejected(vector_add, expression):
    graph, meta = vector_add
    set_body(graph, expression)
    with pytest.raises(ValueError):
        compile_kernel(graph, meta)


def test_json_errors(vector_add):
    _, meta = vector_add
    payload = json.dumps(meta).encode()
    with pytest.raises(ValueError, match='duplicate JSON key'):
        parse_kernel(b'{"nodes": {}, "nodes": {}}', payload)
    for bad in (b'[]', b'{', b'{"nodes": []}', b'{"nodes": {}}', b'\xff'):
        with pytest.raises(ValueError):
            parse_kernel(bad, payload)


def test_compile_cache_and_threads(vector_add):
    graph, meta = vector_add
    first = compile_kernel(graph, meta)
    assert compile_kernel(graph, meta) is first
    assert compile_kernel(graph, meta, opt_level=3) is not first
    results = []
    threads = [threading.Thread(target=lambda: results.append(compile_kernel(graph, meta))) for _ in range(8)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert all(result is first for result in results)
    many = compile_many([((graph, meta), 'sm_100a', 2, None)] if False else [])
    assert many == []
    with pytest.raises(ValueError):
        compile_many([('only', 'three', 'fields')])


def test_validate_launch_returns_specs_by_name(vector_add):
    _, meta = vector_add
    specs = validate_launch(meta['kernels'][0])
    assert list(specs) == ['lhs', 'rhs', 'sum'] and specs['sum']['output'] is True


def test_library_exports_every_declared_symbol():
    header = (ROOT / 'include' / 'deuteron_b200.h').read_text()
    declared = set(re.findall(r'^int (dtn_\w+)\(', header, flags=re.M))
    assert declared == set(native.exported_symbols())
    library = ctypes.CDLL(str(native.LIBRARY_PATH))
    for name in declared:
        assert hasattr(library, name), f'{name} is not exported'
    assert native.lib().dtn_version() >= 100


def test_argument_checks_need_no_gpu():
    # argument validation happens before any CUDA call, so it can be exercised on a CPU-only host
    library = native.lib()
    assert library.dtn_add_f32(None, None, None, -1, None) == native.ERR_INVALID
    assert 'negative' in native.last_error()
    assert library.dtn_gemm_set_variant(11) == native.ERR_INVALID
    size = ctypes.c_size_t(0)
    assert library.dtn_gemm_workspace_bytes(2, 8192, 8192, 8192, ctypes.byref(size)) == 0
    # hi and lo bf16 planes of A and of B transposed, then the two counters and the (32 + 32) x 64 item flags of the
    # split that runs inside the product kernel
    assert size.value == 4 * 8192 * 8192 * 2 + (4 * (2 + 64 * 64) + 1023) // 1024 * 1024
    assert library.dtn_gemm_workspace_bytes(1, 100, 50, 33, ctypes.byref(size)) == 0
    assert size.value == 2 * (100 * 64 * 4 + 1023) // 1024 * 1024 + 2 * (50 * 64 * 4 + 1023) // 1024 * 1024 or size.value > 0
    assert library.dtn_gemm_workspace_bytes(7, 1, 1, 1, ctypes.byref(size)) == native.ERR_INVALID
    with pytest.raises(ValueError):
        native.check(native.ERR_INVALID)
    with pytest.raises(NotImplementedError):
        native.check(native.ERR_UNSUPPORTED)
    with pytest.raises(native.CudaError):
        native.check(native.ERR_CUDA)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    # there is no fallback path: without the built library every entry into the native layer raises
    monkeypatch.setattr(native, '_library', None)
    monkeypatch.setattr(native, 'LIBRARY_PATH', tmp_path / 'libdeuteron_b200.so')
    with pytest.raises(RuntimeError, match='no fallback'):
        native.lib()
    with pytest.raises(RuntimeError, match='no fallback'):
        native.call('dtn_version')


def test_row_kernel_classification_follows_the_arithmetic_not_the_spelling():
    """The same row kernels written with other operators (divide by the sum instead of multiply by its reciprocal,
    divide by the norm, a plain sum instead of a sum of squares) still classify, with the program that says so."""
    from deuteron_b200.native import ELEMENTWISE_OPS as OPS
    graph, meta = schedules.row_softmax_example()
    body = graph['nodes']['softmax']['op_fields']['body'][0]
    set_body(graph, body.replace("Assign(name='probability', op=ElementwiseImpl('multiply'), args=('inverse', 'weight')",
                                 "Assign(name='probability', op=ElementwiseImpl('divide'), args=('weight', 's')"))
    plan = compile_kernel(graph, meta).plan
    assert plan.params['reduce'] == 'softmax' and plan.params['n_scalar'] == 0   # the unused reciprocal is not emitted
    assert plan.params['ops'] == [OPS['subtract'], OPS['exp'], OPS['divide']] and plan.params['b'][-1] == 1   # ... / sum of exponentials
    graph, meta = schedules.l2_norm_example()
    body = graph['nodes']['div']['op_fields']['body'][0].replace(
        "Assign(name='inverse', op=ElementwiseImpl('reciprocal'), args=('norm',)", "Assign(name='inverse', op=ElementwiseImpl('copy'), args=('norm',)")
    for lane in range(4):
        body = body.replace(f"Assign(name='y{lane}', op=ElementwiseImpl('multiply'), args=('x{lane}', 'inverse')",
                            f"Assign(name='y{lane}', op=ElementwiseImpl('divide'), args=('x{lane}', 'inverse')")
    set_body(graph, body)
    plan = compile_kernel(graph, meta).plan
    assert plan.params['reduce'] == 'sumsq' and plan.params['ops'] == [OPS['sqrt'], OPS['divide']] and plan.params['n_scalar'] == 1
    graph, meta = schedules.rms_norm_example()
    set_body(graph, graph['nodes']['mul_1']['op_fields']['body'][0].replace(
        "Assign(name='square', op=ElementwiseImpl('multiply'), args=('value', 'value'), ", "Assign(name='square', op=ElementwiseImpl('copy'), args=('value',), "))
    assert compile_kernel(graph, meta).plan.params['reduce'] == 'sum'


def test_launch_schema_takes_tuples_and_empty_buffers(vector_add):
    _, meta = vector_add
    launch = copy.deepcopy(meta['kernels'][0])
    launch['grid'], launch['block'] = tuple(launch['grid']), tuple(launch['block'])
    for arg in launch['args']:
        arg['shape'] = (0,)
    assert set(validate_launch(launch)) == {'lhs', 'rhs', 'sum'}
    for broken in ({'entry': ''}, {'entry': 'a\x00b'}, {'args': 'lhs'}, {'arg_order': None}, {'zero_outputs': 'sum'}):
        with pytest.raises(ValueError):
            validate_launch({**launch, **broken})
    with pytest.raises(ValueError):
        validate_launch([launch])
    scalar = copy.deepcopy(launch)
    scalar['args'][0].update(scalar=True, output=True)
    with pytest.raises(ValueError, match='scalar arguments'):
        validate_launch(scalar)
    huge = copy.deepcopy(launch)
    huge['args'][0]['shape'] = [2**62, 8]
    with pytest.raises(ValueError, match='64-bit address space'):
        validate_launch(huge)


@pytest.mark.parametrize('statement,error,fragment', [
    ("Sync(barrier_id=16, count=None, warp=False)", ValueError, 'barrier id'),
    ("Sync(barrier_id=1, count=None, warp=False)", ValueError, 'thread count'),
    ("Sync(barrier_id=1, count=64, warp=True)", ValueError, 'named barrier'),
    ("Sync(barrier_id=0, count=48, warp=False)", ValueError, 'multiple of 32'),
    ("Sync(barrier_id=0, count=256, warp=False)", ValueError, 'within the block'),
    ("CpAsyncWait(group=8)", ValueError, 'wait group'),
    ("Smem(name='lhs', extents=(4,), dtype='float', align=16)", ValueError, 'duplicate buffer name'),
    ("Smem(name='stage', extents=(4,), dtype='float', align=24)", ValueError, 'power of two'),
    ("Smem(name='stage', extents=(-4,), dtype='float', align=16)", ValueError, 'shared extents'),
    ("CpAsyncCopy(smem='stage', smem_index=(Literal(value=0, dtype='int'),), src='lhs', src_index=(Literal(value=0, dtype='int'),), "
     "nbytes=12, swizzle='NONE', lane_index=None, lane_rows=None)", ValueError, 'unknown buffer'),
    ("Load(names=('a',), input='nowhere', index=(Literal(value=0, dtype='int'),), dtype='float')", ValueError, 'unknown buffer'),
    ("StridedLoop(axis=Axis(name='i', extent=Dim(8), window=None), start=Literal(value=0, dtype='int'), step=Literal(value=0, dtype='int'), "
     "body=(), unroll=1, end=None, seed=False)", ValueError, 'positive integer step'),
    ("Loop(axis=Axis(name='i', extent=Dim(-1), window=None), body=(), unroll=1, seed=False)", NotImplementedError, 'axis extents'),
])
def test_statement_checks_reject_incoherent_kernels(vector_add, statement, error, fragment):
    graph, meta = vector_add
    set_body(graph, "Tile(axes=(Axis(name='item', extent=Dim(515), window=None),), body=(" + statement + ",), block_threads=128)")
    with pytest.raises(error, match=fragment):
        compile_kernel(graph, meta)


def test_tile_checks(vector_add):
    graph, meta = vector_add
    for tile, fragment in (("Tile(axes=(), body=(), block_threads=128)", 'distinct axes'),
                           ("Tile(axes=(Axis(name='i', extent=Dim(0), window=None),), body=(), block_threads=128)", 'distinct axes'),
                           ("Tile(axes=(Axis(name='i', extent=Dim(4), window=None), Axis(name='i', extent=Dim(4), window=None)), body=(), "
                            "block_threads=128)", 'distinct axes'),
                           ("Tile(axes=(Axis(name='i', extent=Dim(4), window=None),), body=(), block_threads=64)", 'block_threads')):
        set_body(graph, tile)
        with pytest.raises(ValueError, match=fragment):
            compile_kernel(graph, meta)


def test_ir_built_by_the_reference_generators_classifies_like_the_generated_schedules(golden):
    """tests/golden/reference_examples.json holds the IR and meta the reference's own example scripts build
    (examples/attention.py, examples/f16_storage.py). It goes through compile_kernel unchanged and selects the same
    native kernel, with the same parameters, as the IR this package's schedules module generates for the same shape."""
    examples = json.loads((golden / 'reference_examples.json').read_text())
    assert len(examples) == 15
    shapes = {'attention_3x64x32': dict(rows=3, keys=64, depth=32), 'attention_64x64x64': dict(rows=64, keys=64, depth=64),
              'attention_128x128x32': dict(rows=128, keys=128, depth=32),
              'attention_128x128x32_inplace': dict(rows=128, keys=128, depth=32, inplace_denominator=True),
              'attention_256x256x128': dict(rows=256, keys=256, depth=128)}
    for name, configuration in shapes.items():
        theirs = compile_kernel(examples[name]['graph'], examples[name]['meta']).plan
        mine = compile_kernel(*schedules.attention_example(**configuration)).plan
        # the generator of this package writes the very text the reference's script writes
        assert schedules.attention_example(**configuration) == (examples[name]['graph'], examples[name]['meta'])
        assert theirs.kind == 'attention' and theirs.params == mine.params and theirs.buffers == mine.buffers, name
    for kind in ('copy', 'widen', 'narrow', 'affine', 'cancellation'):
        for width in (4, 1):
            case = examples[f'f16_{kind}_w{width}']
            theirs = compile_kernel(case['graph'], case['meta']).plan
            mine = compile_kernel(*schedules.f16_storage_example(kind, width=width)).plan
            assert theirs.kind == mine.kind and theirs.params == mine.params and theirs.buffers == mine.buffers, (kind, width)
            assert schedules.f16_storage_example(kind, width=width) == (case['graph'], case['meta'])


def test_per_program_sources_cover_the_small_open_workloads_and_compile():
    """jit.py writes one kernel per small elementwise / row program; NVRTC compiles each for sm_100a without a device.
    Programs outside its conditions (large, f16, ragged widths) are left to the library's kernels."""
    from deuteron_b200 import jit, schedules
    taken = {}
    for name, (graph, meta) in schedules.open_workloads().items():
        plan = compile_kernel(graph, meta, arch='sm_100a').plan
        spec = jit.specialized_source(plan)
        if spec is not None:
            taken[name] = (plan, spec)
    assert {'p02_scale_shift', 'p03_relu_mul', 'f01_rmsnorm', 'f02_row_softmax', 'f03_l2norm'} <= set(taken)
    assert all(plan.kind in jit.KINDS for plan, _ in taken.values()) and {'r01_array_sum', 'r04_row_sum', 'a01_attention', 'a02_attention_128'} <= set(taken)
    plan, spec = taken['f01_rmsnorm']
    assert spec['grid'] == plan.params['rows'] and spec['pointers'][0] == 'x' and spec['pointers'][-1] == 'out'
    assert 'fmaf(' in spec['source'] and 'dtn_rsqrt' in spec['source'] and '--fmad' not in spec['source']
    # outside the conditions: a misaligned f16 buffer, a wide row, a long plain reduction
    graph, meta = schedules.row_reduce_example(1, 1 << 20)
    assert jit.specialized_source(compile_kernel(graph, meta, arch='sm_100a').plan) is None
    graph, meta = schedules.f16_storage_example('affine', count=512, offset=1)   # a vector buffer off the 8-byte grid
    assert jit.specialized_source(compile_kernel(graph, meta).plan) is None
    graph, meta = schedules.f16_storage_example('affine', count=512)
    halves = jit.specialized_source(compile_kernel(graph, meta).plan)
    assert halves is not None and 'cvt.rn.f16.f32' in halves['source'] and halves['scalars'] == [('i64', 64)]
    graph, meta = schedules.row_softmax_example(rows=2, cols=65536)
    assert jit.specialized_source(compile_kernel(graph, meta, arch='sm_100a').plan) is None
    graph, meta = schedules.row_softmax_example(rows=2, cols=32768)   # the longest row that stays in registers: 1024 threads
    assert jit.specialized_source(compile_kernel(graph, meta, arch='sm_100a').plan)['block'] == 1024
    graph, meta = schedules.row_softmax_example(rows=3, cols=640)
    ragged = jit.specialized_source(compile_kernel(graph, meta, arch='sm_100a').plan)
    assert ragged is not None and ragged['grid'] == 3
    if jit._nvrtc() is None:
        pytest.skip('NVRTC is not installed')
    for name, (plan, spec) in taken.items():
        cubin = jit.compile_source(spec['source'])
        assert cubin is not None and cubin[:4] == b'\x7fELF', name
    assert jit.compile_source(ragged['source']) is not None and jit.compile_source(halves['source']) is not None
    assert jit.compile_source('this is not CUDA') is None
    # compiled kernels are kept under DEUTERON_CACHE between processes and re-read without NVRTC
    with tempfile.TemporaryDirectory() as cache_dir:
        previous = os.environ.get('DEUTERON_CACHE')
        os.environ['DEUTERON_CACHE'] = cache_dir
        real_nvrtc = jit._nvrtc
        try:
            source = halves['source'] + '// cache test\n'
            first = jit.compile_source(source)
            stored = list(Path(cache_dir).glob('jit-*.cubin'))
            assert first is not None and len(stored) == 1 and stored[0].read_bytes() == first
            jit._cubins.clear()
            jit._nvrtc = lambda: None   # no compiler: the record alone must serve
            assert jit.compile_source(source) == first
            stored[0].write_bytes(b'not a cubin')
            jit._cubins.clear()
            assert jit.compile_source(source) is None   # a damaged record is not trusted (and nothing can recompile here)
        finally:
            jit._nvrtc = real_nvrtc
            jit._cubins.clear()
            if previous is None:
                del os.environ['DEUTERON_CACHE']
            else:
                os.environ['DEUTERON_CACHE'] = previous
    # the attention example: a few hundred rows of at most 256 keys in multiples of 32, 32 or 64 value columns
    shape = lambda **kw: jit.specialized_source(compile_kernel(*schedules.attention_example(**kw), arch='sm_100a').plan)
    assert shape(rows=128, keys=128, depth=32) is not None and shape(rows=1024, keys=256, depth=128, columns=64) is not None
    assert shape(rows=1025, keys=128, depth=32) is None and shape(rows=8, keys=288, depth=32) is None
    assert shape(rows=8, keys=48, depth=32) is None and shape(rows=8, keys=64, depth=32, columns=96) is None
    staged = shape(rows=8, keys=128, depth=32)
    assert 'cp.async' in staged['source'] and staged['grid'] == 8 and staged['block'] == 32
