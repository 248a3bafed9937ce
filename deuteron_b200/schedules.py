"""Generators of scheduled Kernel IR + meta.json for the hot workloads, in the reference's format.

The reference ships two generator scripts (examples/attention.py, examples/f16_storage.py) and two
committed examples (examples/vector_add, examples/tensor_matmul); its other workloads live in an
external checkout. These functions produce the same kind of (graph, metadata) pair — a graph whose
single KernelOp body is a list of constructor strings, and a meta.json dictionary with entry,
arg_order, grid, block, smem_bytes, zero_outputs and args — for any size, so that the compile/launch
surface can be driven at benchmark sizes. The constructor strings use the field names of the emmy
IR classes as they appear in the reference's committed IR files; no emmy import is needed.
"""
from __future__ import annotations

import math
from typing import Any

import numpy as np

F32 = "DataType(name='f32', np=dtype('float32'), nbytes=4)"
F16 = "DataType(name='f16', np=dtype('float16'), nbytes=2)"


def lit(value: int | float) -> str:
    return f"Literal(value={value!r}, dtype={'float' if isinstance(value, float) else 'int'!r})"


def var(name: str) -> str:
    return f"Var(name={name!r})"


def binary(op: str, left: str, right: str) -> str:
    return f"BinaryExpr(op={op!r}, left={left}, right={right})"


def add(left: str, right: str) -> str:
    return binary('+', left, right)


def mul(left: str, right: str) -> str:
    return binary('*', left, right)


def axis(name: str, extent: int, window: str = 'None') -> str:
    return f"Axis(name={name!r}, extent=Dim({extent}), window={window})"


def _tuple(items) -> str:
    items = list(items)
    return '(' + ', '.join(items) + (',)' if len(items) == 1 else ')')


def _names(names) -> str:
    return _tuple(repr(n) for n in names)


def load(names, source: str, index, dtype: str = F32) -> str:
    return f"Load(names={_names(names)}, input={source!r}, index={_tuple(index)}, dtype={dtype})"


def assign(name: str, op: str, args, dtype: str = F32) -> str:
    return f"Assign(name={name!r}, op=ElementwiseImpl({op!r}), args={_names(args)}, dtype={dtype})"


def accum(name: str, value: str, op: str, axes, base: str | None = None, dtype: str = F32) -> str:
    return (f"Accum(name={name!r}, value={value!r}, op=ElementwiseImpl({op!r}), dtype={dtype}, axes={_names(axes)}, "
            f"base={base!r})")


def write(output: str, index, values, dtype: str = F32, atomic: bool = False) -> str:
    return (f"Write(output={output!r}, index={_tuple(index)}, values={_names(values)}, value_dtype={dtype}, "
            f"atomic={atomic}, swizzle='NONE')")


def loop(axis_text: str, body, unroll: Any = None, seed: bool = False) -> str:
    return f"Loop(axis={axis_text}, body={_tuple(body)}, unroll={unroll!r}, seed={seed})"


def strided_loop(axis_text: str, start: str, step: str, body, unroll: Any = None, seed: bool = False) -> str:
    return (f"StridedLoop(axis={axis_text}, start={start}, step={step}, body={_tuple(body)}, unroll={unroll!r}, end=None, "
            f"seed={seed})")


def tile(axes, body, block_threads: int) -> str:
    return (f"Tile(axes={_tuple(axes)}, body={_tuple(body)}, block_threads={block_threads}, aux_threads=0, raster_axes=None, "
            f"raster_group=None, raster_orient='m')")


def _graph(entry: str, body: str, inputs: dict[str, tuple[list[int], str]], output: tuple[str, list[int], str]) -> dict:
    nodes = {name: {'op': 'InputOp', 'op_fields': {}, 'inputs': [], 'outputs': [{'name': name, 'shape': shape, 'dtype': dtype}]}
             for name, (shape, dtype) in inputs.items()}
    out_name, out_shape, out_dtype = output
    nodes[out_name] = {'op': 'KernelOp', 'op_fields': {'body': [body], 'name': entry, 'zero_delegated': [], 'serial': []},
                       'inputs': list(inputs), 'outputs': [{'name': out_name, 'shape': out_shape, 'dtype': out_dtype}]}
    return {'inputs': list(inputs), 'outputs': [out_name], 'nodes': nodes}


def _metadata(entry: str, launch: dict, rtol: float, atol: float, inputs, outputs) -> dict:
    return {'id': entry, 'rtol': rtol, 'atol': atol, 'graph_inputs': list(inputs), 'graph_outputs': list(outputs),
            'kernels': [launch]}


# ------------------------------------------------------------------------------------------------


def vector_add_example(count: int = 1030, seeds=(21, 22)) -> tuple[dict, dict]:
    """The schedule of examples/vector_add: two elements per tile item, 128-thread blocks, exact result."""
    if count <= 0 or count % 2:
        raise ValueError('count must be positive and even')
    items = count // 2
    index = mul(var('item'), lit(2))
    body = tile([axis('item', items)], [
        load(('left0', 'left1'), 'lhs', [index]), load(('right0', 'right1'), 'rhs', [index]),
        assign('sum0', 'add', ('left0', 'right0')), assign('sum1', 'add', ('left1', 'right1')),
        write('sum', [index], ('sum0', 'sum1')),
    ], 128)
    graph = _graph('vector_add', body, {'lhs': ([count], 'f32'), 'rhs': ([count], 'f32')}, ('sum', [count], 'f32'))
    launch = {'entry': 'vector_add', 'arg_order': ['lhs', 'rhs', 'sum'], 'grid': [math.ceil(items / 128), 1, 1],
              'block': [128, 1, 1], 'smem_bytes': 0, 'zero_outputs': [],
              'args': [{'name': 'lhs', 'dtype': 'f32', 'shape': [count], 'seed': seeds[0]},
                       {'name': 'rhs', 'dtype': 'f32', 'shape': [count], 'seed': seeds[1]},
                       {'name': 'sum', 'dtype': 'f32', 'shape': [count], 'output': True}]}
    return graph, _metadata('vector_add', launch, 0.0, 0.0, ['lhs', 'rhs'], ['sum'])


def f16_storage_example(kind: str = 'copy', count: int = 512, width: int = 4, offset: int = 0) -> tuple[dict, dict]:
    """The five f16 storage kernels of examples/f16_storage.py:19-60 (same entry names, widths, launch,
    seeds and constant buffers): copy, widen, narrow, affine f16(x * 1.5 - 0.25) and cancellation
    f16((x + y) - x), the last two computed in explicit FP32."""
    if kind not in ('copy', 'widen', 'narrow', 'affine', 'cancellation') or width not in (1, 2, 4) or count <= 0 or count % width:
        raise ValueError('unsupported example configuration')
    source, destination = ('f32', F32) if kind == 'narrow' else ('f16', F16), ('f32', F32) if kind == 'widen' else ('f16', F16)
    index = mul(var('element'), lit(width))
    names = tuple(f'input_{i}' for i in range(width))
    body = [load(names, 'x', [add(index, lit(offset))], source[1])]
    args = [{'name': 'x', 'dtype': source[0], 'shape': [count + offset], 'seed': 7}]
    values, value_dtype = names, source[1]
    if kind == 'affine':
        args += [{'name': 'scale', 'dtype': 'f32', 'shape': [1], 'data': [1.5]}, {'name': 'bias', 'dtype': 'f32', 'shape': [1], 'data': [-0.25]}]
        body += [load(('scale_value',), 'scale', [lit(0)]), load(('bias_value',), 'bias', [lit(0)])]
        values = tuple(f'result_{i}' for i in range(width))
        for i, name in enumerate(names):
            body += [assign(f'product_{i}', 'multiply', (name, 'scale_value')), assign(values[i], 'add', (f'product_{i}', 'bias_value'))]
        value_dtype = F32
    elif kind == 'cancellation':
        args.append({'name': 'y', 'dtype': 'f16', 'shape': [count], 'seed': 8})
        second = tuple(f'other_{i}' for i in range(width))
        body.append(load(second, 'y', [index], F16))
        values = tuple(f'result_{i}' for i in range(width))
        for i, name in enumerate(names):
            body += [assign(f'sum_{i}', 'add', (name, second[i])), assign(values[i], 'subtract', (f'sum_{i}', name))]
        value_dtype = F32
    elif kind == 'widen':
        values = tuple(f'result_{i}' for i in range(width))
        body += [assign(value, 'copy', (name,)) for value, name in zip(values, names)]
        value_dtype = F32
    body.append(write('result', [index], values, value_dtype))
    args.append({'name': 'result', 'dtype': destination[0], 'shape': [count], 'output': True})
    entry = 'f16_storage_' + kind
    text = tile([axis('element', count // width)], body, 128)
    inputs = {a['name']: (a['shape'], a['dtype']) for a in args if not a.get('output')}
    graph = _graph(entry, text, inputs, ('result', [count], destination[0]))
    launch = {'node': 'result', 'entry': entry, 'arg_order': [a['name'] for a in args], 'grid': [math.ceil(count / width / 128), 1, 1],
              'block': [128, 1, 1], 'smem_bytes': 0, 'zero_outputs': [], 'args': args, 'final': True}
    return graph, _metadata(entry, launch, 0.001, 0.00001, list(inputs), ['result'])


def attention_example(rows: int = 3, keys: int = 64, depth: int = 32, inplace_denominator: bool = False, seed: int = 7,
                      columns: int = 32) -> tuple[dict, dict]:
    """The online-softmax recurrence of examples/attention.py:21-69 (same statement chain and launch)."""
    if any(type(value) is not int or value <= 0 for value in (rows, keys, depth, columns)):
        raise ValueError('use positive rows, keys, depth and columns')
    dot = loop(axis('dot', depth), [
        load(('query',), 'q', [var('row'), var('dot')]),
        load(('key_value',), 'kt', [var('dot'), var('key')]),
        assign('product', 'multiply', ('query', 'key_value')),
        accum('score_sum', 'product', 'add', ('dot',)),
    ])
    outer = loop(axis('key', keys), [
        dot,
        assign('score', 'multiply', ('score_sum', 'scale')),
        assign('next_maximum', 'maximum', ('maximum', 'score')),
        assign('old_delta', 'subtract', ('maximum', 'next_maximum')),
        assign('alpha', 'exp', ('old_delta',)),
        assign('new_delta', 'subtract', ('score', 'next_maximum')),
        assign('beta', 'exp', ('new_delta',)),
        assign('mass_carry', 'multiply', ('mass', 'alpha')),
        accum('mass', 'beta', 'add', ('key',), 'mass_carry'),
        assign('weighted_carry', 'multiply', ('weighted', 'alpha')),
        load(('value',), 'v', [var('key'), var('column')]),
        assign('weighted_new', 'multiply', ('value', 'beta')),
        accum('weighted', 'weighted_new', 'add', ('key',), 'weighted_carry'),
        accum('maximum', 'score', 'maximum', ('key',)),
    ])
    inverse = 'mass' if inplace_denominator else 'inverse'
    scale = float(np.float32(1 / math.sqrt(depth)))
    body = tile([axis('row', rows), axis('column', columns)], [
        f"Let(name='scale', value={lit(scale)}, dtype={F32})",
        outer,
        assign(inverse, 'reciprocal', ('mass',)),
        assign('normalized', 'multiply', ('weighted', inverse)),
        write('out', [var('row'), var('column')], ('normalized',)),
    ], columns)
    shapes = {'q': [rows, depth], 'kt': [depth, keys], 'v': [keys, columns], 'out': [rows, columns]}
    entry = 'attention_example'
    graph = _graph(entry, body, {name: (shapes[name], 'f32') for name in ('q', 'kt', 'v')}, ('out', shapes['out'], 'f32'))
    args = [{'name': name, 'dtype': 'f32', 'shape': shapes[name], 'seed': seed + i} for i, name in enumerate(('q', 'kt', 'v'))]
    args.append({'name': 'out', 'dtype': 'f32', 'shape': shapes['out'], 'output': True})
    launch = {'node': 'out', 'entry': entry, 'arg_order': ['q', 'kt', 'v', 'out'], 'grid': [rows, 1, 1], 'block': [columns, 1, 1],
              'smem_bytes': 0, 'zero_outputs': [], 'args': args, 'final': True}
    return graph, _metadata(entry, launch, 0.001, 0.0001, ['q', 'kt', 'v'], ['out'])


def row_reduce_example(rows: int, cols: int, op: str = 'sum', block: int = 128, seed: int = 7) -> tuple[dict, dict]:
    """One CTA per row: a thread-strided loop folded by a warp shuffle and a cross-warp tree, the
    structure compiler/transforms.py:62-95 recognises (launch shape of the reference's row-sum
    workload: grid = rows, block = 128). op: 'sum', 'max' or 'sumsq'."""
    if op not in ('sum', 'max', 'sumsq') or rows <= 0 or cols <= 0 or block % 32 or not 32 <= block <= 1024:
        raise ValueError('unsupported reduction configuration')
    combine, identity = ('maximum', '-inf') if op == 'max' else ('add', '0.0')
    inner = [load(('value',), 'x', [var('row'), var('col')])]
    folded = 'value'
    if op == 'sumsq':
        inner.append(assign('square', 'multiply', ('value', 'value')))
        folded = 'square'
    inner.append(accum('state', folded, combine, ('col',)))
    warps = block // 32
    body = tile([axis('row', rows), axis('lane_id', block)], [
        f"Init(name='state', identity={identity}, dtype={F32})",
        strided_loop(axis('col', cols), var('lane_id'), lit(block), inner),
        f"WarpShuffle(state='state', state_b=None, combine_states=ElementwiseImpl({combine!r}), length=32, dtype={F32})",
        f"TreeHalve(bufs=('partials',), state='state', state_b=None, combine_states=ElementwiseImpl({combine!r}), length={warps}, "
        f"tid_var='warp', inner=None, barrier_id=0, barrier_count=None, dtype={F32})",
        write('out', [var('row')], ('state',)),
    ], block)
    entry = f'row_{op}'
    graph = _graph(entry, body, {'x': ([rows, cols], 'f32')}, ('out', [rows], 'f32'))
    launch = {'node': 'out', 'entry': entry, 'arg_order': ['x', 'out'], 'grid': [rows, 1, 1], 'block': [block, 1, 1],
              'smem_bytes': 0, 'zero_outputs': [],
              'args': [{'name': 'x', 'dtype': 'f32', 'shape': [rows, cols], 'seed': seed},
                       {'name': 'out', 'dtype': 'f32', 'shape': [rows], 'output': True}], 'final': True}
    return graph, _metadata(entry, launch, 1e-4, 1e-4, ['x'], ['out'])


def matmul_example(m: int = 128, n: int = 128, k: int = 128, seeds=(7, 11)) -> tuple[dict, dict]:
    """The tiled contraction schedule of examples/tensor_matmul scaled to M x N x K.

    Same structure as the committed 128^3 IR: 32x64 CTA tiles over a (tile_m, tile_n) grid, 512 threads
    (16 x 32, each a 2x2 micro-tile), K advanced in tiles of 64 through a three-slot shared-memory ring
    filled by 16-byte asynchronous copies whose last prefetch coordinates clamp inside the buffer, an
    inner loop of multiply/add groups, and two 2-value stores per thread. arg_order is right, left, result.
    """
    if m % 32 or n % 64 or k % 64 or min(m, n, k) <= 0:
        raise ValueError('the schedule needs M % 32 == 0, N % 64 == 0 and K % 64 == 0')
    tid = add(mul(var('thread_m'), lit(32)), var('thread_n'))
    slot = binary('%', binary('/', var('tile_k'), lit(64)), lit(3))

    def copies(stage: str, k_origin: str) -> list[str]:
        # left tile: 32 rows x 64 k = 512 x 16 bytes; right tile: 64 k x 64 cols = 1024 x 16 bytes
        flat = mul(tid, lit(4))
        l_row, l_col = binary('/', flat, lit(64)), binary('%', flat, lit(64))
        out = [f"CpAsyncCopy(smem='left_stage', smem_index={_tuple([mul(stage, lit(32)), lit(0)])}, src='left', "
               f"src_index={_tuple([add(mul(var('tile_m'), lit(32)), l_row), add(k_origin, l_col)])}, nbytes=16, swizzle='NONE', "
               f"lane_index={_tuple([l_row, l_col])}, lane_rows=32)"]
        for half in range(2):
            flat_r = mul(add(tid, lit(512 * half)), lit(4))
            r_row, r_col = binary('/', flat_r, lit(64)), binary('%', flat_r, lit(64))
            out.append(f"CpAsyncCopy(smem='right_stage', smem_index={_tuple([mul(stage, lit(64)), lit(0)])}, src='right', "
                       f"src_index={_tuple([add(k_origin, r_row), add(mul(var('tile_n'), lit(64)), r_col)])}, nbytes=16, "
                       f"swizzle='NONE', lane_index={_tuple([r_row, r_col])}, lane_rows=64)")
        return out

    prologue = []
    for stage in range(2):
        prologue += copies(lit(stage), lit(min(stage * 64, k - 64))) + ['CpAsyncCommit()']
    clamp = f"TernaryExpr(cond={binary('<', add(var('tile_k'), lit(128)), lit(k))}, if_true={add(var('tile_k'), lit(128))}, if_false={lit(k - 64)})"
    next_slot = binary('%', add(binary('/', var('tile_k'), lit(64)), lit(2)), lit(3))
    inner = []
    rows = [add(add(mul(slot, lit(32)), mul(var('thread_m'), lit(2))), lit(i)) for i in range(2)]
    cols = [add(mul(var('thread_n'), lit(2)), lit(j)) for j in range(2)]
    for j in range(2):
        inner.append(load((f'b{j}',), 'right_stage', [add(mul(slot, lit(64)), var('inner_k')), cols[j]], 'None'))
    for i in range(2):
        inner.append(load((f'a{i}',), 'left_stage', [rows[i], var('inner_k')], 'None'))
    for i in range(2):
        for j in range(2):
            inner += [assign(f'p{i}{j}', 'multiply', (f'b{j}', f'a{i}')), accum(f'acc{i}{j}', f'p{i}{j}', 'add', ('inner_k',))]
    main = strided_loop(axis('tile_k', k), lit(0), lit(64), [
        'CpAsyncWait(group=1)', 'Sync(barrier_id=0, count=None, warp=False)',
        *copies(next_slot, clamp), 'CpAsyncCommit()',
        loop(axis('inner_k', 64), inner, unroll=True),
        'Sync(barrier_id=0, count=None, warp=False)',
    ], unroll=False, seed=True)
    stores = [write('result', [add(add(mul(var('tile_m'), lit(32)), mul(var('thread_m'), lit(2))), lit(i)),
                               add(mul(var('tile_n'), lit(64)), mul(var('thread_n'), lit(2)))], (f'acc{i}0', f'acc{i}1'))
              for i in range(2)]
    window_m = f"Window(parent={axis('logical_m', m)}, base=None, bound=None, partition=False)"
    window_n = f"Window(parent={axis('logical_n', n)}, base=None, bound=None, partition=False)"
    body = tile([axis('tile_m', m // 32, window_m), axis('tile_n', n // 64, window_n), axis('thread_m', 16), axis('thread_n', 32)], [
        *[f"Init(name='acc{i}{j}', identity=0.0, dtype={F32})" for i in range(2) for j in range(2)],
        "Smem(name='left_stage', extents=(96, 64), dtype='float', align=16)",
        "Smem(name='right_stage', extents=(192, 64), dtype='float', align=16)",
        *prologue, main, *stores,
    ], 512)
    entry = f'matmul_tiled_{m}x{n}x{k}' if (m, n, k) != (128, 128, 128) else 'matmul_tiled_128'
    graph = _graph(entry, body, {'left': ([m, k], 'f32'), 'right': ([k, n], 'f32')}, ('result', [m, n], 'f32'))
    graph['nodes']['result']['inputs'] = ['right', 'left']
    launch = {'node': 'result', 'entry': entry, 'arg_order': ['right', 'left', 'result'], 'grid': [(m // 32) * (n // 64), 1, 1],
              'block': [512, 1, 1], 'smem_bytes': 73728, 'zero_outputs': [],
              'args': [{'name': 'right', 'dtype': 'f32', 'shape': [k, n], 'seed': seeds[1]},
                       {'name': 'left', 'dtype': 'f32', 'shape': [m, k], 'seed': seeds[0]},
                       {'name': 'result', 'dtype': 'f32', 'shape': [m, n], 'output': True}], 'final': True}
    return graph, _metadata('tensor_matmul', launch, 0.001, 0.001, ['left', 'right'], ['result'])


def gqa_attention_example(batch: int = 4, query_heads: int = 32, kv_heads: int = 8, positions: int = 4096, depth: int = 128,
                          storage: str = 'f16', seed: int = 7) -> tuple[dict, dict]:
    """Grouped-query attention forward, non-causal, in the statement vocabulary of examples/attention.py.

    q[B,Hq,S,D], k[B,Hkv,S,D], v[B,Hkv,S,D] in `storage` ('f16' or 'f32'), out[B,Hq,S,D] f32; query head h
    reads key/value head h / (Hq / Hkv). The body is the reference example's online-softmax chain with
    four-dimensional indices; f16 operands are widened by `copy` Assigns before any arithmetic, every
    arithmetic statement is FP32. (The reference's own backend declines f16 buffers in a recurrence,
    compiler/storage.py:29-30; this form is the batched workload written against the same IR.)
    One thread block per (batch, head, row), one thread per output column, like the example.
    """
    if storage not in ('f16', 'f32') or min(batch, query_heads, kv_heads, positions, depth) <= 0 or query_heads % kv_heads:
        raise ValueError('unsupported grouped-query attention configuration')
    dtype = F16 if storage == 'f16' else F32
    ratio = query_heads // kv_heads
    kv_head = binary('/', var('head'), lit(ratio))

    def widened(name: str, source: str, index) -> list[str]:
        if storage == 'f32':
            return [load((name,), source, index)]
        return [load((name + '_stored',), source, index, dtype), assign(name, 'copy', (name + '_stored',))]

    dot = loop(axis('dot', depth), [
        *widened('query', 'q', [var('batch'), var('head'), var('row'), var('dot')]),
        *widened('key_value', 'k', [var('batch'), kv_head, var('key'), var('dot')]),
        assign('product', 'multiply', ('query', 'key_value')),
        accum('score_sum', 'product', 'add', ('dot',)),
    ])
    outer = loop(axis('key', positions), [
        dot,
        assign('score', 'multiply', ('score_sum', 'scale')),
        assign('next_maximum', 'maximum', ('maximum', 'score')),
        assign('old_delta', 'subtract', ('maximum', 'next_maximum')),
        assign('alpha', 'exp', ('old_delta',)),
        assign('new_delta', 'subtract', ('score', 'next_maximum')),
        assign('beta', 'exp', ('new_delta',)),
        assign('mass_carry', 'multiply', ('mass', 'alpha')),
        accum('mass', 'beta', 'add', ('key',), 'mass_carry'),
        assign('weighted_carry', 'multiply', ('weighted', 'alpha')),
        *widened('value', 'v', [var('batch'), kv_head, var('key'), var('column')]),
        assign('weighted_new', 'multiply', ('value', 'beta')),
        accum('weighted', 'weighted_new', 'add', ('key',), 'weighted_carry'),
        accum('maximum', 'score', 'maximum', ('key',)),
    ])
    scale = float(np.float32(1 / math.sqrt(depth)))
    body = tile([axis('batch', batch), axis('head', query_heads), axis('row', positions), axis('column', depth)], [
        f"Let(name='scale', value={lit(scale)}, dtype={F32})",
        outer,
        assign('inverse', 'reciprocal', ('mass',)),
        assign('normalized', 'multiply', ('weighted', 'inverse')),
        write('out', [var('batch'), var('head'), var('row'), var('column')], ('normalized',)),
    ], depth)
    shapes = {'q': [batch, query_heads, positions, depth], 'k': [batch, kv_heads, positions, depth],
              'v': [batch, kv_heads, positions, depth], 'out': [batch, query_heads, positions, depth]}
    entry = 'gqa_attention'
    graph = _graph(entry, body, {name: (shapes[name], storage) for name in ('q', 'k', 'v')}, ('out', shapes['out'], 'f32'))
    args = [{'name': name, 'dtype': storage, 'shape': shapes[name], 'seed': seed + i} for i, name in enumerate(('q', 'k', 'v'))]
    args.append({'name': 'out', 'dtype': 'f32', 'shape': shapes['out'], 'output': True})
    launch = {'node': 'out', 'entry': entry, 'arg_order': ['q', 'k', 'v', 'out'], 'grid': [batch * query_heads * positions, 1, 1],
              'block': [depth, 1, 1], 'smem_bytes': 0, 'zero_outputs': [], 'args': args, 'final': True}
    return graph, _metadata(entry, launch, 0.001, 0.0001, ['q', 'k', 'v'], ['out'])
