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


def loop(axis_text: str, body, unroll: bool = False, seed: bool = False) -> str:
    """`seed=True`: the accumulators of the body start from their operator's identity at loop entry (what a loop built
    without the flag does in the reference's generators); False: they continue from an Init or an enclosing loop."""
    return f"Loop(axis={axis_text}, body={_tuple(body)}, unroll={unroll!r}, seed={seed})"


def strided_loop(axis_text: str, start: str, step: str, body, unroll: bool = False, seed: bool = False) -> str:
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


def pointwise_example(kind: str = 'affine', count: int = 4096, block: int = 256) -> tuple[dict, dict]:
    """The reference's two fused FP32 pointwise workloads, in their launch shapes: 'affine' is
    add = x * mul_c1 + add_c1 with both constants as one-element buffers (mul_c1[1] = 2, add_c1[1] = 1, x[4096],
    grid 4 x block 256, four values per thread); 'relu_multiply' is mul = relu(x) * y (x[2048], y[2048], grid 2)."""
    if kind not in ('affine', 'relu_multiply') or count <= 0 or count % 4:
        raise ValueError('unsupported example configuration')
    index = mul(var('element'), lit(4))
    names = tuple(f'x{i}' for i in range(4))
    results = tuple(f'result{i}' for i in range(4))
    if kind == 'affine':
        output, entry = 'add', 'k_add_pointwise'
        args = [{'name': 'mul_c1', 'dtype': 'f32', 'shape': [1], 'data': [2.0]}, {'name': 'add_c1', 'dtype': 'f32', 'shape': [1], 'data': [1.0]},
                {'name': 'x', 'dtype': 'f32', 'shape': [count], 'seed': 0}]
        body = [load(('scale',), 'mul_c1', [lit(0)]), load(('shift',), 'add_c1', [lit(0)]), load(names, 'x', [index])]
        for i in range(4):
            body += [assign(f'scaled{i}', 'multiply', (names[i], 'scale')), assign(results[i], 'add', (f'scaled{i}', 'shift'))]
    else:
        output, entry = 'mul', 'k_mul_pointwise'
        args = [{'name': 'x', 'dtype': 'f32', 'shape': [count], 'seed': 0}, {'name': 'y', 'dtype': 'f32', 'shape': [count], 'seed': 1}]
        others = tuple(f'y{i}' for i in range(4))
        body = [load(names, 'x', [index]), load(others, 'y', [index])]
        for i in range(4):
            body += [assign(f'positive{i}', 'relu', (names[i],)), assign(results[i], 'multiply', (f'positive{i}', others[i]))]
    body.append(write(output, [index], results))
    args.append({'name': output, 'dtype': 'f32', 'shape': [count], 'output': True})
    inputs = {a['name']: (a['shape'], a['dtype']) for a in args if not a.get('output')}
    graph = _graph(entry, tile([axis('element', count // 4)], body, block), inputs, (output, [count], 'f32'))
    launch = {'node': output, 'entry': entry, 'arg_order': [a['name'] for a in args], 'grid': [math.ceil(count / 4 / block), 1, 1],
              'block': [block, 1, 1], 'smem_bytes': 0, 'zero_outputs': [], 'args': args, 'final': True}
    return graph, _metadata(entry, launch, 1e-5, 1e-6, list(inputs), [output])


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
    ], seed=True)
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
    ], seed=True)
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


def _int_eq(left: str, right: str) -> str:
    return binary('==', left, right)


def reduction_tail(states, others, combines, warps: int) -> list[str]:
    """The statements that fold per-thread partial states into one value per CTA, in the form the
    reference matches (compiler/transforms.py:88-94, compiler/passes/hybrid_normalizer.py:53-66,
    compiler/passes/tailtree.py:63-110): a 32-lane WarpShuffle, one shared-memory slot per warp and state
    written by lane 0, a barrier, and a TreeHalve over the warp partials."""
    combine_body = _tuple(combines)
    buffers = [f'{state}_partials' for state in states]
    out = [f"WarpShuffle(state={_names(states)}, state_b={_names(others)}, combine_states={combine_body}, length=32, dtype={F32})"]
    out += [f"Smem(name={buffer!r}, extents=({warps},), dtype='float', align=0)" for buffer in buffers]
    stores = [write(buffer, [var('warp')], (state,)) for buffer, state in zip(buffers, states)]
    out.append(f"Cond(cond={_int_eq(var('lane'), lit(0))}, body={_tuple(stores)}, else_body=())")
    out.append('Sync(barrier_id=0, count=None, warp=False)')
    out.append(f"TreeHalve(bufs={_names(buffers)}, state={_names(states)}, state_b={_names(others)}, combine_states={combine_body}, "
               f"length={warps}, tid_var='warp', inner=None, barrier_id=0, barrier_count=None, dtype={F32})")
    return out


def _row_launch(entry: str, rows: int, block: int, args: list[dict], node: str) -> dict:
    return {'node': node, 'entry': entry, 'arg_order': [a['name'] for a in args], 'grid': [rows, 1, 1], 'block': [block, 1, 1],
            'smem_bytes': 0, 'zero_outputs': [], 'args': args, 'final': True}


def _check_rows(rows: int, cols: int, block: int) -> None:
    if rows <= 0 or cols <= 0 or block % 32 or not 32 <= block <= 1024:
        raise ValueError('unsupported row kernel configuration')


def row_reduce_example(rows: int, cols: int, op: str = 'sum', block: int = 128, seed: int = 7) -> tuple[dict, dict]:
    """One CTA per row: a thread-strided loop folded by a warp shuffle and a cross-warp tree, the
    structure compiler/transforms.py:62-95 recognises (launch shape of the reference's row-sum
    workload: grid = rows, block = 128). op: 'sum', 'max' or 'sumsq'."""
    if op not in ('sum', 'max', 'sumsq'):
        raise ValueError('unsupported reduction configuration')
    _check_rows(rows, cols, block)
    combine, identity = ('maximum', '-inf') if op == 'max' else ('add', '0.0')
    inner = [load(('value',), 'x', [var('row'), var('col')])]
    folded = 'value'
    if op == 'sumsq':
        inner.append(assign('square', 'multiply', ('value', 'value')))
        folded = 'square'
    inner.append(accum('state', folded, combine, ('col',)))
    body = tile([axis('row', rows), axis('lane_id', block)], [
        f"Init(name='state', identity={identity}, dtype={F32})",
        strided_loop(axis('col', cols), var('lane_id'), lit(block), inner, seed=True),
        *reduction_tail(('state',), ('state_b',), [assign('state', combine, ('state', 'state_b'))], block // 32),
        write('out', [var('row')], ('state',)),
    ], block)
    entry = f'row_{op}'
    graph = _graph(entry, body, {'x': ([rows, cols], 'f32')}, ('out', [rows], 'f32'))
    launch = _row_launch(entry, rows, block, [{'name': 'x', 'dtype': 'f32', 'shape': [rows, cols], 'seed': seed},
                                              {'name': 'out', 'dtype': 'f32', 'shape': [rows], 'output': True}], 'out')
    return graph, _metadata(entry, launch, 1e-4, 1e-4, ['x'], ['out'])


def mean_example(count: int = 32768, block: int = 128, seed: int = 0) -> tuple[dict, dict]:
    """Mean of a vector with the element count as a one-element buffer, the shape of the reference's
    mean workload (x[32768], mean_keepdim_count[1] -> mean[1], one CTA of 128 threads)."""
    _check_rows(1, count, block)
    body = tile([axis('lane_id', block)], [
        f"Init(name='state', identity=0.0, dtype={F32})",
        strided_loop(axis('i', count), var('lane_id'), lit(block), [load(('value',), 'x', [var('i')]), accum('state', 'value', 'add', ('i',))],
                     seed=True),
        *reduction_tail(('state',), ('state_b',), [assign('state', 'add', ('state', 'state_b'))], block // 32),
        load(('count',), 'mean_keepdim_count', [lit(0)]),
        assign('result', 'divide', ('state', 'count')),
        write('mean', [lit(0)], ('result',)),
    ], block)
    graph = _graph('k_mean', body, {'x': ([count], 'f32'), 'mean_keepdim_count': ([1], 'f32')}, ('mean', [1], 'f32'))
    launch = _row_launch('k_mean', 1, block, [{'name': 'x', 'dtype': 'f32', 'shape': [count], 'seed': seed},
                                              {'name': 'mean_keepdim_count', 'dtype': 'f32', 'shape': [1], 'data': [float(count)]},
                                              {'name': 'mean', 'dtype': 'f32', 'shape': [1], 'output': True}], 'mean')
    return graph, _metadata('k_mean', launch, 1e-4, 1e-5, ['x'], ['mean'])


def _vector_consumer(rows_index: list[str], cols: int, block: int, width: int, loads: list[tuple[str, str, bool]], steps, result: str,
                     output: str) -> str:
    """The elementwise loop of a row kernel: `width` consecutive columns per thread step. loads:
    (value prefix, buffer, indexed by row too); steps(lane) -> list of (name, op, args) for that lane."""
    column = mul(lit(width), var('j')) if width > 1 else var('j')
    body = []
    for prefix, buffer, by_row in loads:
        body.append(load(tuple(f'{prefix}{lane}' for lane in range(width)), buffer, [*(rows_index if by_row else []), column]))
    for lane in range(width):
        body += [assign(name, op, args) for name, op, args in steps(lane)]
    body.append(write(output, [*rows_index, column], tuple(f'{result}{lane}' for lane in range(width))))
    return strided_loop(axis('j', cols // width), var('lane_id'), lit(block), body)


def rms_norm_example(rows: int = 64, cols: int = 1024, block: int = 128, epsilon: float = 1e-5, seeds=(0, 1)) -> tuple[dict, dict]:
    """RMS norm, out = x * rsqrt(sum(x^2) / count + eps) * w, in the reference's kernel shape: arguments
    mean_count[1], add_c1[1], x[rows, cols], w[cols] -> mul_1[rows, cols], one CTA of 128 threads per row, a
    sum-of-squares loop, the shuffle/tree tail, and a four-wide consumer loop that reloads the row (the form
    compiler/passes/regforward.py:88-148 forwards through registers)."""
    _check_rows(rows, cols, block)
    if cols % (4 * block):
        raise ValueError('the four-wide consumer needs cols to be a multiple of 4 * block')
    steps = lambda lane: [(f'scaled{lane}', 'multiply', (f'x{lane}', 'inverse')), (f'y{lane}', 'multiply', (f'scaled{lane}', f'w{lane}'))]
    body = tile([axis('row', rows), axis('lane_id', block)], [
        f"Init(name='state', identity=0.0, dtype={F32})",
        strided_loop(axis('col', cols), var('lane_id'), lit(block),
                     [load(('value',), 'x', [var('row'), var('col')]), assign('square', 'multiply', ('value', 'value')),
                      accum('state', 'square', 'add', ('col',))], seed=True),
        *reduction_tail(('state',), ('state_b',), [assign('state', 'add', ('state', 'state_b'))], block // 32),
        load(('count',), 'mean_count', [lit(0)]), load(('eps',), 'add_c1', [lit(0)]),
        assign('mean_square', 'divide', ('state', 'count')), assign('shifted', 'add', ('mean_square', 'eps')),
        assign('inverse', 'rsqrt', ('shifted',)),
        _vector_consumer([var('row')], cols, block, 4, [('x', 'x', True), ('w', 'w', False)], steps, 'y', 'mul_1'),
    ], block)
    inputs = {'mean_count': ([1], 'f32'), 'add_c1': ([1], 'f32'), 'x': ([rows, cols], 'f32'), 'w': ([cols], 'f32')}
    graph = _graph('k_rms_norm', body, inputs, ('mul_1', [rows, cols], 'f32'))
    launch = _row_launch('k_rms_norm', rows, block, [
        {'name': 'mean_count', 'dtype': 'f32', 'shape': [1], 'data': [float(cols)]},
        {'name': 'add_c1', 'dtype': 'f32', 'shape': [1], 'data': [float(epsilon)]},
        {'name': 'x', 'dtype': 'f32', 'shape': [rows, cols], 'seed': seeds[0]},
        {'name': 'w', 'dtype': 'f32', 'shape': [cols], 'seed': seeds[1]},
        {'name': 'mul_1', 'dtype': 'f32', 'shape': [rows, cols], 'output': True}], 'mul_1')
    return graph, _metadata('k_rms_norm', launch, 1e-4, 1e-5, ['x', 'w'], ['mul_1'])


def l2_norm_example(rows: int = 64, cols: int = 512, block: int = 128, seed: int = 0) -> tuple[dict, dict]:
    """L2 norm, out = x / sqrt(sum(x^2)), in the reference's kernel shape (x[64, 512] -> div[64, 512], grid 64 x
    block 128): sqrt followed by reciprocal, which the reference fuses into rsqrt (compiler/transforms.py:6-9)."""
    _check_rows(rows, cols, block)
    if cols % (4 * block):
        raise ValueError('the four-wide consumer needs cols to be a multiple of 4 * block')
    steps = lambda lane: [(f'y{lane}', 'multiply', (f'x{lane}', 'inverse'))]
    body = tile([axis('row', rows), axis('lane_id', block)], [
        f"Init(name='state', identity=0.0, dtype={F32})",
        strided_loop(axis('col', cols), var('lane_id'), lit(block),
                     [load(('value',), 'x', [var('row'), var('col')]), assign('square', 'multiply', ('value', 'value')),
                      accum('state', 'square', 'add', ('col',))], seed=True),
        *reduction_tail(('state',), ('state_b',), [assign('state', 'add', ('state', 'state_b'))], block // 32),
        assign('norm', 'sqrt', ('state',)), assign('inverse', 'reciprocal', ('norm',)),
        _vector_consumer([var('row')], cols, block, 4, [('x', 'x', True)], steps, 'y', 'div'),
    ], block)
    graph = _graph('k_div_reduce', body, {'x': ([rows, cols], 'f32')}, ('div', [rows, cols], 'f32'))
    launch = _row_launch('k_div_reduce', rows, block, [{'name': 'x', 'dtype': 'f32', 'shape': [rows, cols], 'seed': seed},
                                                        {'name': 'div', 'dtype': 'f32', 'shape': [rows, cols], 'output': True}], 'div')
    return graph, _metadata('k_div_reduce', launch, 1e-4, 1e-5, ['x'], ['div'])


def row_softmax_example(rows: int = 64, cols: int = 256, block: int = 128, seed: int = 0) -> tuple[dict, dict]:
    """Row softmax in the form compiler/passes/hybrid_normalizer.py:45-120 matches: an online (maximum, sum)
    pair in the reduction loop, the pair combined by the shuffle/tree tail, a reciprocal of the sum, and a
    consumer loop computing reciprocal * exp(x - maximum). Launch shape of the reference's workload:
    x[64, 256] -> softmax[64, 256], grid 64 x block 128."""
    _check_rows(rows, cols, block)
    if cols % block:
        raise ValueError('cols must be a multiple of block')
    online = [
        load(('value',), 'x', [var('row'), var('col')]),
        assign('top', 'maximum', ('m', 'value')), assign('shift_old', 'subtract', ('m', 'top')), assign('alpha', 'exp', ('shift_old',)),
        assign('shift_new', 'subtract', ('value', 'top')), assign('beta', 'exp', ('shift_new',)),
        assign('scaled', 'multiply', ('s', 'alpha')),
        accum('s', 'beta', 'add', ('col',), base='scaled'), accum('m', 'value', 'maximum', ('col',)),
    ]
    merge = [
        assign('top_b', 'maximum', ('m', 'm_b')), assign('da', 'subtract', ('m', 'top_b')), assign('ea', 'exp', ('da',)),
        assign('db', 'subtract', ('m_b', 'top_b')), assign('eb', 'exp', ('db',)),
        assign('sa', 'multiply', ('s', 'ea')), assign('sb', 'multiply', ('s_b', 'eb')),
        assign('s', 'add', ('sa', 'sb')), assign('m', 'copy', ('top_b',)),
    ]
    consumer = strided_loop(axis('j', cols), var('lane_id'), lit(block), [
        load(('again',), 'x', [var('row'), var('j')]), assign('delta', 'subtract', ('again', 'm')), assign('weight', 'exp', ('delta',)),
        assign('probability', 'multiply', ('inverse', 'weight')), write('softmax', [var('row'), var('j')], ('probability',)),
    ])
    body = tile([axis('row', rows), axis('lane_id', block)], [
        f"Init(name='m', identity=-3.4028234663852886e+38, dtype={F32})", f"Init(name='s', identity=0.0, dtype={F32})",
        strided_loop(axis('col', cols), var('lane_id'), lit(block), online, seed=True),
        *reduction_tail(('m', 's'), ('m_b', 's_b'), merge, block // 32),
        assign('inverse', 'reciprocal', ('s',)),
        consumer,
    ], block)
    graph = _graph('k_softmax', body, {'x': ([rows, cols], 'f32')}, ('softmax', [rows, cols], 'f32'))
    launch = _row_launch('k_softmax', rows, block, [{'name': 'x', 'dtype': 'f32', 'shape': [rows, cols], 'seed': seed},
                                                     {'name': 'softmax', 'dtype': 'f32', 'shape': [rows, cols], 'output': True}], 'softmax')
    return graph, _metadata('k_softmax', launch, 1e-4, 1e-6, ['x'], ['softmax'])


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


def split_k_matmul_example(m: int = 128, n: int = 64, k: int = 256, depth: int = 4, seeds=(0, 1)) -> tuple[dict, dict]:
    """Split-K contraction with atomic stores into a zeroed output, in the statement order
    compiler/passes/gridfold.py:60-62 matches (two copy loops, commit, wait, barrier, product loop, barrier) and
    with the launch shape of the reference's rectangular matmul workload (x1[256, 64], x0[128, 256] ->
    matmul[128, 64], zero_outputs = [matmul], grid 512 x block 256).

    The grid is (tile_m, tile_n, split): every CTA multiplies a 32 x depth slice of x0 by a depth x 32 slice of
    x1 and adds its 32 x 32 partial product into the output; 16 x 16 threads hold 2 x 2 micro-tiles."""
    if m % 32 or n % 32 or k % depth or depth % 4 or min(m, n, k) <= 0:
        raise ValueError('the schedule needs M % 32 == 0, N % 32 == 0, K % depth == 0 and depth % 4 == 0')
    splits = k // depth
    thread = add(mul(var('thread_m'), lit(16)), var('thread_n'))
    flat = mul(var('piece'), lit(4))

    def copy_loop(smem: str, source: str, shape: tuple[int, int], origin: tuple[str, str]) -> str:
        inside = (binary('/', flat, lit(shape[1])), binary('%', flat, lit(shape[1])))
        copy = (f"CpAsyncCopy(smem={smem!r}, smem_index={_tuple(inside)}, src={source!r}, "
                f"src_index={_tuple([add(origin[0], inside[0]), add(origin[1], inside[1])])}, nbytes=16, swizzle='NONE', "
                f"lane_index=None, lane_rows=None)")
        return strided_loop(axis('piece', shape[0] * shape[1] // 4), thread, lit(256), [copy])

    k_origin = add(mul(var('split'), lit(depth)), var('k0'))
    inner = []
    for j in range(2):
        inner.append(load((f'b{j}',), 'rhs_tile', [var('inner_k'), add(mul(var('thread_n'), lit(2)), lit(j))], 'None'))
    for i in range(2):
        inner.append(load((f'a{i}',), 'lhs_tile', [add(mul(var('thread_m'), lit(2)), lit(i)), var('inner_k')], 'None'))
    for i in range(2):
        for j in range(2):
            inner += [assign(f'p{i}{j}', 'multiply', (f'b{j}', f'a{i}')), accum(f'acc{i}{j}', f'p{i}{j}', 'add', ('inner_k',))]
    outer = strided_loop(axis('k0', depth), lit(0), lit(depth), [
        copy_loop('lhs_tile', 'x0', (32, depth), (mul(var('tile_m'), lit(32)), k_origin)),
        copy_loop('rhs_tile', 'x1', (depth, 32), (k_origin, mul(var('tile_n'), lit(32)))),
        'CpAsyncCommit()', 'CpAsyncWait(group=0)', 'Sync(barrier_id=0, count=None, warp=False)',
        loop(axis('inner_k', depth), inner, unroll=True),
        'Sync(barrier_id=0, count=None, warp=False)',
    ])
    stores = []
    for i in range(2):
        row = add(add(mul(var('tile_m'), lit(32)), mul(var('thread_m'), lit(2))), lit(i))
        col = add(mul(var('tile_n'), lit(32)), mul(var('thread_n'), lit(2)))
        stores.append(write('matmul', [row, col], (f'acc{i}0', f'acc{i}1'), atomic=True))
    body = tile([axis('tile_m', m // 32), axis('tile_n', n // 32), axis('split', splits), axis('thread_m', 16), axis('thread_n', 16)], [
        *[f"Init(name='acc{i}{j}', identity=0.0, dtype={F32})" for i in range(2) for j in range(2)],
        f"Smem(name='lhs_tile', extents=(32, {depth}), dtype='float', align=16)",
        f"Smem(name='rhs_tile', extents=({depth}, 32), dtype='float', align=16)",
        outer, *stores,
    ], 256)
    graph = _graph('k_matmul', body, {'x0': ([m, k], 'f32'), 'x1': ([k, n], 'f32')}, ('matmul', [m, n], 'f32'))
    graph['nodes']['matmul']['inputs'] = ['x1', 'x0']
    launch = {'node': 'matmul', 'entry': 'k_matmul', 'arg_order': ['x1', 'x0', 'matmul'], 'grid': [(m // 32) * (n // 32) * splits, 1, 1],
              'block': [256, 1, 1], 'smem_bytes': 0, 'zero_outputs': ['matmul'],
              'args': [{'name': 'x1', 'dtype': 'f32', 'shape': [k, n], 'seed': seeds[1]},
                       {'name': 'x0', 'dtype': 'f32', 'shape': [m, k], 'seed': seeds[0]},
                       {'name': 'matmul', 'dtype': 'f32', 'shape': [m, n], 'output': True}], 'final': True}
    return graph, _metadata('k_matmul', launch, 0.001, 0.001, ['x0', 'x1'], ['matmul'])


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
    ], seed=True)
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
    ], seed=True)
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


# ------------------------------------------------------------------------------------------------
# problem directories
# ------------------------------------------------------------------------------------------------


def open_workloads() -> dict[str, tuple[dict, dict]]:
    """The reference's fifteen open workloads (README.md:163-180) in their published shapes and launch geometries
    (benchmarks/rtx5090-2026-10-24-r6.json, `variants[].launch`), regenerated as (graph, metadata) pairs: the IR files
    of that set are not part of the reference's repository."""
    return {
        'p00_scalar_add': vector_add_example(128), 'p01_vector_add': vector_add_example(1024),
        'p02_scale_shift': pointwise_example('affine', 4096), 'p03_relu_mul': pointwise_example('relu_multiply', 2048),
        'r01_array_sum': row_reduce_example(1, 1024, 'sum'), 'r02_big_sum': row_reduce_example(1, 65536, 'sum'),
        'r03_mean': mean_example(32768), 'r04_row_sum': row_reduce_example(64, 512, 'sum'),
        'm01_matmul_512': matmul_example(512, 512, 512), 'm02_matmul_rect': split_k_matmul_example(128, 64, 256),
        'f01_rmsnorm': rms_norm_example(64, 1024), 'f02_row_softmax': row_softmax_example(64, 256),
        'f03_l2norm': l2_norm_example(64, 512),
        'a01_attention': attention_example(64, 64, 64, columns=64), 'a02_attention_128': attention_example(128, 128, 32),
    }


def write_problem(directory: Any, graph: dict, metadata: dict) -> None:
    """Writes one problem directory in the layout the reference's benchmark driver reads (benchmark.py:447-466):
    `meta.json` and `<entry>.ir.json` for the (single) kernel of the metadata. `expected.npz` is the caller's to add."""
    import json
    from pathlib import Path
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    (directory / 'meta.json').write_text(json.dumps(metadata, indent=1) + '\n')
    (directory / (metadata['kernels'][0]['entry'] + '.ir.json')).write_text(json.dumps(graph) + '\n')
