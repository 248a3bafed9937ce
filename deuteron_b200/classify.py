"""Workload classifier: maps a parsed, scheduled kernel to the native kernel that computes it.

The reference recognises the same structures before it emits specialised code: a dense
shared-memory contraction (compiler/passes/contraction.py:58-213), the online-softmax recurrence
(compiler/passes/recurrence.py:193-388), thread-strided reductions (compiler/transforms.py:62-95) and
Load/Assign/Write elementwise tiles (compiler/passes/vectorize.py:31-128, compiler/storage.py:27-58).
Here the recognised structure selects a hand-written sm_100a kernel; anything else raises
NotImplementedError. Classification reads structure and buffer shapes, never names.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from . import ir
from .classify_rows import classify_rows
from .native import BINARY_OPS, ELEMENTWISE_OPS


@dataclass(frozen=True)
class Plan:
    """What to run: `kind` picks the C-ABI entry point, `params` its shape arguments, `buffers` the
    role of each meta.json buffer (role -> (buffer name, element offset))."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    buffers: dict[str, tuple[str, int]] = field(default_factory=dict)

    def describe(self) -> str:
        roles = ', '.join(f'{role}={name}+{offset}' if offset else f'{role}={name}' for role, (name, offset) in self.buffers.items())
        settings = ', '.join(f'{key}={value}' for key, value in self.params.items())
        return f'{self.kind}({settings}; {roles})'


def _op_name(op: Any) -> str:
    return op.name if isinstance(op, ir.Node) else str(op)


def _dtype_name(dtype: Any) -> str | None:
    if isinstance(dtype, ir.Node) and dtype.kind == 'DataType':
        return dtype.name
    return None


def _single_tile(kernel: ir.Kernel) -> ir.Node:
    tiles = [stmt for stmt in kernel.body if stmt.kind == 'Tile']
    if len(tiles) != 1 or len(kernel.body) != 1:
        raise NotImplementedError('expected a kernel body of exactly one Tile')
    return tiles[0]


def _shape(specs: dict, name: str) -> tuple[int, ...]:
    return tuple(specs[name]['shape'])


# ------------------------------------------------------------------------------------------------
# contraction
# ------------------------------------------------------------------------------------------------


def _classify_gemm(tile: ir.Node, specs: dict, precision: str, launch: dict) -> Plan | None:
    statements = list(ir.walk([tile]))
    accums = [s for s in statements if s.kind == 'Accum' and _op_name(s.op) == 'add']
    assigns = {s.name: s for s in statements if s.kind == 'Assign'}
    products = [assigns[a.value] for a in accums if a.value in assigns and _op_name(assigns[a.value].op) == 'multiply'
                and len(assigns[a.value].args) == 2]
    writes = [s for s in statements if s.kind == 'Write']
    if not products or not writes or any(len(w.index) != 2 for w in writes):
        return None
    if any(_op_name(s.op) in ('exp', 'maximum') for s in assigns.values()):
        return None
    output = writes[0].output
    if any(w.output != output for w in writes):
        return None
    split_depth = _split_k_depth(tile, writes, launch) if any(w.atomic for w in writes) else None
    loads = {}
    for stmt in statements:
        if stmt.kind == 'Load':
            for name in stmt.names:
                loads[name] = stmt
    copies: dict[str, str] = {}
    for stmt in statements:
        if stmt.kind == 'CpAsyncCopy':
            if copies.setdefault(stmt.smem, stmt.src) != stmt.src:
                return None
    # the reduction axis is the loop variable that indexes both operands of the product
    accum_axes = set()
    for accum in accums:
        accum_axes.update(accum.axes or ())
    left = right = None
    for product in products:
        for operand in product.args:
            load = loads.get(operand)
            if load is None or len(load.index) != 2:
                return None
            source = copies.get(load.input, load.input)
            if source not in specs:
                return None
            in_row = bool(ir.expression_vars(load.index[0]) & accum_axes)
            in_col = bool(ir.expression_vars(load.index[1]) & accum_axes)
            if in_col and not in_row:      # indexed [row, k]
                if left not in (None, source):
                    return None
                left = source
            elif in_row and not in_col:    # indexed [k, col]
                if right not in (None, source):
                    return None
                right = source
            else:
                return None
    if left is None or right is None or left == right:
        return None
    (m, k), (k2, n), out_shape = _shape(specs, left), _shape(specs, right), _shape(specs, output)
    if k != k2 or out_shape != (m, n):
        raise ValueError(f'contraction shapes disagree: {left}{[m, k]} @ {right}{[k2, n]} -> {output}{list(out_shape)}')
    if split_depth is not None and split_depth != k:
        raise NotImplementedError(f'split-K partial products cover {split_depth} of the {k} reduction steps')
    for name in (left, right, output):
        if specs[name]['dtype'] != 'f32':
            raise NotImplementedError('contractions take f32 buffers')
    # The reference runs a contraction on the tensor cores (compensated products) only when both operands are staged
    # through shared memory by its asynchronous copies (compiler/passes/contraction.py:58-213); every other
    # contraction schedule, the split-K one among them, is lowered to plain FP32 multiply-adds
    # (compiler/codegen/lower.py:600-653). The native mode follows, so that the error level is the reference's.
    staged = {copies.get(loads[operand].input) for product in products for operand in product.args}
    mode = precision if staged == {left, right} and _tensor_core_shape(tile, statements, products, writes, precision, launch) else 'f32'
    if mode == 'f32' and split_depth is not None:
        mode = 'f32_splitk'     # the reference adds partial sums over slices of k there: no sequential k order to keep
    return Plan('gemm', {'mode': mode, 'm': m, 'n': n, 'k': k},
                {'left': (left, 0), 'right': (right, 0), 'out': (output, 0)})


def _tensor_core_shape(tile: ir.Node, statements: list, products: list, writes: list, precision: str, launch: dict) -> bool:
    """The shape conditions under which the reference turns a staged contraction into tensor-core products
    (compiler/passes/contraction.py:135, 211): the CTA's output tile is made of 16 x 8 warp tiles, exactly one per
    warp, and the staged depth of the inner product loop is a multiple of the instruction's k (16 for bf16x3, 8 for
    tf32x3). A schedule that fails them is lowered to FP32 multiply-adds there."""
    product_names = {product.name for product in products}
    depths = {ir.axis_extent(stmt.axis) for stmt in statements if stmt.kind == 'Loop'
              and any(child.kind == 'Assign' and child.name in product_names for child in stmt.body)}
    if len(depths) != 1 or len(tile.axes) < 2:
        return False
    depth = depths.pop()
    rows, cols = len(writes), len(writes[0].values)
    tile_rows, tile_cols = ir.axis_extent(tile.axes[-2]) * rows, ir.axis_extent(tile.axes[-1]) * cols
    threads = launch['block'][0]
    step = 16 if precision == 'bf16x3' else 8
    return (depth % step == 0 and tile_rows % 16 == 0 and tile_cols % 8 == 0
            and (tile_rows // 16) * (tile_cols // 8) * 32 == threads)


def _split_k_depth(tile: ir.Node, writes: list, launch: dict) -> int:
    """Reduction steps covered by an atomic (split-K) contraction: every CTA adds a partial product into an output
    that the launch zeroes first (zero_outputs, benchmark.py:240-243), so the sum over the split axis is the full
    product and one overwriting GEMM computes the same matrix. The split axis is the grid axis the stores do not
    depend on (compiler/passes/gridfold.py:66-70); the steps per CTA are the extent of the loop around the products."""
    output = writes[0].output
    if not all(w.atomic for w in writes):
        raise NotImplementedError('atomic and plain stores of a contraction must not be mixed')
    if output not in (launch.get('zero_outputs') or []):
        raise NotImplementedError('atomic (split-K) contractions need their output in zero_outputs')
    stored = set()
    for w in writes:
        for expr in w.index:
            stored |= ir.expression_vars(expr)
    split_axes = [a for a in tile.axes if a.extent.value > 1 and a.name not in stored]
    outer = [s for s in tile.body if s.kind in ('Loop', 'StridedLoop') and any(c.kind == 'Accum' for c in ir.walk(s.body))]
    if len(split_axes) != 1 or len(outer) != 1:
        raise NotImplementedError('atomic (split-K) contractions have one split axis and one reduction loop nest')
    return split_axes[0].extent.value * outer[0].axis.extent.value


# ------------------------------------------------------------------------------------------------
# attention recurrence
# ------------------------------------------------------------------------------------------------


def _classify_attention(tile: ir.Node, specs: dict) -> Plan | None:
    statements = list(ir.walk([tile]))
    assigns = [s for s in statements if s.kind == 'Assign']
    ops = [_op_name(s.op) for s in assigns]
    if ops.count('exp') + ops.count('exp_fast') < 2 or 'reciprocal' not in ops:
        return None
    if not any(s.kind == 'Accum' and _op_name(s.op) == 'maximum' for s in statements):
        return None
    outer = [s for s in tile.body if s.kind == 'Loop']
    if len(outer) != 1:
        return None
    key_axis = outer[0].axis.name
    inner = [s for s in outer[0].body if s.kind == 'Loop']
    if len(inner) != 1:
        return None
    dot_axis = inner[0].axis.name
    q = kt = v = None
    ranks = {len(load.index) for load in statements if load.kind == 'Load' and math.prod(_shape(specs, load.input)) != 1}
    if ranks == {4}:
        return _classify_gqa(tile, outer[0], inner[0], specs)
    for load in (s for s in inner[0].body if s.kind == 'Load'):
        if len(load.index) != 2:
            return None
        first, second = (ir.expression_vars(e) for e in load.index)
        if dot_axis in second and key_axis not in first | second:
            q = load.input
        elif dot_axis in first and key_axis in second:
            kt = load.input
    for load in (s for s in outer[0].body if s.kind == 'Load'):
        if len(load.index) == 2 and key_axis in ir.expression_vars(load.index[0]):
            v = load.input
    writes = [s for s in tile.body if s.kind == 'Write']
    if None in (q, kt, v) or len(writes) != 1:
        return None
    out = writes[0].output
    (rows, depth), (depth2, keys), (keys2, cols) = _shape(specs, q), _shape(specs, kt), _shape(specs, v)
    if depth != depth2 or keys != keys2 or _shape(specs, out) != (rows, cols):
        raise ValueError('attention buffer shapes disagree')
    if outer[0].axis.extent.value != keys or inner[0].axis.extent.value != depth:
        raise ValueError('attention loop extents disagree with the buffer shapes')
    for name in (q, kt, v, out):
        if specs[name]['dtype'] != 'f32':
            raise NotImplementedError('the attention recurrence takes f32 buffers')
    scale = _attention_scale(tile, outer[0], inner[0], specs)
    if scale is None:
        return None
    return Plan('attention', {'rows': rows, 'keys': keys, 'depth': depth, 'cols': cols, 'scale': scale},
                {'q': (q, 0), 'kt': (kt, 0), 'v': (v, 0), 'out': (out, 0)})


def _classify_gqa(tile: ir.Node, outer: ir.Node, inner: ir.Node, specs: dict) -> Plan | None:
    """The same recurrence over [batch, head, position, depth] buffers with grouped key/value heads:
    q[B,Hq,S,D], k[B,Hkv,S,D], v[B,Hkv,S,D] -> out[B,Hq,S,D], the key/value head of query head h being
    h / (Hq / Hkv). The reference's own attention IR is the single-head 2-D form; this 4-D form is how the
    batched grouped-query workload is written against the same statement vocabulary. Operands may be f16
    (widened by `copy` Assigns) or f32; the output is f32."""
    key_axis, dot_axis = outer.axis.name, inner.axis.name
    q = k = v = None
    for load in (s for s in inner.body if s.kind == 'Load'):
        if len(load.index) != 4:
            return None
        position, depth = ir.expression_vars(load.index[2]), ir.expression_vars(load.index[3])
        if dot_axis not in depth:
            return None
        if key_axis in position:
            k = load.input
        else:
            q = load.input
    for load in (s for s in outer.body if s.kind == 'Load'):
        if len(load.index) == 4 and key_axis in ir.expression_vars(load.index[2]):
            v = load.input
    writes = [s for s in tile.body if s.kind == 'Write']
    if None in (q, k, v) or len(writes) != 1 or len(writes[0].index) != 4:
        return None
    out = writes[0].output
    (batch, hq, s, d), k_shape, v_shape = _shape(specs, q), _shape(specs, k), _shape(specs, v)
    if k_shape != v_shape or k_shape[0] != batch or k_shape[2:] != (s, d) or _shape(specs, out) != (batch, hq, s, d):
        raise ValueError('grouped-query attention buffer shapes disagree')
    hkv = k_shape[1]
    if hkv == 0 or hq % hkv:
        raise ValueError('query heads must be a multiple of key/value heads')
    if outer.axis.extent.value != s or inner.axis.extent.value != d:
        raise ValueError('attention loop extents disagree with the buffer shapes')
    storage = {specs[name]['dtype'] for name in (q, k, v)}
    if len(storage) != 1 or specs[out]['dtype'] != 'f32':
        raise NotImplementedError('grouped-query attention takes q, k, v of one storage type and an f32 output')
    scale = _attention_scale(tile, outer, inner, specs)
    if scale is None:
        return None
    return Plan('gqa', {'batch': batch, 'hq': hq, 'hkv': hkv, 's': s, 'd': d, 'scale': scale, 'storage': storage.pop()},
                {'q': (q, 0), 'k': (k, 0), 'v': (v, 0), 'out': (out, 0)})


def _attention_scale(tile: ir.Node, outer_loop: ir.Node, inner_loop: ir.Node, specs: dict) -> float | None:
    outer, inner = [outer_loop], [inner_loop]
    # the uniform score scale: a Let literal that multiplies the score, or a one-element data buffer
    # the score is multiplied or divided by
    scale = None
    lets = {s.name: s for s in tile.body if s.kind == 'Let'}
    scalar_loads = {}
    for load in (s for s in tile.body if s.kind == 'Load'):
        if math.prod(_shape(specs, load.input)) == 1 and 'data' in specs[load.input]:
            for name in load.names:
                scalar_loads[name] = float(specs[load.input]['data'][0] if isinstance(specs[load.input]['data'], (list, tuple)) else specs[load.input]['data'])
    score_sums = {s.name for s in inner[0].body if s.kind == 'Accum'}
    for assign in (s for s in outer[0].body if s.kind == 'Assign'):
        op = _op_name(assign.op)
        if op in ('multiply', 'divide') and len(assign.args) == 2 and set(assign.args) & score_sums:
            other = next(a for a in assign.args if a not in score_sums) if len(set(assign.args) & score_sums) == 1 else None
            if other in lets and isinstance(lets[other].value, ir.Node) and lets[other].value.kind == 'Literal':
                value = float(lets[other].value.value)
            elif other in scalar_loads:
                value = scalar_loads[other]
            else:
                return None
            if op == 'divide':
                if assign.args[0] not in score_sums:
                    return None
                value = 1.0 / value
            scale = value
            break
    return 1.0 if scale is None else scale


# ------------------------------------------------------------------------------------------------
# row reductions
# ------------------------------------------------------------------------------------------------


def _classify_reduction(tile: ir.Node, specs: dict) -> Plan | None:
    """Row reductions and the fused row kernels built on them (classify_rows.py)."""
    return classify_rows(tile, specs, Plan)


# ------------------------------------------------------------------------------------------------
# elementwise / f16 storage
# ------------------------------------------------------------------------------------------------


def _flat_access(index: tuple, element_vars: dict[str, int], width: int, label: str) -> int | None:
    """Offset of a 1-D access `element * width + offset`, None for a constant (broadcast) index;
    raises when the access has another form."""
    if len(index) != 1:
        raise NotImplementedError(f'{label}: elementwise kernels take 1-D buffers')
    form = ir.affine(index[0])
    if form is None:
        raise NotImplementedError(f'{label}: index is not affine')
    coefficients, offset = form
    if not coefficients:
        return None
    if len(coefficients) != 1 or next(iter(coefficients)) not in element_vars or next(iter(coefficients.values())) != width:
        raise NotImplementedError(f'{label}: access is not a contiguous run of {width} elements per tile item')
    if offset < 0:
        raise ValueError(f'{label}: negative origin')
    return offset


def _classify_elementwise(tile: ir.Node, specs: dict) -> Plan | None:
    body = tuple(tile.body)
    element_vars = {axis.name: axis.extent.value for axis in tile.axes}
    count_items = math.prod(element_vars.values())
    if len(body) == 1 and body[0].kind == 'StridedLoop' and len(tile.axes) == 1:
        loop = body[0]
        # thread-strided walk over the items: the loop axis replaces the tile axis
        start = ir.affine(loop.start)
        if start is None or start[0] != {tile.axes[0].name: 1} or start[1] != 0:
            raise NotImplementedError('strided elementwise loops start at the tile item')
        element_vars = {loop.axis.name: loop.axis.extent.value}
        count_items = loop.axis.extent.value
        body = tuple(loop.body)
    if not body or any(s.kind not in ('Load', 'Assign', 'Write') for s in body):
        return None
    if len(element_vars) != 1:
        raise NotImplementedError('elementwise kernels use one tile axis')
    loads = [s for s in body if s.kind == 'Load']
    writes = [s for s in body if s.kind == 'Write']
    assigns = [s for s in body if s.kind == 'Assign']
    if len(writes) != 1 or not loads:
        return None
    write = writes[0]
    width = len(write.values)
    n = count_items * width
    out_offset = _flat_access(write.index, element_vars, width, write.output)
    if out_offset is None:
        raise NotImplementedError('elementwise output must advance with the tile item')
    # symbolic value of every name: ('load', buffer, lane) or ('op', name, args)
    values: dict[str, tuple] = {}
    origins: dict[str, int | None] = {}
    constants: dict[str, int] = {}
    for load in loads:
        offset = _flat_access(load.index, element_vars, len(load.names), load.input)
        if offset is None:
            constants[load.input] = ir.affine(load.index[0])[1]
            if not 0 <= constants[load.input] < math.prod(_shape(specs, load.input)):
                raise ValueError(f'{load.input}: constant index outside the buffer')
        if offset is not None and len(load.names) != width:
            raise NotImplementedError('vector loads and stores must have the same width')
        if origins.setdefault(load.input, offset) != offset:
            raise NotImplementedError('one origin per input buffer')
        for lane, name in enumerate(load.names):
            values[name] = ('load', load.input, lane if offset is not None else None)
    for assign in assigns:
        values[assign.name] = ('op', _op_name(assign.op), tuple(assign.args))

    def resolve(name: str, lane: int) -> tuple:
        if name not in values:
            raise ValueError(f'undefined value {name}')
        entry = values[name]
        if entry[0] == 'load':
            if entry[2] is not None and entry[2] != lane:
                raise NotImplementedError('elementwise lanes must not mix vector elements')
            return ('load', entry[1])
        op, args = entry[1], entry[2]
        if op == 'copy':
            return resolve(args[0], lane)
        return ('op', op, tuple(resolve(a, lane) for a in args))

    trees = {resolve(name, lane) for lane, name in enumerate(write.values)}
    if len(trees) != 1:
        raise NotImplementedError('every vector lane must compute the same expression')
    tree = trees.pop()
    out_dtype = specs[write.output]['dtype']
    check = [(write.output, out_offset)] + [(name, offset) for name, offset in origins.items() if offset is not None]
    for name, offset in check:
        if math.prod(_shape(specs, name)) < offset + n:
            raise ValueError(f'{name}: access runs past the end of the buffer')
    if tree[0] == 'load':
        source = tree[1]
        in_dtype = specs[source]['dtype']
        kind = {('f16', 'f16'): 'f16_copy', ('f16', 'f32'): 'f16_widen', ('f32', 'f16'): 'f16_narrow',
                ('f32', 'f32'): 'elementwise'}[(in_dtype, out_dtype)]
        params = {'n': n} if kind != 'elementwise' else {'op': 'copy', 'n': n}
        return Plan(kind, params, {'x': (source, origins[source]), 'out': (write.output, out_offset)})
    op, args = tree[1], tree[2]
    if op not in ELEMENTWISE_OPS:
        raise NotImplementedError(f'elementwise operation {op}')
    simple = (all(arg[0] == 'load' and origins[arg[1]] is not None and specs[arg[1]]['dtype'] == 'f32' for arg in args)
              and out_dtype == 'f32')
    if not simple:
        return _program_plan(tree, specs, origins, constants, write.output, out_offset, n)
    names = [arg[1] for arg in args]
    if op in BINARY_OPS:
        if len(names) != 2:
            raise ValueError(f'{op} takes two operands')
        return Plan('elementwise', {'op': op, 'n': n},
                    {'x': (names[0], origins[names[0]]), 'y': (names[1], origins[names[1]]), 'out': (write.output, out_offset)})
    if len(names) != 1:
        raise ValueError(f'{op} takes one operand')
    return Plan('elementwise', {'op': op, 'n': n}, {'x': (names[0], origins[names[0]]), 'out': (write.output, out_offset)})


PROGRAM_REGISTERS, PROGRAM_INSTRUCTIONS, PROGRAM_INPUTS = 8, 24, 6


def _program_plan(tree: tuple, specs: dict, origins: dict, constants: dict, output: str, out_offset: int, n: int) -> Plan:
    """Linearises an expression tree into the register program dtn_elementwise_program interprets.

    Inputs take registers 0..k-1 in order of first use; every operator result takes the lowest free
    register; a register is free again after the last instruction that reads it.
    """
    order: list[tuple] = []          # unique nodes, operands before users

    def visit(node: tuple) -> None:
        if node in order:
            return
        if node[0] == 'op':
            if node[1] not in ELEMENTWISE_OPS:
                raise NotImplementedError(f'elementwise operation {node[1]}')
            arity = 2 if node[1] in BINARY_OPS else 1
            if len(node[2]) != arity:
                raise ValueError(f'{node[1]} takes {arity} operand(s)')
            for operand in node[2]:
                visit(operand)
        order.append(node)

    visit(tree)
    inputs = [node for node in order if node[0] == 'load']
    operators = [node for node in order if node[0] == 'op']
    if len(inputs) > PROGRAM_INPUTS or len(operators) > PROGRAM_INSTRUCTIONS:
        raise NotImplementedError('elementwise expression is too large for the fused kernel')
    last_use = {}
    for position, node in enumerate(operators):
        for operand in node[2]:
            last_use[operand] = position
    register = {node: index for index, node in enumerate(inputs)}
    free = [r for r in range(PROGRAM_REGISTERS) if r >= len(inputs)]
    program = {'ops': [], 'dst': [], 'a': [], 'b': []}
    for position, node in enumerate(operators):
        sources = [register[operand] for operand in node[2]]
        for operand in set(node[2]):
            if last_use[operand] == position:
                free.append(register[operand])
        if not free:
            raise NotImplementedError('elementwise expression needs more than 8 live values')
        free.sort()
        target = free.pop(0)
        register[node] = target
        program['ops'].append(ELEMENTWISE_OPS[node[1]])
        program['dst'].append(target)
        program['a'].append(sources[0])
        program['b'].append(sources[-1])
    buffers = {'out': (output, out_offset)}
    described = []
    for index, node in enumerate(inputs):
        name = node[1]
        scalar = origins[name] is None
        buffers[f'in{index}'] = (name, constants[name] if scalar else origins[name])
        described.append({'f16': specs[name]['dtype'] == 'f16', 'scalar': scalar})
    params = {'n': n, 'inputs': described, 'out_reg': register[tree], 'out_f16': specs[output]['dtype'] == 'f16', **program}
    return Plan('elementwise_program', params, buffers)


# ------------------------------------------------------------------------------------------------


def classify(kernel: ir.Kernel, launch: dict, specs: dict, precision: str) -> Plan:
    """Returns the native plan of a validated kernel or raises NotImplementedError."""
    tile = _single_tile(kernel)
    for recogniser in (lambda: _classify_attention(tile, specs), lambda: _classify_gemm(tile, specs, precision, launch),
                       lambda: _classify_reduction(tile, specs), lambda: _classify_elementwise(tile, specs)):
        plan = recogniser()
        if plan is not None:
            return plan
    raise NotImplementedError(f'kernel {kernel.name}: no native sm_100a kernel matches this schedule')
