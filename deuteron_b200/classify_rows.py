"""Recognition of row kernels: a reduction over each row, an optional scalar stage on the reduced
value and an optional elementwise stage over the same row.

The scheduled IR of these kernels has one shape in the reference (compiler/transforms.py:62-95,
compiler/passes/regforward.py:88-148, compiler/passes/hybrid_normalizer.py:45-120): a Tile whose last
axis is the thread index, a thread-strided reduction loop with one Load and one or two Accum
statements, a WarpShuffle, a shared-memory round (Smem, Cond, Sync, TreeHalve), scalar Assign
statements, and then either a Write of one value per row or a second thread-strided loop that
reloads the row (one or four values at a time), applies Assign statements and writes the result.
A plain sum / max / sum of squares maps to the row-reduction kernel; everything else becomes a
register program for the fused row kernel (row softmax, RMS norm, L2 norm, mean).
"""
from __future__ import annotations

import math
from typing import Any

from . import ir
from .native import BINARY_OPS, ELEMENTWISE_OPS

ROW_REGISTERS, ROW_INSTRUCTIONS, ROW_INPUTS = 12, 32, 5
_COMMUTATIVE = frozenset(('add', 'multiply', 'maximum', 'minimum'))
_STATE0, _STATE1, _ELEMENT = ('state', 0), ('state', 1), ('x',)


def _op_name(op: Any) -> str:
    return op.name if isinstance(op, ir.Node) else str(op)


def _sym(op: str, *args: tuple) -> tuple:
    """Canonical expression node: commutative operands in a fixed order, copies removed."""
    if op == 'copy':
        return args[0]
    if op == 'exp_fast':
        op = 'exp'
    if op in _COMMUTATIVE:
        args = tuple(sorted(args, key=repr))
    return ('op', op, tuple(args))


def _is_var(expr: Any, name: str) -> bool:
    return isinstance(expr, ir.Node) and expr.kind == 'Var' and expr.name == name


def _thread_strided(loop: ir.Node, thread_axis: ir.Node) -> bool:
    start = ir.affine(loop.start)
    step = ir.affine(loop.step)
    return (loop.end is None and start is not None and start[0] == {thread_axis.name: 1} and start[1] == 0
            and step is not None and not step[0] and step[1] == thread_axis.extent.value)


def _row_index_ok(index: tuple, row_axes: list[ir.Node]) -> bool:
    """True when `index` names the row axes in order (axes of extent 1 may be a literal 0)."""
    if len(index) != len(row_axes):
        return False
    for expr, axis in zip(index, row_axes):
        if _is_var(expr, axis.name):
            continue
        form = ir.affine(expr)
        if axis.extent.value == 1 and form is not None and not form[0] and form[1] == 0:
            continue
        return False
    return True


def _constant_index(index: tuple) -> int | None:
    if len(index) != 1:
        return None
    form = ir.affine(index[0])
    if form is None or form[0]:
        return None
    return form[1]


class _Rows:
    """Symbolic walk over one row kernel."""

    def __init__(self, tile: ir.Node, specs: dict) -> None:
        self.tile, self.specs = tile, specs
        self.thread_axis = tile.axes[-1]
        self.row_axes = list(tile.axes[:-1])
        self.rows = math.prod(a.extent.value for a in self.row_axes)
        self.env: dict[str, tuple] = {}
        self.source: str | None = None
        self.cols = 0

    # -- reduction loop ------------------------------------------------------------------------
    def reduction(self, loop: ir.Node) -> str | None:
        """Consumes the reduction loop; returns 'sum', 'sumsq', 'max' or 'softmax' and leaves the state
        names bound to ('state', 0) / ('state', 1) in env."""
        loads = [s for s in loop.body if s.kind == 'Load']
        accums = [s for s in loop.body if s.kind == 'Accum']
        if len(loads) != 1 or len(loads[0].names) != 1 or not 1 <= len(accums) <= 2:
            return None
        if any(s.kind not in ('Load', 'Assign', 'Accum', 'Let') for s in loop.body):
            return None
        load = loads[0]
        if not load.index or not _is_var(load.index[-1], loop.axis.name) or not _row_index_ok(load.index[:-1], self.row_axes):
            raise NotImplementedError('row kernels read x[row axes..., column] with the loop variable as the column')
        self.source, self.cols = load.input, loop.axis.extent.value
        shape = tuple(self.specs[self.source]['shape'])
        expected = tuple(a.extent.value for a in self.row_axes) + (self.cols,)
        if math.prod(shape) != math.prod(expected) or shape[-1] != self.cols:
            raise ValueError(f'{self.source}: shape {list(shape)} does not match rows {self.rows} x columns {self.cols}')
        if self.specs[self.source]['dtype'] != 'f32':
            raise NotImplementedError('row kernels take f32 buffers')
        states = [a.name for a in accums]
        env = {name: ('old', name) for name in states}
        for stmt in loop.body:
            if stmt.kind == 'Load':
                env[stmt.names[0]] = _ELEMENT
            elif stmt.kind == 'Let':
                value = stmt.value
                if not (isinstance(value, ir.Node) and value.kind == 'Literal'):
                    return None
                env[stmt.name] = ('imm', float(value.value))
            elif stmt.kind == 'Assign':
                if any(a not in env for a in stmt.args):
                    raise ValueError(f'undefined value in {stmt.name}')
                env[stmt.name] = _sym(_op_name(stmt.op), *(env[a] for a in stmt.args))
            else:
                base = stmt.base or stmt.name
                if base not in env or stmt.value not in env:
                    raise ValueError(f'undefined value in accumulation {stmt.name}')
                env[stmt.name] = _sym(_op_name(stmt.op), env[base], env[stmt.value])
        if len(states) == 1:
            state = ('old', states[0])
            forms = {_sym('add', state, _ELEMENT): 'sum', _sym('maximum', state, _ELEMENT): 'max',
                     _sym('add', state, _sym('multiply', _ELEMENT, _ELEMENT)): 'sumsq'}
            kind = forms.get(env[states[0]])
            if kind is None:
                raise NotImplementedError('row reductions fold the value or its square with add, or the value with maximum')
            self.env = {states[0]: _STATE0}
            return kind
        for m, s in (states, states[::-1]):
            a, b = ('old', m), ('old', s)
            top = _sym('maximum', a, _ELEMENT)
            total = _sym('add', _sym('multiply', b, _sym('exp', _sym('subtract', a, top))), _sym('exp', _sym('subtract', _ELEMENT, top)))
            if env[m] == top and env[s] == total:
                self.env = {m: _STATE0, s: _STATE1}
                return 'softmax'
        raise NotImplementedError('a two-state row reduction must be the online maximum / sum of exponentials')

    # -- statements after the reduction ----------------------------------------------------------
    def scalar_statement(self, stmt: ir.Node) -> bool:
        """Binds a top-level Load of a constant element, a Let or an Assign; False for anything else."""
        if stmt.kind == 'Load':
            position = _constant_index(stmt.index)
            if position is None or len(stmt.names) != 1:
                return False
            if self.specs[stmt.input]['dtype'] != 'f32':
                raise NotImplementedError('row kernels take f32 buffers')
            if not 0 <= position < math.prod(self.specs[stmt.input]['shape']):
                raise ValueError(f'{stmt.input}: constant index outside the buffer')
            self.env[stmt.names[0]] = ('scalar', stmt.input, position)
            return True
        if stmt.kind == 'Let':
            if not (isinstance(stmt.value, ir.Node) and stmt.value.kind == 'Literal'):
                return False
            self.env[stmt.name] = ('imm', float(stmt.value.value))
            return True
        if stmt.kind == 'Assign':
            if any(a not in self.env for a in stmt.args):
                raise ValueError(f'undefined value in {stmt.name}')
            self.env[stmt.name] = _sym(_op_name(stmt.op), *(self.env[a] for a in stmt.args))
            return True
        return False

    def consumer(self, loop: ir.Node) -> tuple[str, tuple]:
        """The elementwise loop: returns (output buffer, expression of one output element)."""
        if not _thread_strided(loop, self.thread_axis):
            raise NotImplementedError('the elementwise loop of a row kernel is thread-strided like its reduction loop')
        writes = [s for s in loop.body if s.kind == 'Write']
        if len(writes) != 1 or any(s.kind not in ('Load', 'Assign', 'Let', 'Write') for s in loop.body):
            raise NotImplementedError('the elementwise loop of a row kernel holds loads, assignments and one store')
        width = len(writes[0].values)
        if loop.axis.extent.value * width != self.cols:
            raise ValueError('the elementwise loop does not cover the row')

        def column_form(expr: Any) -> bool:
            form = ir.affine(expr)
            return form is not None and form[0] == {loop.axis.name: width} and form[1] == 0

        lanes: dict[str, int | None] = {}
        env = dict(self.env)
        for stmt in loop.body:
            if stmt.kind == 'Load':
                if _constant_index(stmt.index) is not None:
                    saved, self.env = self.env, env
                    self.scalar_statement(stmt)
                    self.env = saved
                    lanes[stmt.names[0]] = None
                    continue
                if len(stmt.names) != width or not column_form(stmt.index[-1]):
                    raise NotImplementedError('loads of the elementwise loop move `width` consecutive columns per step')
                if stmt.input == self.source:
                    if not _row_index_ok(stmt.index[:-1], self.row_axes):
                        raise NotImplementedError('the elementwise loop reloads the row it reduced')
                    leaf = _ELEMENT
                else:
                    if len(stmt.index) != 1 or tuple(self.specs[stmt.input]['shape']) != (self.cols,):
                        raise NotImplementedError('extra vector inputs of a row kernel are indexed by the column alone')
                    if self.specs[stmt.input]['dtype'] != 'f32':
                        raise NotImplementedError('row kernels take f32 buffers')
                    leaf = ('columns', stmt.input)
                for lane, name in enumerate(stmt.names):
                    env[name], lanes[name] = leaf, lane
            elif stmt.kind == 'Let':
                if not (isinstance(stmt.value, ir.Node) and stmt.value.kind == 'Literal'):
                    raise NotImplementedError('Let statements of a row kernel bind literals')
                env[stmt.name], lanes[stmt.name] = ('imm', float(stmt.value.value)), None
            elif stmt.kind == 'Assign':
                if any(a not in env for a in stmt.args):
                    raise ValueError(f'undefined value in {stmt.name}')
                used = {lanes.get(a) for a in stmt.args} - {None}
                if len(used) > 1:
                    raise NotImplementedError('elementwise lanes must not mix vector elements')
                env[stmt.name] = _sym(_op_name(stmt.op), *(env[a] for a in stmt.args))
                lanes[stmt.name] = used.pop() if used else None
        write = writes[0]
        if write.atomic or not column_form(write.index[-1]) or not _row_index_ok(write.index[:-1], self.row_axes):
            raise NotImplementedError('a row kernel stores out[row axes..., column] without atomics')
        if any(v not in env for v in write.values):
            raise ValueError('undefined value in the store of the elementwise loop')
        if any(lanes.get(v) not in (None, lane) for lane, v in enumerate(write.values)):
            raise NotImplementedError('elementwise lanes must not mix vector elements')
        trees = {env[v] for v in write.values}
        if len(trees) != 1:
            raise NotImplementedError('every vector lane must compute the same expression')
        return write.output, trees.pop()


def _depends_on_element(node: tuple, memo: dict) -> bool:
    if node not in memo:
        if node == _ELEMENT or node[0] == 'columns':
            memo[node] = True
        elif node[0] == 'op':
            memo[node] = any(_depends_on_element(child, memo) for child in node[2])
        else:
            memo[node] = False
    return memo[node]


def _row_program(tree: tuple) -> dict:
    """Linearises `tree` into the register program of dtn_row_fused: scalar-stage instructions first."""
    order: list[tuple] = []

    def visit(node: tuple) -> None:
        if node in order:
            return
        if node[0] == 'op':
            if node[1] not in ELEMENTWISE_OPS:
                raise NotImplementedError(f'elementwise operation {node[1]}')
            arity = 2 if node[1] in BINARY_OPS else 1
            if len(node[2]) != arity:
                raise ValueError(f'{node[1]} takes {arity} operand(s)')
            for child in node[2]:
                visit(child)
        order.append(node)

    visit(tree)
    memo: dict = {}
    inputs = [n for n in order if n[0] in ('scalar', 'columns', 'imm')]
    scalar_ops = [n for n in order if n[0] == 'op' and not _depends_on_element(n, memo)]
    element_ops = [n for n in order if n[0] == 'op' and _depends_on_element(n, memo)]
    operators = scalar_ops + element_ops
    if len(inputs) > ROW_INPUTS or len(operators) > ROW_INSTRUCTIONS:
        raise NotImplementedError('row kernel expression is too large for the fused kernel')
    register: dict[tuple, int] = {_STATE0: 0, _STATE1: 1, _ELEMENT: 2}
    for index, node in enumerate(inputs):
        register[node] = 3 + index
    last_use: dict[tuple, int] = {}
    for position, node in enumerate(operators):
        for child in node[2]:
            last_use[child] = position
    # a scalar-stage value read by the elementwise stage must survive every element, so it is never recycled
    pinned = {child for node in element_ops for child in node[2] if child in scalar_ops}
    free = list(range(3 + len(inputs), ROW_REGISTERS))
    program = {'ops': [], 'dst': [], 'a': [], 'b': []}
    for position, node in enumerate(operators):
        sources = [register[child] for child in node[2]]
        for child in set(node[2]):
            if child[0] == 'op' and child not in pinned and last_use[child] == position:
                free.append(register[child])
        if not free:
            raise NotImplementedError(f'row kernel expression needs more than {ROW_REGISTERS} live values')
        free.sort()
        register[node] = free.pop(0)
        program['ops'].append(ELEMENTWISE_OPS[node[1]])
        program['dst'].append(register[node])
        program['a'].append(sources[0])
        program['b'].append(sources[-1])
    described = []
    for node in inputs:
        if node[0] == 'imm':
            described.append({'kind': 'immediate', 'value': node[1]})
        else:
            described.append({'kind': node[0], 'buffer': node[1], 'offset': node[2] if node[0] == 'scalar' else 0})
    return {'inputs': described, 'n_scalar': len(scalar_ops), 'out_reg': register[tree],
            'elementwise': bool(element_ops) or _depends_on_element(tree, memo), **program}


def classify_rows(tile: ir.Node, specs: dict, make_plan: Any) -> Any:
    """Plan of a row kernel, or None when the tile is not one. `make_plan(kind, params, buffers)` builds it."""
    body = list(tile.body)
    if not tile.axes or any(s.kind == 'CpAsyncCopy' for s in ir.walk([tile])):
        return None
    loops = [i for i, s in enumerate(body) if s.kind == 'StridedLoop']
    if not loops or not any(s.kind == 'Accum' for s in body[loops[0]].body):
        return None
    first = body[loops[0]]
    walk = _Rows(tile, specs)
    if not _thread_strided(first, walk.thread_axis):
        return None
    if any(s.kind not in ('Init', 'Smem') for s in body[:loops[0]]):
        return None
    reduce = walk.reduction(first)
    if reduce is None:
        return None
    shared = {s.name for s in body if s.kind == 'Smem'}
    output = tree = None
    for stmt in body[loops[0] + 1:]:
        if output is not None:
            raise NotImplementedError('statements after the store of a row kernel')
        if stmt.kind in ('WarpShuffle', 'TreeHalve'):
            if set(stmt.state) - set(walk.env):
                raise NotImplementedError('the shuffle / tree tail must combine the states of the reduction loop')
            continue
        if stmt.kind in ('Smem', 'Sync', 'Init'):
            continue
        if stmt.kind == 'Cond':
            inner = [s for s in stmt.body if s.kind == 'Write']
            if len(inner) == len(stmt.body) and inner and all(w.output in shared for w in inner) and not stmt.else_body:
                continue   # warp partials on their way to the tree
            if len(stmt.body) == 1 and inner and not stmt.else_body:
                stmt = inner[0]   # a guarded store of the per-row result
            else:
                raise NotImplementedError('conditionals of a row kernel guard the stores of partials or of the result')
        if stmt.kind == 'Write':
            if len(stmt.values) != 1 or stmt.atomic or stmt.values[0] not in walk.env:
                raise NotImplementedError('a row kernel stores one value per row without atomics')
            if not (_row_index_ok(stmt.index, walk.row_axes) or (walk.rows == 1 and _constant_index(stmt.index) == 0)):
                raise NotImplementedError('the per-row result is stored at out[row axes...]')
            output, tree = stmt.output, walk.env[stmt.values[0]]
            if math.prod(specs[output]['shape']) != walk.rows:
                raise ValueError(f'{output}: one value per row expected')
            continue
        if stmt.kind == 'StridedLoop':
            output, tree = walk.consumer(stmt)
            if math.prod(specs[output]['shape']) != walk.rows * walk.cols or tuple(specs[output]['shape'])[-1] != walk.cols:
                raise ValueError(f'{output}: shape does not match the reduced buffer')
            continue
        if not walk.scalar_statement(stmt):
            raise NotImplementedError(f'{stmt.kind} is outside the row kernels this build recognises')
    if output is None:
        return None
    if specs[output]['dtype'] != 'f32':
        raise NotImplementedError('row kernels take f32 buffers')
    if tree == _STATE0 and reduce != 'softmax':
        return make_plan('row_reduce', {'op': reduce, 'rows': walk.rows, 'cols': walk.cols}, {'x': (walk.source, 0), 'out': (output, 0)})
    program = _row_program(tree)
    per_row = not program.pop('elementwise')
    if per_row and math.prod(specs[output]['shape']) != walk.rows:
        raise ValueError(f'{output}: the stored value does not depend on the column')
    if not per_row and math.prod(specs[output]['shape']) != walk.rows * walk.cols:
        raise ValueError(f'{output}: an elementwise result needs a full-size output')
    buffers = {'x': (walk.source, 0), 'out': (output, 0)}
    for index, item in enumerate(program['inputs']):
        if item['kind'] != 'immediate':
            buffers[f'in{index}'] = (item.pop('buffer'), item.pop('offset'))
    params = {'reduce': reduce, 'rows': walk.rows, 'cols': walk.cols, 'per_row': per_row, **program}
    return make_plan('row_fused', params, buffers)
