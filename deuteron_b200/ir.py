"""Scheduled Kernel IR: a restricted parser for the constructor strings in `op_fields.body`.

The reference evaluates each body string with an `ast` walker that only calls whitelisted IR
constructors of the external emmy package (compiler/validation.py:177-206). This module accepts the
same grammar without emmy: every constructor becomes a `Node(kind, fields)` whose fields are named
after the emmy dataclass fields the reference's compiler reads (compiler/codegen/lower.py).
"""
from __future__ import annotations

import ast
import math
from typing import Any, Iterator

# Positional field order of each accepted constructor. Dataclass reprs print keywords, but a few
# emmy reprs (`Dim(515)`, `ElementwiseImpl('add')`, `dtype('float32')`) and hand-written IR use
# positions.
FIELDS: dict[str, tuple[str, ...]] = {
    'Dim': ('value',),
    'DataType': ('name', 'np', 'nbytes'),
    'StructuredType': ('name', 'fields'),
    'dtype': ('name',),
    'Axis': ('name', 'extent', 'window'),
    'Window': ('parent', 'base', 'bound', 'partition'),
    'BinaryExpr': ('op', 'left', 'right'),
    'Builtin': ('name',),
    'CastExpr': ('expr', 'dtype'),
    'FlatIndex': ('buffer', 'index'),
    'FuncCallExpr': ('name', 'args'),
    'Literal': ('value', 'dtype'),
    'TernaryExpr': ('cond', 'if_true', 'if_false'),
    'Var': ('name',),
    'CpAsyncCommit': (),
    'CpAsyncCopy': ('smem', 'smem_index', 'src', 'src_index', 'nbytes', 'swizzle', 'lane_index', 'lane_rows'),
    'CpAsyncWait': ('group',),
    'Smem': ('name', 'extents', 'dtype', 'align'),
    'Sync': ('barrier_id', 'count', 'warp'),
    'Tile': ('axes', 'body', 'block_threads', 'aux_threads', 'raster_axes', 'raster_group', 'raster_orient'),
    'TreeHalve': ('bufs', 'state', 'state_b', 'combine_states', 'length', 'tid_var', 'inner', 'barrier_id',
                  'barrier_count', 'dtype'),
    'WarpShuffle': ('state', 'state_b', 'combine_states', 'length', 'dtype'),
    'Accum': ('name', 'value', 'op', 'dtype', 'axes', 'base'),
    'Assign': ('name', 'op', 'args', 'dtype'),
    'Body': ('stmts',),
    'Cond': ('cond', 'body', 'else_body'),
    'Init': ('name', 'identity', 'dtype'),
    'Let': ('name', 'value', 'dtype'),
    'Load': ('names', 'input', 'index', 'dtype'),
    'Loop': ('axis', 'body', 'unroll', 'seed'),
    'Select': ('name', 'branches'),
    'SelectBranch': ('value', 'select'),
    'StridedLoop': ('axis', 'start', 'step', 'body', 'unroll', 'end', 'seed'),
    'Write': ('output', 'index', 'values', 'value_dtype', 'atomic', 'swizzle'),
    'ElementwiseImpl': ('name',),
}

DEFAULTS: dict[str, dict[str, Any]] = {
    'Axis': {'window': None},
    'Window': {'base': None, 'bound': None, 'partition': False},
    'Literal': {'dtype': 'int'},
    'CpAsyncCopy': {'swizzle': 'NONE', 'lane_index': None, 'lane_rows': None},
    'Smem': {'dtype': 'float', 'align': 0},
    'Sync': {'barrier_id': 0, 'count': None, 'warp': False},
    'Tile': {'block_threads': None, 'aux_threads': 0, 'raster_axes': None, 'raster_group': None, 'raster_orient': 'm'},
    'TreeHalve': {'state_b': None, 'combine_states': None, 'tid_var': None, 'inner': None, 'barrier_id': 0,
                  'barrier_count': None, 'dtype': None},
    'WarpShuffle': {'state_b': None, 'combine_states': None, 'length': 32, 'dtype': None},
    'Accum': {'dtype': None, 'axes': (), 'base': None},
    'Assign': {'dtype': None},
    'Cond': {'else_body': ()},
    'Init': {'dtype': None},
    'Let': {'dtype': None},
    'Load': {'dtype': None},
    'Loop': {'unroll': None, 'seed': False},
    'StridedLoop': {'unroll': None, 'end': None, 'seed': False},
    'Write': {'value_dtype': None, 'atomic': False, 'swizzle': 'NONE'},
    'DataType': {'np': None, 'nbytes': None},
    'StructuredType': {'fields': ()},
}

STATEMENTS = frozenset(('Tile', 'Loop', 'StridedLoop', 'Load', 'Assign', 'Accum', 'Init', 'Let', 'Write', 'Smem',
                        'CpAsyncCopy', 'CpAsyncCommit', 'CpAsyncWait', 'Sync', 'WarpShuffle', 'TreeHalve', 'Select',
                        'Cond'))


class Node:
    """One IR constructor call: `kind` is the constructor name, fields are attributes."""

    __slots__ = ('kind', 'fields')

    def __init__(self, kind: str, fields: dict[str, Any]) -> None:
        self.kind = kind
        self.fields = fields

    def __getattr__(self, name: str) -> Any:
        try:
            return self.fields[name]
        except KeyError:
            raise AttributeError(f'{self.kind} has no field {name!r}') from None

    def __repr__(self) -> str:
        return f"{self.kind}({', '.join(f'{k}={v!r}' for k, v in self.fields.items())})"

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Node) and self.kind == other.kind and self.fields == other.fields

    def __hash__(self) -> int:
        return hash((self.kind, repr(self.fields)))


def _construct(kind: str, args: list[Any], kwargs: dict[str, Any]) -> Any:
    order = FIELDS[kind]
    if len(args) > len(order):
        raise ValueError(f'{kind} takes at most {len(order)} positional arguments')
    fields = dict(DEFAULTS.get(kind, {}))
    for name, value in zip(order, args):
        fields[name] = value
    for name, value in kwargs.items():
        if kind == 'Load' and name == 'name':  # emmy accepts Load(name=...) for a one-value load
            fields['names'] = (value,)
            continue
        if name not in order:
            raise ValueError(f'{kind} has no field {name!r}')
        if name in order[:len(args)]:
            raise ValueError(f'{kind} got {name!r} twice')
        fields[name] = value
    missing = [name for name in order if name not in fields]
    if missing:
        raise ValueError(f'{kind} is missing {missing}')
    if kind == 'dtype':
        return str(fields['name'])
    if kind == 'Body':
        return tuple(fields['stmts'])
    if kind == 'Dim':
        if type(fields['value']) is not int:
            raise NotImplementedError('axis extents must be concrete integers')
    if kind == 'Load':
        names = fields['names']
        fields['names'] = (names,) if isinstance(names, str) else tuple(names)
    if kind == 'Write':
        values = fields['values']
        fields['values'] = (values,) if isinstance(values, str) else tuple(values)
    if kind in ('Assign', 'Accum') and isinstance(fields['op'], str):  # emmy coerces operator names
        fields['op'] = Node('ElementwiseImpl', {'name': fields['op']})
    if kind == 'Assign':
        args_field = fields['args']
        fields['args'] = (args_field,) if isinstance(args_field, str) else tuple(args_field)
    ordered = {name: fields[name] for name in order}
    return Node(kind, ordered)


def parse_statement(text: Any) -> Any:
    """Parses one constructor string; raises ValueError for anything outside the grammar."""
    if type(text) is not str:
        raise ValueError('IR statements must be constructor strings')

    def parse(node: ast.AST) -> Any:
        if isinstance(node, ast.Constant) and type(node.value) in (str, int, float, bool, type(None)):
            return node.value
        if isinstance(node, (ast.List, ast.Tuple)):
            values = [parse(item) for item in node.elts]
            return tuple(values) if isinstance(node, ast.Tuple) else values
        if isinstance(node, ast.Dict) and all(key is not None for key in node.keys):
            return {parse(key): parse(value) for key, value in zip(node.keys, node.values)}
        if isinstance(node, ast.Name) and node.id in ('inf', 'nan'):
            return math.inf if node.id == 'inf' else math.nan
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.UAdd, ast.USub)):
            value = parse(node.operand)
            if type(value) in (int, float):
                return -value if isinstance(node.op, ast.USub) else value
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in FIELDS:
            keywords = node.keywords
            if any(k.arg is None for k in keywords) or len({k.arg for k in keywords}) != len(keywords):
                raise ValueError('IR constructors require distinct explicit keyword arguments')
            return _construct(node.func.id, [parse(a) for a in node.args], {k.arg: parse(k.value) for k in keywords})
        raise ValueError('IR accepts only known constructors, literals, and literal containers')

    try:
        return parse(ast.parse(text, mode='eval').body)
    except (SyntaxError, TypeError, AttributeError, KeyError, IndexError, RecursionError, OverflowError) as exc:
        raise ValueError(f'invalid IR constructor expression: {exc}') from exc


class Kernel:
    """The parsed KernelOp: name, body statements, zero_delegated and serial lists."""

    def __init__(self, name: str, body: tuple, zero_delegated: tuple = (), serial: tuple = ()) -> None:
        self.name = name
        self.body = body
        self.zero_delegated = zero_delegated
        self.serial = serial


def kind(node: Any) -> str:
    return node.kind if isinstance(node, Node) else type(node).__name__


def children(stmt: Node) -> tuple:
    """Nested statement bodies of a block statement."""
    if stmt.kind in ('Tile', 'Loop', 'StridedLoop'):
        return tuple(stmt.body)
    if stmt.kind == 'Cond':
        return tuple(stmt.body) + tuple(stmt.else_body or ())
    return ()


def walk(body: Any) -> Iterator[Node]:
    """Every statement of a body, depth first, parents before children."""
    for stmt in body:
        if isinstance(stmt, Node):
            yield stmt
            yield from walk(children(stmt))


def axis_extent(axis: Any) -> int:
    """Static extent of an Axis node (Axis(name, extent=Dim(n), window))."""
    extent = axis.extent
    return int(extent.value) if isinstance(extent, Node) else int(extent)


def expression_vars(expr: Any) -> set[str]:
    """Names of the Var nodes inside an index expression."""
    found: set[str] = set()

    def visit(value: Any) -> None:
        if isinstance(value, Node):
            if value.kind == 'Var':
                found.add(value.name)
            for field in value.fields.values():
                visit(field)
        elif isinstance(value, (tuple, list)):
            for item in value:
                visit(item)

    visit(expr)
    return found


def affine(expr: Any) -> tuple[dict[str, int], int] | None:
    """Coefficients and constant of an integer expression that is affine in its Vars, else None.

    Covers what index expressions of elementwise kernels use: + - * with literals
    (compiler/analysis.py:62-110 normalises the same forms).
    """
    if isinstance(expr, bool):
        return None
    if isinstance(expr, int):
        return {}, expr
    if not isinstance(expr, Node):
        return None
    if expr.kind == 'Literal':
        return ({}, expr.value) if type(expr.value) is int else None
    if expr.kind == 'Var':
        return {expr.name: 1}, 0
    if expr.kind == 'BinaryExpr' and expr.op in ('+', '-', '*'):
        left, right = affine(expr.left), affine(expr.right)
        if left is None or right is None:
            return None
        (lc, lk), (rc, rk) = left, right
        if expr.op == '*':
            if lc and rc:
                return None
            if rc:
                lc, lk, rc, rk = rc, rk, lc, lk
            return {name: c * rk for name, c in lc.items() if c * rk}, lk * rk
        sign = 1 if expr.op == '+' else -1
        merged = dict(lc)
        for name, c in rc.items():
            merged[name] = merged.get(name, 0) + sign * c
        return {name: c for name, c in merged.items() if c}, lk + sign * rk
    return None
