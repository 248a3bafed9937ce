"""Front-end checks with the contract of the reference's compiler/validation.py.

`validate_launch` and `validate_kernel_launch` accept and reject the same meta.json launches
(compiler/validation.py:52-174) and raise the same exception types: ValueError for malformed
input, NotImplementedError for well-formed input outside the backend subset.
"""
from __future__ import annotations

import json
import math
from typing import Any

from . import ir
from .options import Options

_DTYPES = {'f16': 2, 'f32': 4, 'f64': 8, 'i32': 4, 'i64': 8}
ARCHITECTURES = ('sm_100a', 'sm_100')


def validate_compile_arguments(arch: Any, opt_level: Any, options: Any) -> Options:
    """Checks the keyword arguments of compile_kernel and returns the Options to use. The accepted values are those of
    compiler/validation.py:22-32 with the target list reduced to the one this build serves; everything else is a
    ValueError. A frozen Options object that was mutated behind its back is checked again."""
    problems = (
        (type(arch) is str and arch in ARCHITECTURES,
         f'unsupported target {arch!r}; this build emits sm_100a kernels only (use sm_100a)'),
        (type(opt_level) is int and 0 <= opt_level <= 3, 'optimization level must be an integer 0, 1, 2, or 3'),
        (options is None or isinstance(options, Options), 'options must be an Options instance or None'),
    )
    for accepted, message in problems:
        if not accepted:
            raise ValueError(message)
    chosen = Options() if options is None else options
    chosen.__post_init__()
    return chosen


# ------------------------------------------------------------------------------------------------
# meta.json launch schema (accept / reject sets of compiler/validation.py:52-100)
# ------------------------------------------------------------------------------------------------

_DIMENSION_LIMITS = {'grid': (2**31 - 1, 65535, 65535), 'block': (1024, 1024, 64)}
_ARGUMENT_FLAGS = ('scalar', 'output', 'intermediate')


def _text(value: Any, what: str) -> str:
    """A usable identifier: a non-empty str with no NUL in it."""
    if type(value) is str and value and '\x00' not in value:
        return value
    raise ValueError(f'{what} must be a nonempty string without NUL bytes')


def _listing(value: Any, what: str) -> list | tuple:
    if isinstance(value, (list, tuple)):
        return value
    raise ValueError(f'{what} must be a list or tuple')


def _strict_int(value: Any, low: int, high: int) -> bool:
    """bool is not an int here, and neither is 32.0."""
    return type(value) is int and low <= value <= high


def _check_geometry(launch: dict) -> None:
    for field, limits in _DIMENSION_LIMITS.items():
        dims = _listing(launch.get(field), field)
        if len(dims) != 3 or not all(_strict_int(extent, 1, limit) for extent, limit in zip(dims, limits)):
            raise ValueError(f'{field} must contain three positive integer CUDA dimensions within {limits}')
    if math.prod(launch['block']) > 1024:
        raise ValueError('block must contain at most 1024 threads')
    if not _strict_int(launch.get('smem_bytes', 0), 0, 2**32 - 1):
        raise ValueError('smem_bytes must be a nonnegative 32-bit integer')


def _check_argument(arg: Any) -> str:
    if not isinstance(arg, dict):
        raise ValueError('each argument must be an object')
    name = _text(arg.get('name'), 'argument name')
    dtype = arg.get('dtype')
    if type(dtype) is not str or dtype not in _DTYPES:
        raise ValueError(f'unsupported argument dtype {dtype!r}')
    flags = {flag: arg[flag] for flag in _ARGUMENT_FLAGS if flag in arg}
    for flag, value in flags.items():
        if type(value) is not bool:
            raise ValueError(f'argument {flag} must be a boolean')
    if flags.get('scalar'):
        if flags.get('output') or flags.get('intermediate'):
            raise ValueError('scalar arguments cannot be output or intermediate buffers')
        return name
    shape = _listing(arg.get('shape'), f'{name} shape')
    if not all(_strict_int(extent, 0, 2**63 - 1) for extent in shape):
        raise ValueError('buffer shapes require nonnegative 64-bit integer extents')
    if math.prod(shape) * _DTYPES[dtype] >= 2**64:
        raise ValueError('buffer byte size does not fit a 64-bit address space')
    return name


def validate_launch(launch: Any) -> dict[str, Any]:
    """Checks one `kernels[]` entry of a meta.json and returns its argument specs keyed by name. Tuples are accepted
    wherever lists are, and empty buffers are legal (tests/test_validation.py of the reference)."""
    if not isinstance(launch, dict):
        raise ValueError('launch metadata must be an object')
    _text(launch.get('entry'), 'launch entry')
    _check_geometry(launch)
    by_name: dict[str, Any] = {}
    for arg in _listing(launch.get('args'), 'args'):
        name = _check_argument(arg)
        if name in by_name:
            raise ValueError('meta.json args and arg_order disagree: duplicate argument name')
        by_name[name] = arg
    order = [_text(name, 'arg_order name') for name in _listing(launch.get('arg_order'), 'arg_order')]
    if sorted(order) != sorted(by_name):       # same names, each exactly once
        raise ValueError('meta.json args and arg_order disagree')
    resets = [_text(name, 'zero_outputs name') for name in _listing(launch.get('zero_outputs', ()), 'zero_outputs')]
    for name in resets:
        spec = by_name.get(name)
        if spec is None or spec.get('scalar') or not spec.get('output'):
            raise ValueError('zero_outputs must name output buffers')
    if len(set(resets)) < len(resets):
        raise ValueError('zero_outputs cannot contain duplicate names')
    return by_name


# ------------------------------------------------------------------------------------------------
# backend subset on the parsed kernel (accept / reject sets of compiler/validation.py:103-174)
# ------------------------------------------------------------------------------------------------

class _KernelChecker:
    """Walks the statements of one kernel once per pass and applies the check registered for each statement kind.
    ValueError = malformed, NotImplementedError = well-formed but outside what the backend takes."""

    def __init__(self, specs: dict[str, Any], launch: dict) -> None:
        self.specs, self.launch = specs, launch
        self.shared: dict[str, ir.Node] = {}
        self.threads = math.prod(launch['block'])

    # -- buffers ---------------------------------------------------------------------------------

    def declare_shared(self, stmt: ir.Node) -> None:
        name = _text(stmt.name, 'shared buffer name')
        if name in self.specs or name in self.shared:
            raise ValueError(f'duplicate buffer name {name}')
        extents = _listing(stmt.extents, 'shared extents')
        if not all(_strict_int(extent, 0, 2**63) for extent in extents) or math.prod(extents) > 2**31:
            raise ValueError('shared extents must fit signed 32-bit indexing')
        align = stmt.align
        if not _strict_int(align, 0, 2**63) or align & (align - 1):
            raise ValueError('shared alignment must be zero or a power of two')
        self.shared[name] = stmt

    def _access(self, name: Any, index: Any, stores: bool) -> None:
        if name in self.specs:
            shape = self.specs[name]['shape']
        elif name in self.shared:
            shape = self.shared[name].extents
        else:
            raise ValueError(f'unknown buffer {name}')
        scalar_cell = not index and math.prod(shape) == 1
        if len(index) != len(shape) and not scalar_cell:
            raise ValueError(f'{name}: index rank does not match its shape')
        if stores and name in self.specs and not self.specs[name].get('output'):
            raise NotImplementedError(f'ordinary global stores require output buffers: {name}')

    # -- statements ------------------------------------------------------------------------------

    def _axis(self, axis: Any) -> int:
        if not isinstance(axis, ir.Node) or axis.kind != 'Axis':
            raise ValueError('loop axes must be Axis nodes')
        _text(axis.name, 'axis name')
        extent = axis.extent.value if isinstance(axis.extent, ir.Node) and axis.extent.kind == 'Dim' else None
        if not _strict_int(extent, 0, 2**31 - 1):
            raise NotImplementedError('axis extents must be nonnegative signed 32-bit integers')
        return extent

    def tile(self, stmt: ir.Node) -> None:
        extents = [self._axis(axis) for axis in stmt.axes]
        names = [axis.name for axis in stmt.axes]
        if not extents or 0 in extents or len(set(names)) != len(names):
            raise ValueError('Tile requires distinct axes with positive extents')
        declared = stmt.block_threads
        if declared is not None and not (type(declared) is int and declared == self.launch['block'][0]):
            raise ValueError('Tile block_threads disagrees with the launch')

    def loop(self, stmt: ir.Node) -> None:
        self._axis(stmt.axis)

    def strided_loop(self, stmt: ir.Node) -> None:
        self._axis(stmt.axis)
        if ir.kind(stmt.step) == 'Literal' and not _strict_int(stmt.step.value, 1, 2**63):
            raise ValueError('StridedLoop requires a positive integer step')

    def load(self, stmt: ir.Node) -> None:
        self._access(stmt.input, stmt.index, stores=False)

    def write(self, stmt: ir.Node) -> None:
        self._access(stmt.output, stmt.index, stores=True)

    def async_copy(self, stmt: ir.Node) -> None:
        self._access(stmt.src, stmt.src_index, stores=False)
        self._access(stmt.smem, stmt.smem_index, stores=True)
        if stmt.src not in self.specs or stmt.smem not in self.shared:
            raise ValueError('cp.async requires global source and shared destination')
        if type(stmt.nbytes) is not int or stmt.nbytes not in (4, 8, 16):
            raise ValueError('cp.async copy size must be 4, 8, or 16')

    def async_wait(self, stmt: ir.Node) -> None:
        if not _strict_int(stmt.group, 0, 7):
            raise ValueError('cp.async wait group must be an integer from 0 to 7')

    def barrier(self, stmt: ir.Node) -> None:
        if not _strict_int(stmt.barrier_id, 0, 15) or type(stmt.warp) is not bool:
            raise ValueError('barrier id must be 0..15 and warp must be boolean')
        if stmt.warp and stmt.barrier_id:
            raise ValueError('warp synchronization cannot use a named barrier')
        if stmt.count is None:
            if stmt.barrier_id:
                raise ValueError('named barrier requires a thread count')
        elif not _strict_int(stmt.count, 1, self.threads) or stmt.count % 32:
            raise ValueError('barrier count must be a positive multiple of 32 within the block')

    CHECKS = {'Tile': tile, 'Loop': loop, 'StridedLoop': strided_loop, 'Load': load, 'Write': write,
              'CpAsyncCopy': async_copy, 'CpAsyncWait': async_wait, 'Sync': barrier}

    def run(self, kernel: ir.Kernel) -> None:
        statements = tuple(ir.walk(kernel.body))
        for stmt in statements:                     # shared buffers first: a copy may precede the declaration in the text
            if stmt.kind == 'Smem':
                self.declare_shared(stmt)
        for stmt in statements:
            check = self.CHECKS.get(stmt.kind)
            if check is not None:
                check(self, stmt)


def validate_kernel_launch(kernel: ir.Kernel, launch: Any) -> dict[str, Any]:
    """The launch schema plus what the backend takes: a linear launch of a kernel without serial axes, f16 / f32
    buffers of at most 2^31 elements, and statements whose buffers, ranks, axes, copies and barriers are coherent."""
    specs = validate_launch(launch)
    if launch['entry'] != kernel.name:
        raise ValueError('launch entry and kernel name disagree')
    if any(extent != 1 for extent in (*launch['grid'][1:], *launch['block'][1:])):
        raise NotImplementedError('only linear launches are supported')
    if kernel.serial:
        raise NotImplementedError('serial launch axes are outside the supported subset')
    for spec in specs.values():
        if spec.get('scalar') or spec['dtype'] not in ('f16', 'f32'):
            raise NotImplementedError('the backend accepts f16/f32 buffer arguments')
        if math.prod(spec['shape']) > 2**31:
            raise NotImplementedError('buffer element count exceeds signed 32-bit indexing')
    _KernelChecker(specs, launch).run(kernel)
    return specs


def _json(payload: Any, label: str) -> Any:
    """JSON object with duplicate keys rejected (compiler/validation.py:209-223)."""
    def unique(pairs: Any) -> Any:
        result = {}
        for key, value in pairs:
            if key in result:
                raise ValueError(f'duplicate JSON key {key!r}')
            result[key] = value
        return result
    if isinstance(payload, dict):
        return payload
    try:
        result = json.loads(payload, object_pairs_hook=unique)
        if not isinstance(result, dict):
            raise ValueError('expected an object')
        return result
    except (TypeError, ValueError, RecursionError) as exc:
        raise ValueError(f'invalid {label}: {exc}') from exc


def parse_kernel(payload: Any, meta_payload: Any) -> tuple[ir.Kernel, dict]:
    """IR JSON + meta.json (text, bytes or already-decoded objects) -> (kernel, launch).

    Exactly one KernelOp node and exactly one launch whose entry equals its name
    (compiler/validation.py:226-258).
    """
    data, metadata = _json(payload, 'IR JSON'), _json(meta_payload, 'metadata JSON')
    try:
        if not isinstance(data['nodes'], dict) or any(not isinstance(node, dict) for node in data['nodes'].values()):
            raise ValueError('graph nodes must be objects')
        kernels = [node for node in data['nodes'].values() if node.get('op') == 'KernelOp']
        if len(kernels) != 1:
            raise ValueError('expected exactly one KernelOp in the input graph')
        fields = kernels[0].get('op_fields', {})
        if not isinstance(fields, dict) or set(fields) - {'body', 'name', 'zero_delegated', 'serial'}:
            raise ValueError('unsupported KernelOp fields')
        _text(fields.get('name'), 'kernel name')
        body = _listing(fields.get('body', ()), 'KernelOp body')
        serial = _listing(fields.get('serial', ()), 'KernelOp serial')
        delegated = _listing(fields.get('zero_delegated', ()), 'KernelOp zero_delegated')
        for name in delegated:
            _text(name, 'zero_delegated name')
        statements = tuple(ir.parse_statement(item) for item in body)
        for stmt in statements:
            if not isinstance(stmt, ir.Node) or stmt.kind not in ir.STATEMENTS:
                raise ValueError('KernelOp body entries must be IR statements')
        kernel = ir.Kernel(fields['name'], statements, tuple(delegated), tuple(ir.parse_statement(item) for item in serial))
        launches = _listing(metadata['kernels'], 'metadata kernels')
        if any(not isinstance(launch, dict) for launch in launches):
            raise ValueError('metadata kernels must contain objects')
        matches = [launch for launch in launches if launch.get('entry') == kernel.name]
        if len(matches) != 1:
            raise ValueError(f'meta.json must contain exactly one launch for {kernel.name}')
        launch = matches[0]
        validate_kernel_launch(kernel, launch)
        return kernel, launch
    except (KeyError, TypeError, AttributeError, IndexError, RecursionError, OverflowError) as exc:
        raise ValueError(f'invalid scheduled Kernel IR or launch metadata: {exc}') from exc
