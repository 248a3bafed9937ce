"""ctypes binding of libdeuteron_b200.so (the C ABI declared in include/deuteron_b200.h).

The library is the product's only compute path: if it is missing or fails to load, importing this
module's `lib()` raises. There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as ct
import threading
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / 'libdeuteron_b200.so'

OK, ERR_INVALID, ERR_CUDA, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_DEVICE = range(6)

GEMM_MODES = {'f32': 0, 'tf32x3': 1, 'bf16x3': 2, 'f32_splitk': 3}
REDUCE_OPS = {'sum': 0, 'max': 1, 'sumsq': 2, 'softmax': 3}
ROW_INPUT_KINDS = {'scalar': 0, 'columns': 1, 'immediate': 2}
STORAGE = {'f32': 0, 'f16': 1}
ELEMENTWISE_OPS = {
    'add': 0, 'subtract': 1, 'multiply': 2, 'divide': 3, 'maximum': 4, 'minimum': 5, 'relu': 6, 'exp': 7,
    'sqrt': 8, 'rsqrt': 9, 'reciprocal': 10, 'negative': 11, 'absolute': 12, 'copy': 13, 'exp_fast': 7,
}
BINARY_OPS = frozenset(('add', 'subtract', 'multiply', 'divide', 'maximum', 'minimum'))


class CudaError(RuntimeError):
    """A CUDA call inside the library failed (mirrors benchmark.py:31-32 of the reference)."""


class DeviceWaitError(RuntimeError):
    """A kernel's bounded wait ran out and the kernel returned early with a status code."""


_I64, _P, _F, _I = ct.c_int64, ct.c_void_p, ct.c_float, ct.c_int
_SIGNATURES = {
    'dtn_version': [],
    'dtn_last_error': [ct.c_char_p, ct.c_size_t],
    'dtn_device_status': [ct.POINTER(ct.c_int), _P],
    'dtn_selftest_wait_timeout': [ct.c_longlong, _P],
    'dtn_copy_block': [_P, ct.c_size_t, _P, ct.c_size_t, ct.c_size_t, ct.c_size_t, _I, _P],
    'dtn_capture_begin': [_P],
    'dtn_capture_end': [_P, ct.POINTER(ct.c_int), ct.POINTER(ct.c_int), ct.POINTER(ct.c_int), ct.POINTER(ct.c_int)],
    'dtn_add_f32': [_P, _P, _P, _I64, _P],
    'dtn_elementwise_f32': [_I, _P, _P, _P, _I64, _P],
    'dtn_elementwise_program': [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _P, _I, _I64, _P],
    'dtn_f16_copy': [_P, _P, _I64, _P],
    'dtn_push_block': [_P, _I64, ct.POINTER(ct.c_void_p), _I, _I64, _I64, _I64, _P],
    'dtn_f16_widen': [_P, _P, _I64, _P],
    'dtn_f16_narrow': [_P, _P, _I64, _P],
    'dtn_row_reduce_f32': [_I, _P, _P, _I64, _I64, _I64, _P],
    'dtn_row_fused': [_I, _P, _I64, _I64, _I64, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _P, _I64, _P],
    'dtn_gemm_workspace_bytes': [_I, _I64, _I64, _I64, ct.POINTER(ct.c_size_t)],
    'dtn_gemm_x3': [_I, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P, ct.c_size_t, _P],
    'dtn_gemm_x3_phase': [_I, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P, ct.c_size_t, _I, _P],
    'dtn_gemm_x3_static': [_I, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    'dtn_gemm_x3_static_status': [ct.POINTER(ct.c_int), _P],
    'dtn_gemm_tile_schedule': [_I64, _I64, _I, ct.POINTER(ct.c_uint32), _I, ct.POINTER(ct.c_int), ct.POINTER(ct.c_double),
                               ct.POINTER(ct.c_double)],
    'dtn_gemm_skinny_plan': [_I64, _I64, _I, ct.POINTER(ct.c_int64), ct.POINTER(ct.c_int), ct.POINTER(ct.c_int)],
    'dtn_gemm_set_variant': [_I],
    'dtn_attention_f32': [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _F, _P],
    'dtn_gqa_fwd': [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _I64, _I64, _P],
    'dtn_gqa_set_variant': [_I],
}

_lock = threading.Lock()
_library = None


def exported_symbols() -> tuple[str, ...]:
    """Names this binding expects the shared library to export."""
    return tuple(_SIGNATURES)


def lib() -> ct.CDLL:
    """The loaded shared library. Raises RuntimeError when it has not been built."""
    global _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.exists():
                raise RuntimeError(
                    f'{LIBRARY_PATH} is missing: build it with `python -m deuteron_b200.csrc.build` '
                    '(there is no fallback path)')
            library = ct.CDLL(str(LIBRARY_PATH))
            for name, argtypes in _SIGNATURES.items():
                function = getattr(library, name)
                function.argtypes = argtypes
                function.restype = ct.c_int
            _library = library
        return _library


def last_error() -> str:
    buffer = ct.create_string_buffer(512)
    lib().dtn_last_error(buffer, len(buffer))
    return buffer.value.decode(errors='replace')


def check(status: int) -> None:
    """Turns a non-zero status into the exception the reference's surface would raise."""
    if status == OK:
        return
    message = last_error() or f'deuteron_b200 status {status}'
    if status in (ERR_INVALID, ERR_WORKSPACE):
        raise ValueError(message)
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(message)
    if status == ERR_DEVICE:
        raise DeviceWaitError(message)
    raise CudaError(message)


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args))


def elementwise_program(params: dict, input_pointers: list[int], out_pointer: int, stream: int) -> None:
    """Launches dtn_elementwise_program for a classifier-built register program (classify._program_plan)."""
    count = len(params['ops'])
    as_bytes = lambda values: (ct.c_ubyte * max(len(values), 1))(*values)
    inputs = (ct.c_void_p * len(input_pointers))(*input_pointers)
    call('dtn_elementwise_program', as_bytes(params['ops']), as_bytes(params['dst']), as_bytes(params['a']),
         as_bytes(params['b']), count, inputs, as_bytes([int(i['f16']) for i in params['inputs']]),
         as_bytes([int(i['scalar']) for i in params['inputs']]), len(input_pointers), params['out_reg'], out_pointer,
         int(params['out_f16']), params['n'], stream)


def row_fused(params: dict, x_pointer: int, input_pointers: list[int | None], out_pointer: int, ldx: int, ldo: int, stream: int) -> None:
    """Launches dtn_row_fused for a classifier-built row program (classify_rows._row_program).
    input_pointers holds one device pointer per extra input, None for immediates."""
    count = len(params['ops'])
    as_bytes = lambda values: (ct.c_ubyte * max(len(values), 1))(*values)
    described = params['inputs']
    inputs = (ct.c_void_p * max(len(described), 1))(*[p or 0 for p in input_pointers])
    immediates = (ct.c_float * max(len(described), 1))(*[float(i.get('value', 0.0)) for i in described])
    call('dtn_row_fused', REDUCE_OPS[params['reduce']], x_pointer, params['rows'], params['cols'], ldx, inputs,
         as_bytes([ROW_INPUT_KINDS[i['kind']] for i in described]), immediates, len(described), as_bytes(params['ops']),
         as_bytes(params['dst']), as_bytes(params['a']), as_bytes(params['b']), params['n_scalar'], count, params['out_reg'],
         out_pointer, ldo, stream)


def device_status(stream: int = 0) -> int:
    """Synchronises `stream` and returns (and clears) the device status word; 0 means clean."""
    value = ct.c_int(0)
    call('dtn_device_status', ct.byref(value), stream)
    return value.value


def raise_on_device_status(stream: int = 0) -> None:
    status = device_status(stream)
    if status:
        role = {0x71: 'bounded-wait self-test', 0x11: 'attention K loader', 0x12: 'attention V loader', 0x13: 'attention Q loader', 0x31: 'attention softmax (scores)', 0x32: 'attention output', 0x33: 'attention softmax (row exchange)', 0x21: 'attention MMA issuer (queries)', 0x23: 'attention MMA issuer (values)', 0x24: 'attention MMA issuer (probabilities)', 0x25: 'attention MMA issuer (keys)', 0x26: 'attention MMA issuer (probabilities)', 0x51: 'fused-split GEMM producers', 0x52: 'fused-split GEMM MMA issuer', 0x53: 'fused-split GEMM epilogue', 5: 'TMA producer (split of A)', 1: 'TMA producer', 2: 'MMA issuer (accumulator)', 3: 'MMA issuer (operands)', 4: 'epilogue'}.get(status >> 8, 'kernel')
        raise DeviceWaitError(f'bounded wait ran out in the {role}, CTA {status & 0xff} (status {status:#x})')
