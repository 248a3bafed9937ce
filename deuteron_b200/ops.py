"""Device-resident operators: thin wrappers that hand torch CUDA tensors' pointers to the C ABI.

torch is used for device memory and streams only; every computation below runs in
libdeuteron_b200.so on the current torch stream. Tensors must live on the current CUDA device.
"""
from __future__ import annotations

import ctypes as ct

import torch

from . import native


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            raise ValueError('deuteron_b200 operators take CUDA tensors')


def _flat(tensor: torch.Tensor, dtype: torch.dtype, label: str) -> torch.Tensor:
    if tensor.dtype != dtype:
        raise ValueError(f'{label} must have dtype {dtype}, got {tensor.dtype}')
    if not tensor.is_contiguous():
        raise ValueError(f'{label} must be contiguous')
    return tensor


# ------------------------------------------------------------------------------------------------
# elementwise / f16
# ------------------------------------------------------------------------------------------------


def elementwise(op: str, x: torch.Tensor, y: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = op(x, y) or op(x) elementwise in FP32 (operator names of the reference's ElementwiseImpl)."""
    if op not in native.ELEMENTWISE_OPS:
        raise NotImplementedError(f'elementwise operation {op}')
    binary = op in native.BINARY_OPS
    _require_cuda(x)
    _flat(x, torch.float32, 'x')
    if binary:
        if y is None:
            raise ValueError(f'{op} needs two operands')
        _require_cuda(y)
        _flat(y, torch.float32, 'y')
        if y.shape != x.shape:
            raise ValueError('operand shapes differ')
    if out is None:
        out = torch.empty_like(x)
    _require_cuda(out)
    _flat(out, torch.float32, 'out')
    if out.shape != x.shape:
        raise ValueError('output shape differs')
    native.call('dtn_elementwise_f32', native.ELEMENTWISE_OPS[op], x.data_ptr(), y.data_ptr() if binary else None,
                out.data_ptr(), x.numel(), _stream())
    return out


def add(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    return elementwise('add', x, y, out)


def f16_copy(src: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(src)
    _flat(src, torch.float16, 'src')
    out = torch.empty_like(src) if out is None else _flat(out, torch.float16, 'out')
    native.call('dtn_f16_copy', src.data_ptr(), out.data_ptr(), src.numel(), _stream())
    return out


def f16_widen(src: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(src)
    _flat(src, torch.float16, 'src')
    out = torch.empty(src.shape, dtype=torch.float32, device=src.device) if out is None else _flat(out, torch.float32, 'out')
    native.call('dtn_f16_widen', src.data_ptr(), out.data_ptr(), src.numel(), _stream())
    return out


def f16_narrow(src: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(src)
    _flat(src, torch.float32, 'src')
    out = torch.empty(src.shape, dtype=torch.float16, device=src.device) if out is None else _flat(out, torch.float16, 'out')
    native.call('dtn_f16_narrow', src.data_ptr(), out.data_ptr(), src.numel(), _stream())
    return out


# ------------------------------------------------------------------------------------------------
# row reductions
# ------------------------------------------------------------------------------------------------


def row_reduce(op: str, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = sum / max / sumsq of row r of the 2-D FP32 tensor x (rows may be strided)."""
    if op not in ('sum', 'max', 'sumsq'):
        raise NotImplementedError(f'row reduction {op}')
    _require_cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or (x.shape[1] > 1 and x.stride(1) != 1):
        raise ValueError('row_reduce takes a 2-D float32 tensor with unit column stride')
    rows, cols = x.shape
    ldx = x.stride(0) if rows > 1 else max(cols, 1)
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=x.device)
    _flat(out, torch.float32, 'out')
    native.call('dtn_row_reduce_f32', native.REDUCE_OPS[op], x.data_ptr(), out.data_ptr(), rows, cols, max(ldx, cols), _stream())
    return out


def _row_matrix(x: torch.Tensor, label: str) -> tuple[int, int, int]:
    _require_cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or (x.shape[1] > 1 and x.stride(1) != 1):
        raise ValueError(f'{label} takes a 2-D float32 tensor with unit column stride')
    rows, cols = x.shape
    return rows, cols, max(x.stride(0) if rows > 1 else cols, cols, 1)


def _row_fused(reduce: str, x: torch.Tensor, program: list[tuple[str, int, int, int]], n_scalar: int, out_reg: int, inputs=(),
               per_row: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """One launch of the fused row kernel. program: (operator, destination, a, b) over the registers
    0 = reduced value, 1 = sum of exponentials, 2 = row element, 3 + i = inputs[i]; inputs: a float
    (immediate), a one-element tensor (scalar) or a tensor of `cols` values (one per column)."""
    rows, cols, ldx = _row_matrix(x, 'row kernel')
    described, pointers = [], []
    for item in inputs:
        if isinstance(item, (int, float)):
            described.append({'kind': 'immediate', 'value': float(item)})
            pointers.append(None)
            continue
        _flat(item, torch.float32, 'row kernel input')
        if item.numel() not in (1, cols):
            raise ValueError('row kernel inputs hold one value or one value per column')
        described.append({'kind': 'columns' if item.numel() == cols and cols != 1 else 'scalar'})
        pointers.append(item.data_ptr())
    if out is None:
        out = torch.empty(rows if per_row else (rows, cols), dtype=torch.float32, device=x.device)
    _flat(out, torch.float32, 'out')
    params = {'reduce': reduce, 'rows': rows, 'cols': cols, 'inputs': described, 'n_scalar': n_scalar, 'out_reg': out_reg,
              'ops': [native.ELEMENTWISE_OPS[p[0]] for p in program], 'dst': [p[1] for p in program],
              'a': [p[2] for p in program], 'b': [p[3] for p in program], 'per_row': per_row}
    if not _row_specialized(params, x, pointers, out, ldx):
        native.row_fused(params, x.data_ptr(), pointers, out.data_ptr(), ldx, 0 if per_row else max(cols, 1), _stream())
    return out


_row_kernels: dict[tuple, tuple | None] = {}


def _row_specialized(params: dict, x: torch.Tensor, pointers: list, out: torch.Tensor, ldx: int) -> bool:
    """Runs the kernel written for this one program (jit.py) when there is one: dense rows, 16-byte aligned buffers.
    With no program to decode and a row's loads all requested up front it is the faster kernel at every size it
    takes; False sends the launch to the library's kernel."""
    from . import jit
    addresses = [x.data_ptr(), out.data_ptr(), *[p for p in pointers if p is not None]]
    if not jit.enabled() or ldx != params['cols'] or params['rows'] == 0 or any(a % 16 for a in addresses):
        return False
    device = x.device.index if x.device.index is not None else torch.cuda.current_device()
    key = (device, repr(sorted(params.items())))
    if key not in _row_kernels:
        if torch.cuda.is_current_stream_capturing():   # a module is not loaded inside a capture: the library kernel this once
            return False
        buffers = {'x': ('x', 0), 'out': ('out', 0), **{f'in{i}': (f'in{i}', 0) for i in range(len(pointers))}}
        spec = jit.row_source(params, buffers)
        kernel = jit.kernel_for(spec, device) if spec is not None else None
        _row_kernels[key] = (spec, kernel) if kernel is not None else None
    entry = _row_kernels[key]
    if entry is None:
        return False
    roles = {'x': x.data_ptr(), 'out': out.data_ptr(), **{f'in{i}': p for i, p in enumerate(pointers)}}
    jit.launch(entry[0], entry[1], roles.__getitem__, _stream())
    return True


def row_softmax(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, c] = exp(x[r, c] - max_r) / sum_c exp(x[r, c] - max_r), one launch."""
    return _row_fused('softmax', x, [('reciprocal', 3, 1, 1), ('subtract', 4, 2, 0), ('exp', 4, 4, 4), ('multiply', 4, 4, 3)], 1, 4, out=out)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, epsilon: float = 1e-5, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, c] = x[r, c] * rsqrt(mean_c(x[r, :]^2) + epsilon) * weight[c], one launch."""
    program = [('divide', 6, 0, 4), ('add', 6, 6, 5), ('rsqrt', 6, 6, 6), ('multiply', 7, 2, 6), ('multiply', 7, 7, 3)]
    return _row_fused('sumsq', x, program, 3, 7, inputs=(weight, float(x.shape[1]), float(epsilon)), out=out)


def l2_norm(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, c] = x[r, c] * rsqrt(sum_c x[r, :]^2), one launch."""
    return _row_fused('sumsq', x, [('rsqrt', 3, 0, 0), ('multiply', 4, 2, 3)], 1, 4, out=out)


def row_mean(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = sum_c x[r, c] / cols, one launch."""
    return _row_fused('sum', x, [('divide', 4, 0, 3)], 1, 4, inputs=(float(x.shape[1]),), per_row=True, out=out)


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def gemm_workspace_bytes(mode: str, m: int, n: int, k: int) -> int:
    size = ct.c_size_t(0)
    native.call('dtn_gemm_workspace_bytes', native.GEMM_MODES[mode], m, n, k, ct.byref(size))
    return size.value


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Scratch for the operand planes, cached per (device, stream) and grown on demand."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    buffer = _workspaces.get(key)
    if buffer is None or buffer.numel() < nbytes + 1024:
        buffer = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        _workspaces[key] = buffer
    return buffer


def _row_major(tensor: torch.Tensor, label: str) -> int:
    if tensor.dtype != torch.float32 or tensor.dim() != 2:
        raise ValueError(f'{label} must be a 2-D float32 tensor')
    if tensor.shape[1] > 1 and tensor.stride(1) != 1:
        raise ValueError(f'{label} must be row-major (unit column stride)')
    return tensor.stride(0) if tensor.shape[0] > 1 else max(tensor.shape[1], 1)


def gemm(a: torch.Tensor, b: torch.Tensor, mode: str = 'bf16x3', out: torch.Tensor | None = None,
         workspace: torch.Tensor | None = None, phase: int = 3) -> torch.Tensor:
    """C = A @ B with FP32 storage and the reference's contraction_precision `mode`.

    a[M,K], b[K,N], out[M,N]: row-major; rows may be strided (a column block of a wider matrix).
    `phase` 1 runs only the operand split into the workspace, 2 only the product kernel on planes
    already there, 3 (default) both.
    """
    if mode not in native.GEMM_MODES:
        raise ValueError(f'unsupported contraction precision {mode!r}')
    _require_cuda(a, b)
    lda, ldb = _row_major(a, 'a'), _row_major(b, 'b')
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError(f'inner dimensions differ: {k} vs {k2}')
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    _require_cuda(out)
    ldc = _row_major(out, 'out')
    if tuple(out.shape) != (m, n):
        raise ValueError('output shape differs')
    nbytes = gemm_workspace_bytes(mode, m, n, k)
    ws_ptr, ws_bytes = None, 0
    if nbytes:
        if workspace is None:
            workspace = _workspace(nbytes, a.device)
        base = workspace.data_ptr()
        ws_ptr = (base + 1023) // 1024 * 1024
        ws_bytes = workspace.numel() * workspace.element_size() - (ws_ptr - base)
    native.call('dtn_gemm_x3_phase', native.GEMM_MODES[mode], a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k,
                max(lda, k), max(ldb, n), max(ldc, n), ws_ptr, ws_bytes, phase, _stream())
    return out


def push_block(src: torch.Tensor, destinations: list[torch.Tensor]) -> None:
    """Writes the 2-D float32 block `src` into every tensor of `destinations` (same shape, equal row strides; up to
    seven; they may be views of other GPUs' memory) with one kernel that reads the block once."""
    _require_cuda(src)
    lds = _row_major(src, 'src')
    if not destinations:
        return
    rows, cols = src.shape
    strides = set()
    for dst in destinations:
        if dst.dtype != torch.float32 or tuple(dst.shape) != (rows, cols):
            raise ValueError('every destination must be a float32 tensor of the shape of src')
        strides.add(_row_major(dst, 'destination'))
    if len(strides) != 1:
        raise ValueError('the destinations must share one row stride')
    pointers = (ct.c_void_p * len(destinations))(*[dst.data_ptr() for dst in destinations])
    native.call('dtn_push_block', src.data_ptr(), max(lds, cols), pointers, len(destinations), max(strides.pop(), cols), rows, cols,
                _stream())


def set_gemm_variant(variant: int) -> None:
    native.call('dtn_gemm_set_variant', variant)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------


def attention(q: torch.Tensor, kt: torch.Tensor, v: torch.Tensor, scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """Single-head attention in the reference's example layout: q[rows,depth], kt[depth,keys], v[keys,cols]."""
    _require_cuda(q, kt, v)
    for tensor, label in ((q, 'q'), (kt, 'kt'), (v, 'v')):
        _flat(tensor, torch.float32, label)
        if tensor.dim() != 2:
            raise ValueError(f'{label} must be 2-D')
    rows, depth = q.shape
    depth2, keys = kt.shape
    keys2, cols = v.shape
    if depth != depth2 or keys != keys2:
        raise ValueError('attention operand shapes disagree')
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float32, device=q.device)
    _flat(out, torch.float32, 'out')
    native.call('dtn_attention_f32', q.data_ptr(), kt.data_ptr(), v.data_ptr(), out.data_ptr(), rows, keys, depth, cols,
                float(scale), _stream())
    return out


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, out: torch.Tensor | None = None,
                  groups: tuple[int, int] | None = None) -> torch.Tensor:
    """Grouped-query attention forward, non-causal: q[B,Hq,S,D], k/v[B,Hkv,S,D] (f16 or f32) -> out[B,Hq,S,D] f32.

    `groups=(begin, end)` restricts the computation to that range of the B*Hkv (batch, kv-head) groups.
    """
    _require_cuda(q, k, v)
    if q.dtype not in (torch.float16, torch.float32) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError('q, k, v must share dtype float16 or float32')
    for tensor, label in ((q, 'q'), (k, 'k'), (v, 'v')):
        if tensor.dim() != 4 or not tensor.is_contiguous():
            raise ValueError(f'{label} must be a contiguous [B,H,S,D] tensor')
    b, hq, s, d = q.shape
    if k.shape != v.shape or k.shape[0] != b or k.shape[2] != s or k.shape[3] != d:
        raise ValueError('k/v shapes disagree with q')
    hkv = k.shape[1]
    if out is None:
        out = torch.empty((b, hq, s, d), dtype=torch.float32, device=q.device)
    _flat(out, torch.float32, 'out')
    begin, end = groups if groups is not None else (0, b * hkv)
    native.call('dtn_gqa_fwd', q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, hq, hkv, s, d, float(scale),
                native.STORAGE['f16' if q.dtype == torch.float16 else 'f32'], begin, end, _stream())
    return out


def set_gqa_variant(variant: int) -> None:
    native.call('dtn_gqa_set_variant', variant)


def check_device_status() -> None:
    """Synchronises the current stream and raises if a kernel reported a wait that ran out."""
    native.raise_on_device_status(_stream())
