"""LocalRunner: the reference's launch surface (benchmark.py:160-287) over the native kernels.

`run_kernel(launch, compiled, produced=None, *, warmup, iters, samples)` takes a meta.json launch
and the Compilation returned by compile_kernel, builds the host arrays exactly as
benchmark.py:54-73 does (outputs zero-filled, `data` literals, seeded standard_normal), copies them
to the device in `arg_order`, resets `zero_outputs` before every launch, times `iters` launches
captured in a CUDA graph `samples` times and returns the same result dictionary, with the outputs
copied back to host arrays. Host<->device copies and timing go through torch; compute goes through
the C ABI only.
"""
from __future__ import annotations

import os
import statistics
import threading
import time
from pathlib import Path
from typing import Any

import numpy as np

from . import jit, native
from .build import Compilation
from .validation import validate_launch

DTYPES: dict[str, Any] = {'f32': np.float32, 'f16': np.float16, 'f64': np.float64, 'i32': np.int32, 'i64': np.int64}


def argument_array(arg: Any, produced: Any = None) -> np.ndarray:
    """Host array of one meta.json argument (benchmark.py:54-73)."""
    dtype = DTYPES[arg['dtype']]
    shape = tuple(arg['shape'])
    if arg.get('intermediate'):
        if produced is None or arg['name'] not in produced:
            raise ValueError(f"missing intermediate buffer {arg['name']}")
        array = np.asarray(produced[arg['name']])
        if array.shape != shape or array.dtype != np.dtype(dtype):
            raise ValueError(f"intermediate buffer {arg['name']} must have shape {shape} and dtype {np.dtype(dtype)}")
    elif arg.get('output'):
        array = np.zeros(shape, dtype=dtype)
    elif 'data' in arg:
        array = np.asarray(arg['data'], dtype=dtype)
    elif 'seed' in arg:
        if type(arg['seed']) is not int or arg['seed'] < 0:
            raise ValueError(f"buffer {arg['name']} requires a nonnegative integer seed")
        array = np.random.default_rng(arg['seed']).standard_normal(shape).astype(dtype)
    else:
        raise ValueError(f"buffer {arg['name']} has no seed, data, output, or intermediate")
    return np.ascontiguousarray(np.asarray(array, dtype=dtype).reshape(shape)).reshape(shape)


def validate_timing(warmup: Any, iters: Any, samples: Any) -> None:
    if any(type(value) is not int for value in (warmup, iters, samples)) or warmup < 0 or iters < 1 or samples < 1:
        raise ValueError('warmup must be a nonnegative integer and iters/samples must be positive integers')


def compare_outputs(problem: Any, metadata: Any, produced: Any) -> dict[str, float]:
    """Checks produced outputs against `problem`/expected.npz with meta's rtol/atol (benchmark.py:100-124)."""
    errors = {}
    declared_shapes = {arg['name']: tuple(arg['shape']) for launch in metadata.get('kernels', [])
                       for arg in launch['args'] if arg.get('output') and not arg.get('scalar')}
    with np.load(Path(problem) / 'expected.npz') as expected:
        for name in expected.files:
            if name not in produced:
                raise AssertionError(f'kernel did not produce expected buffer {name}')
            actual = np.asarray(produced[name])
            reference = expected[name]
            declared = declared_shapes.get(name)
            if declared is not None and actual.shape != declared:
                raise AssertionError(f'{Path(problem).name}/{name}: output shape {actual.shape} does not match declared {declared}')
            if reference.shape == () and actual.shape == declared == (1,):
                actual = actual.reshape(())
            if actual.shape != reference.shape:
                raise AssertionError(f'{Path(problem).name}/{name}: output shape {actual.shape} does not match {reference.shape}')
            errors[name] = float(np.max(np.abs(actual.astype(np.float64) - reference))) if actual.size else 0.0
            np.testing.assert_allclose(actual, reference, rtol=metadata['rtol'], atol=metadata['atol'], equal_nan=False,
                                       err_msg=f'{Path(problem).name}/{name}')
    return errors


def _overwrites(plan: Any, name: str) -> bool:
    """True when the native kernel of `plan` writes every element of buffer `name` without reading it first."""
    return plan.kind == 'gemm' and plan.buffers['out'] == (name, 0)


class LocalRunner:
    """One CUDA device, one stream; must be used and closed by the thread that created it."""

    def __init__(self, device: Any = 0) -> None:
        if type(device) is not int or device < 0:
            raise ValueError('device must be a nonnegative integer')
        import torch
        if not torch.cuda.is_available():
            raise native.CudaError('no CUDA device is available')
        if device >= torch.cuda.device_count():
            raise ValueError(f'CUDA device {device} does not exist')
        native.lib()  # fail now, loudly, if the kernels are not built
        self._torch = torch
        self.device = device
        self.torch_device = torch.device('cuda', device)
        self.pid, self.thread = os.getpid(), threading.get_ident()
        self.stream = torch.cuda.Stream(device=self.torch_device)
        self._copy_in = torch.cuda.Stream(device=self.torch_device)
        self._copy_out = torch.cuda.Stream(device=self.torch_device)
        properties = torch.cuda.get_device_properties(device)
        self.device_info = {'name': properties.name, 'arch': f'sm_{properties.major}{properties.minor}',
                            'multiprocessors': properties.multi_processor_count}
        self.open = True
        self._resident: dict[int, Any] = {}
        self._pinned: list[Any] = []
        self._jit: dict[int, tuple[Any, Any]] = {}

    def __enter__(self) -> 'LocalRunner':
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    def close(self) -> None:
        if not self.open:
            return
        self._assert_owner()
        self.stream.synchronize()
        self._resident.clear()
        self._pinned.clear()
        self.open = False

    def _assert_owner(self) -> None:
        if self.pid != os.getpid() or self.thread != threading.get_ident() or not self.open:
            raise RuntimeError('LocalRunner must be open and used in its creating process and thread')

    # -- launching ---------------------------------------------------------------------------

    def _specialized(self, plan: Any) -> tuple[dict, Any] | None:
        """The kernel compiled for this one program (jit.py), for small FP32 elementwise and row programs; None for
        everything else, with `DTN_JIT=0`, or when NVRTC or the module load fails: the library's kernel runs then."""
        if not jit.enabled():
            return None
        entry = self._jit.get(id(plan))
        if entry is None or entry[0] is not plan:
            spec = jit.specialized_source(plan)
            kernel = jit.kernel_for(spec, self.device) if spec is not None else None
            entry = (plan, (spec, kernel) if kernel is not None else None)
            self._jit[id(plan)] = entry
        return entry[1]

    def _enqueue(self, plan: Any, pointers: dict[str, int], stream: int, workspace: Any) -> None:
        kind, p = plan.kind, plan.params

        def ptr(role: str, element_bytes: int) -> int:
            name, offset = plan.buffers[role]
            return pointers[name] + offset * element_bytes

        if kind in jit.KINDS:
            special = self._specialized(plan)
            if special is not None:
                def width(role: str) -> int:   # bytes per element of the buffer behind a role
                    if kind != 'elementwise_program':
                        return 4
                    return 2 if (p['out_f16'] if role == 'out' else p['inputs'][int(role[2:])]['f16']) else 4
                jit.launch(special[0], special[1], lambda role: ptr(role, width(role)), stream)
                return
        if kind == 'elementwise':
            binary = 'y' in plan.buffers
            native.call('dtn_elementwise_f32', native.ELEMENTWISE_OPS[p['op']], ptr('x', 4), ptr('y', 4) if binary else None,
                        ptr('out', 4), p['n'], stream)
        elif kind == 'elementwise_program':
            sizes = [2 if spec['f16'] else 4 for spec in p['inputs']]
            native.elementwise_program(p, [ptr(f'in{i}', size) for i, size in enumerate(sizes)],
                                       ptr('out', 2 if p['out_f16'] else 4), stream)
        elif kind == 'f16_copy':
            native.call('dtn_f16_copy', ptr('x', 2), ptr('out', 2), p['n'], stream)
        elif kind == 'f16_widen':
            native.call('dtn_f16_widen', ptr('x', 2), ptr('out', 4), p['n'], stream)
        elif kind == 'f16_narrow':
            native.call('dtn_f16_narrow', ptr('x', 4), ptr('out', 2), p['n'], stream)
        elif kind == 'row_reduce':
            native.call('dtn_row_reduce_f32', native.REDUCE_OPS[p['op']], ptr('x', 4), ptr('out', 4), p['rows'], p['cols'],
                        max(p['cols'], 1), stream)
        elif kind == 'row_fused':
            extra = [None if item['kind'] == 'immediate' else ptr(f'in{i}', 4) for i, item in enumerate(p['inputs'])]
            native.row_fused(p, ptr('x', 4), extra, ptr('out', 4), max(p['cols'], 1), 0 if p['per_row'] else max(p['cols'], 1), stream)
        elif kind == 'gemm':
            ws_ptr, ws_bytes = workspace
            native.call('dtn_gemm_x3', native.GEMM_MODES[p['mode']], ptr('left', 4), ptr('right', 4), ptr('out', 4), p['m'],
                        p['n'], p['k'], max(p['k'], 1), max(p['n'], 1), max(p['n'], 1), ws_ptr, ws_bytes, stream)
        elif kind == 'attention':
            native.call('dtn_attention_f32', ptr('q', 4), ptr('kt', 4), ptr('v', 4), ptr('out', 4), p['rows'], p['keys'],
                        p['depth'], p['cols'], float(np.float32(p['scale'])), stream)
        elif kind == 'gqa':
            size = 2 if p['storage'] == 'f16' else 4
            native.call('dtn_gqa_fwd', ptr('q', size), ptr('k', size), ptr('v', size), ptr('out', 4), p['batch'], p['hq'],
                        p['hkv'], p['s'], p['d'], float(np.float32(p['scale'])), native.STORAGE[p['storage']], 0,
                        p['batch'] * p['hkv'], stream)
        else:
            raise NotImplementedError(f'no launcher for plan kind {kind}')

    def pinned(self, shape: Any, dtype: Any) -> np.ndarray:
        """A page-locked host array (so that copies to and from the device run at full PCIe rate)."""
        torch = self._torch
        count = int(np.prod(shape)) if len(tuple(shape)) else 1
        holder = torch.empty(max(count * np.dtype(dtype).itemsize, 1), dtype=torch.uint8, pin_memory=True)
        array = holder.numpy()[:count * np.dtype(dtype).itemsize].view(dtype).reshape(shape)
        self._pinned.append(holder)
        return array

    def execute(self, compiled: Any, arrays: dict[str, np.ndarray], outputs: dict[str, np.ndarray] | None = None,
                *, synchronize: bool = True) -> dict[str, np.ndarray]:
        """One launch of a compiled kernel on caller-supplied HOST arrays.

        Copies every non-output buffer of the launch to the device, resets `zero_outputs`, launches
        the native kernel and copies the output buffers back into `outputs` (allocated if omitted).
        This is the launch half of benchmark.py:205-287 without the timing loop, for callers that
        bring their own data. Device buffers are kept between calls with the same compiled kernel.
        """
        self._assert_owner()
        if not isinstance(compiled, Compilation) or compiled.plan is None:
            raise ValueError('execute takes the Compilation returned by compile_kernel')
        torch = self._torch
        launch, plan = compiled.launch, compiled.plan
        by_name = {arg['name']: arg for arg in launch['args']}
        state = self._resident.get(id(compiled))
        with torch.cuda.device(self.torch_device), torch.cuda.stream(self.stream):
            stream = self.stream.cuda_stream
            if state is None:
                tensors, pointers = {}, {}
                for name in launch['arg_order']:
                    arg = by_name[name]
                    nbytes = int(np.prod(arg['shape'])) * np.dtype(DTYPES[arg['dtype']]).itemsize if arg['shape'] else np.dtype(DTYPES[arg['dtype']]).itemsize
                    tensors[name] = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=self.torch_device)
                    pointers[name] = tensors[name].data_ptr()
                workspace = (None, 0)
                if plan.kind == 'gemm':
                    import ctypes as ct
                    size = ct.c_size_t(0)
                    native.call('dtn_gemm_workspace_bytes', native.GEMM_MODES[plan.params['mode']], plan.params['m'],
                                plan.params['n'], plan.params['k'], ct.byref(size))
                    if size.value:
                        scratch = torch.empty(size.value + 1024, dtype=torch.uint8, device=self.torch_device)
                        ws_ptr = (scratch.data_ptr() + 1023) // 1024 * 1024
                        workspace = (ws_ptr, scratch.numel() - (ws_ptr - scratch.data_ptr()))
                        tensors['__workspace__'] = scratch
                state = (compiled, tensors, pointers, workspace)
                self._resident[id(compiled)] = state
            _, tensors, pointers, workspace = state
            for name, arg in by_name.items():
                if arg.get('output'):
                    continue
                host = arrays[name]
                if host.dtype != np.dtype(DTYPES[arg['dtype']]) or list(host.shape) != list(arg['shape']):
                    raise ValueError(f'buffer {name} must have shape {arg["shape"]} and dtype {arg["dtype"]}')
            blocks = self._gemm_row_blocks(plan) if plan.kind == 'gemm' and not launch.get('zero_outputs') else 1
            if blocks > 1:
                out_name = plan.buffers['out'][0]
                out_arg = by_name[out_name]
                host_out = outputs[out_name] if outputs is not None and out_name in outputs else np.empty(out_arg['shape'], dtype=np.float32)
                self._execute_gemm_blocks(plan, tensors, pointers, workspace, arrays, host_out, blocks)
                if synchronize:
                    self.stream.synchronize()
                return {out_name: host_out}
            for name, arg in by_name.items():
                if arg.get('output'):
                    continue
                host = np.ascontiguousarray(arrays[name])
                if host.nbytes:
                    tensors[name][:host.nbytes].copy_(torch.from_numpy(host.reshape(-1).view(np.uint8)), non_blocking=True)
            for name in launch.get('zero_outputs', []):
                tensors[name].zero_()
            self._enqueue(plan, pointers, stream, workspace)
            results = {}
            for name, arg in by_name.items():
                if not arg.get('output'):
                    continue
                host = outputs[name] if outputs is not None and name in outputs else np.empty(arg['shape'], dtype=DTYPES[arg['dtype']])
                if host.nbytes:
                    torch.from_numpy(host.reshape(-1).view(np.uint8)).copy_(tensors[name][:host.nbytes], non_blocking=True)
                results[name] = host
            if synchronize:
                self.stream.synchronize()
        return results

    def _gemm_row_blocks(self, plan: Any) -> int:
        """Number of row blocks a large compensated GEMM is walked in when its operands come from the host, so
        that copies and products overlap; 1 = no blocking."""
        return len(self._gemm_row_plan(plan))

    @staticmethod
    def _gemm_row_plan(plan: Any) -> list[int]:
        """Rows of every block of A, in order: eighths (quarters, halves) of the rows, except that the last of them is
        cut into a half and two quarters: the host link is the bottleneck, every product hides behind the copy of the
        next block, and what stays exposed at the end is the last block's product and its way back to the host, so
        that block should be small (8192^3: 11.82 -> 11.55 ms). One block = no blocking."""
        m, k = plan.params['m'], plan.params['k']
        if plan.params['mode'] in ('f32', 'f32_splitk') or m * k * 4 < (32 << 20):
            return [m]
        for blocks in (8, 4, 2):
            if m % blocks == 0 and (m // blocks) % 256 == 0 and (m // blocks) >= 512:
                rows = m // blocks
                tail = [rows // 2, rows // 4, rows // 4] if rows % 1024 == 0 else [rows]
                return [rows] * (blocks - 1) + tail
        return [m]

    @staticmethod
    def _gemm_column_plan(n: int) -> list[int]:
        """Column blocks of B and C for the host-fed pipeline. One block: B goes to the device whole, before A.
        Feeding B by column blocks (first block, then A by row blocks, then the other blocks against all of A) lets
        the result start its way back after an eighth of the bytes instead of half of them, but measured slower on
        this host (8192^3: 12.2-13.6 ms against 11.6 ms for quarters, halves and graded blocks alike): the link is
        bound by the 512 MB going in, and every byte coming back at the same time slows those down.
        DTN_E2E_COLUMNS=w1,w2,... (widths summing to n) selects a cut for measurements."""
        import os
        forced = os.environ.get('DTN_E2E_COLUMNS')
        if forced:
            widths = [int(x) for x in forced.split(',')]
            if sum(widths) == n and all(w > 0 for w in widths):
                return widths
        return [n]

    def _execute_gemm_blocks(self, plan: Any, tensors: dict, pointers: dict, workspace: Any, arrays: dict, host_out: np.ndarray,
                             blocks: int) -> None:
        """Host-fed compensated GEMM as a three-stream pipeline over row blocks of A and column blocks of B and C.

        The host link is the bottleneck (for an 8192^3 product 805 MB cross it against 2 ms of arithmetic), so the
        order of the copies is what matters: nothing can be multiplied before a column block of B is on the device and
        nothing can return before something is multiplied. The first column block of B goes first, then A row block
        by row block, each multiplied against that column block as it lands (its part of C returns at once); then the
        remaining column blocks of B, each multiplied against all of A, which is resident by then. The copy-in stream
        is never idle, the result's way back overlaps it from the first quarter of B on, and the last blocks are small.
        Per-element arithmetic (and so every bit of the result) is the same as in the one-launch path: a block of C
        is the product of A's rows and B's columns over the whole of k.
        """
        torch = self._torch
        m, n, k = plan.params['m'], plan.params['n'], plan.params['k']
        mode = native.GEMM_MODES[plan.params['mode']]
        row_plan = self._gemm_row_plan(plan)
        row_starts = [sum(row_plan[:i]) for i in range(len(row_plan))]
        column_plan = self._gemm_column_plan(n)
        column_starts = [sum(column_plan[:j]) for j in range(len(column_plan))]
        left_name, right_name, out_name = plan.buffers['left'][0], plan.buffers['right'][0], plan.buffers['out'][0]
        compute, copy_in, copy_out = self.stream, self._copy_in, self._copy_out
        copy_in.wait_stream(compute)       # earlier launches may still read the operand buffers
        left = np.ascontiguousarray(arrays[left_name])
        right = np.ascontiguousarray(arrays[right_name])
        left_host, right_host, out_host = left.ctypes.data, right.ctypes.data, host_out.ctypes.data
        keep = (left, right)               # the host arrays stay alive until the copies have been issued and waited for
        row_in, row_b, row_out = k * 4, n * 4, n * 4
        ws_ptr, ws_bytes = workspace

        def b_columns_in(first: int, width: int):
            native.call('dtn_copy_block', pointers[right_name] + first * 4, row_b, right_host + first * 4, row_b, width * 4, k, 1,
                        copy_in.cuda_stream)
            event = torch.cuda.Event()
            event.record(copy_in)
            return event

        def c_block_out(first_row: int, rows: int, first_col: int, width: int) -> None:
            done = torch.cuda.Event()
            done.record(compute)
            copy_out.wait_event(done)
            offset = first_row * row_out + first_col * 4
            native.call('dtn_copy_block', out_host + offset, row_out, pointers[out_name] + offset, row_out, width * 4, rows, 0,
                        copy_out.cuda_stream)

        def product(first_row: int, rows: int, first_col: int, width: int, phase: int) -> None:
            native.call('dtn_gemm_x3_phase', mode, pointers[left_name] + first_row * row_in, pointers[right_name] + first_col * 4,
                        pointers[out_name] + first_row * row_out + first_col * 4, rows, width, k, k, n, n, ws_ptr, ws_bytes, phase,
                        compute.cuda_stream)

        # first column block of B, then A by row blocks
        first_ready = b_columns_in(0, column_plan[0])
        a_ready = []
        for first, rows in zip(row_starts, row_plan):
            native.call('dtn_copy_block', pointers[left_name] + first * row_in, row_in, left_host + first * row_in, row_in, row_in, rows, 1,
                        copy_in.cuda_stream)
            event = torch.cuda.Event()
            event.record(copy_in)
            a_ready.append(event)
        later_ready = [b_columns_in(first, width) for first, width in zip(column_starts[1:], column_plan[1:])]
        compute.wait_event(first_ready)
        # B's first block is split once, on its own (1|4: split, keep A), before any row block: every row block then
        # runs 3|8 (split A, keep B, multiply), which always takes the plane-reading kernels. A plain phase 3 on the
        # first block could pick a single-kernel form that writes no planes, and the later blocks would multiply by
        # whatever the workspace held.
        product(0, row_plan[0], 0, column_plan[0], 1 | 4)
        for i, (first, rows) in enumerate(zip(row_starts, row_plan)):
            compute.wait_event(a_ready[i])
            product(first, rows, 0, column_plan[0], 3 | 8)
            c_block_out(first, rows, 0, column_plan[0])
        # the other column blocks against all of A
        for ready, first, width in zip(later_ready, column_starts[1:], column_plan[1:]):
            compute.wait_event(ready)
            product(0, m, first, width, 3)
            c_block_out(0, m, first, width)
        compute.wait_stream(copy_out)      # a synchronize of the runner's stream now covers the whole call
        compute.wait_stream(copy_in)
        self._held_host_arrays = keep      # released by the next call; the copies above may still be reading them

    def run_kernel(self, launch: Any, compiled: Any, produced: Any = None, *, warmup: Any = 10, iters: Any = 100,
                   samples: Any = 7) -> dict[str, Any]:
        """Runs one compiled kernel on seeded inputs and times it (benchmark.py:205-287)."""
        self._assert_owner()
        validate_timing(warmup, iters, samples)
        if not isinstance(compiled, Compilation) or compiled.plan is None:
            raise ValueError('run_kernel takes the Compilation returned by compile_kernel')
        by_name = validate_launch(launch)
        if launch['entry'] != compiled.launch['entry'] or list(launch['arg_order']) != list(compiled.launch['arg_order']):
            raise ValueError('launch does not match the compiled kernel')
        for name, arg in by_name.items():
            compiled_arg = next(a for a in compiled.launch['args'] if a['name'] == name)
            if list(arg['shape']) != list(compiled_arg['shape']) or arg['dtype'] != compiled_arg['dtype']:
                raise ValueError(f'buffer {name} differs from the compiled kernel')
        torch = self._torch
        plan = compiled.plan
        arrays = {name: argument_array(arg, produced) for name, arg in by_name.items() if not arg.get('scalar')}
        started = time.perf_counter()
        with torch.cuda.device(self.torch_device), torch.cuda.stream(self.stream):
            stream = self.stream.cuda_stream
            device_buffers, pointers = {}, {}
            for name in launch['arg_order']:
                host = arrays[name]
                tensor = torch.empty(max(host.nbytes, 1) + 16, dtype=torch.uint8, device=self.torch_device)
                base = tensor.data_ptr()
                aligned = (base + 15) // 16 * 16
                view = tensor[aligned - base: aligned - base + host.nbytes]
                if host.nbytes:
                    view.copy_(torch.from_numpy(host.reshape(-1).view(np.uint8)), non_blocking=False)
                device_buffers[name], pointers[name] = (tensor, view), aligned
            workspace = (None, 0)
            if plan.kind == 'gemm':
                import ctypes as ct
                size = ct.c_size_t(0)
                native.call('dtn_gemm_workspace_bytes', native.GEMM_MODES[plan.params['mode']], plan.params['m'],
                            plan.params['n'], plan.params['k'], ct.byref(size))
                if size.value:
                    scratch = torch.empty(size.value + 1024, dtype=torch.uint8, device=self.torch_device)
                    ws_ptr = (scratch.data_ptr() + 1023) // 1024 * 1024
                    workspace = (ws_ptr, scratch.numel() - (ws_ptr - scratch.data_ptr()))
                    device_buffers['__workspace__'] = (scratch, scratch)
            # zero_outputs exist for kernels that accumulate into their output with atomics (benchmark.py:240-243). The
            # timed launches reset them exactly as the reference's runner does, so that the figures compare like with
            # like; where the native kernel overwrites the whole buffer anyway the launch is timed a second time
            # without the resets and reported as `kernel_only_us`.
            resets = [device_buffers[name][1] for name in launch.get('zero_outputs', [])]
            redundant = bool(resets) and all(_overwrites(plan, name) for name in launch.get('zero_outputs', []))

            def enqueue(with_resets: bool = True) -> None:
                if with_resets:
                    for view in resets:   # a memset, as in the reference's runner (benchmark.py:240-243: cuMemsetD8Async)
                        if view.numel():
                            jit.memset_zero(view.data_ptr(), view.numel(), stream)
                self._enqueue(plan, pointers, stream, workspace)

            prepare_seconds = time.perf_counter() - started
            # One launch outside any capture performs the library's per-device set-up.
            enqueue()
            for _ in range(max(warmup - 1, 0)):
                enqueue()
            self.stream.synchronize()

            def timed_graph(with_resets: bool) -> list[float]:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=self.stream):
                    for _ in range(iters):
                        enqueue(with_resets)
                graph.replay()
                self.stream.synchronize()
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                measured = []
                for _ in range(samples):
                    begin.record(self.stream)
                    graph.replay()
                    end.record(self.stream)
                    end.synchronize()
                    measured.append(begin.elapsed_time(end) * 1000 / iters)
                return measured

            # registers and shared memory of the native kernels one launch runs (the reference reports those of its
            # one PTX entry): the launch is recorded in a capture, not run, and its kernel nodes are looked up
            import ctypes as ct
            counts = [ct.c_int(0) for _ in range(4)]
            special = self._specialized(plan) if plan.kind in jit.KINDS else None
            if special is not None:   # a kernel loaded through the driver API: its attributes come from there
                kernels, dynamic_smem = 1, 0
                registers, static_smem = special[1].attributes()
            else:
                native.call('dtn_capture_begin', stream)
                try:
                    self._enqueue(plan, pointers, stream, workspace)
                finally:
                    native.call('dtn_capture_end', stream, *[ct.byref(c) for c in counts])
                kernels, registers, static_smem, dynamic_smem = (c.value for c in counts)

            timings = timed_graph(True)
            kernel_only = statistics.median(timed_graph(False)) if redundant else None
            native.raise_on_device_status(stream)
            outputs = {}
            for name, arg in by_name.items():
                if arg.get('output'):
                    host = np.empty_like(arrays[name])
                    if host.nbytes:
                        host.reshape(-1).view(np.uint8)[:] = device_buffers[name][1].cpu().numpy()
                    outputs[name] = host
        return {'entry': launch['entry'], 'median_us': statistics.median(timings), 'min_us': min(timings),
                'samples_us': timings, 'iters': iters, 'samples': samples, 'warmup': warmup,
                'timing_method': 'cuda_graph_batch_events', 'timing_includes_output_resets': bool(resets),
                'kernel_only_us': kernel_only,
                'registers': registers, 'static_smem_bytes': static_smem, 'dynamic_smem_bytes': launch.get('smem_bytes', 0),
                'native_kernels': kernels, 'native_dynamic_smem_bytes': dynamic_smem,
                'jit_seconds': prepare_seconds, 'native_kernel': plan.describe(), 'outputs': outputs}
