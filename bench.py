"""Benchmark of the hot path: compensated BF16x3 GEMM, M = N = K = 8192, FP32 in/out, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sweep]

A step is one full pass of the hot path over one batch of seeded synthetic input: the operand
split plus the tensor-core product kernel for C = A @ B with A, B uniform[-1, 1) (seeds 7, 11),
through the C ABI. With N GPUs the ONE 8192^3 product is divided by output column blocks: rank r
owns columns [r*8192/N, (r+1)*8192/N) and needs all of A and its columns of B (strong scaling, no
collective in the data path); the value is 2*M*N*K useful flops over the slowest rank's time,
timed on the device with CUDA events.

Printed JSON (one line, rank 0): the driver's contract keys plus
  roofline     the product kernel's achieved TFLOP/s (its own launch time, measured with events
               inside the timed steps) against the measured dense BF16 peak / 3
  cpu_baseline the float64 NumPy product (the reference's own CPU check) timed on a bounded sample
  e2e          the same metric through compile_kernel + LocalRunner.execute with HOST buffers
               (pinned host -> device copies of A and B and the device -> host copy of C inside the
               timed region); at N > 1 through sharding.ShardedHostProduct: every rank feeds its columns
               of B and 1/N of the rows of A from its host, the rows of A are exchanged over NVLink
               (NCCL all-gather), so every operand byte crosses the host link once; `host_link` is the
               measured rate of the same bytes as plain copies, the bound of this figure
  sustained    (N = 1) the same step back to back for about 3 s with the clocks it ran at, against the
               sustained library peak
  extras       the other hot kernels (tf32x3 GEMM, attention, memory-bound kernels) at their
               benchmark sizes, for context

`--sweep` times the mixed sweep instead (GEMMs 1024^3 ... 16384^3 and 16 x 8192 x 8192, attention at 512 ... 16384
keys), each problem split over the ranks, and prints its own line.

`--impl reference` times the reference's CPU implementation of the path (NumPy float64 product of
the same operands, all host cores) on a bounded sample per step and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 8192
FLOPS_PER_GEMM = 2.0 * M * N * K
WORKLOAD = 'gemm_bf16x3_8192x8192x8192_f32io'
# dram__bytes_read.sum + dram__bytes_write.sum of one 8192^3 launch of the product kernel, from the ncu capture
# summarised in profiles/gemm_x3_kernel_bf16_8192_dram.md (2.32 GB read + 0.26 GB written)
PRODUCT_KERNEL_DRAM_BYTES = 3.06e9   # gemm_x3_stream_kernel, 8192^3: 2 537 MB read + 522 MB written (profiles/gemm_x3_stream_kernel_bf16_8192_dram.md)
PRODUCT_KERNEL_ALGORITHMIC_BYTES = 4 * M * K * 2 + 4 * M * N   # four bf16 planes read once + C written once


def bench_config(world: int) -> dict:
    """The `config` of the line, the same for this build's arm and for the reference arm."""
    return {'workload': WORKLOAD, 'm': M, 'n': N, 'k': K, 'inputs': 'uniform[-1,1), seeds 7 and 11',
            'parallelism': f'one {M} x {N} x {K} product, output column blocks x{world}, no collective',
            'l2': 'inputs and operand planes of a rank exceed the 126 MB L2; no flush between steps'}


def measured_peaks() -> dict:
    path = ROOT / 'MEASURED_PEAKS.json'
    if path.exists():
        data = json.loads(path.read_text())
        return {'hbm_gbs': data['hbm_gbs'], 'bf16_tflops': data['bf16_tflops'],
                'bf16_tflops_sustained': data.get('bf16_tflops_sustained', data['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    QUERY = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.process, self.thread = index, [], None, None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(['nvidia-smi', f'--id={self.index}', f'--query-gpu={self.QUERY}',
                                             '--format=csv,noheader,nounits', '-lms', '50'], stdout=subprocess.PIPE,
                                            stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.process.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, begin: float, end: float) -> dict:
        if self.process is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        rows = [line for stamp, line in self.samples if begin - 0.05 <= stamp <= end + 0.15] or [line for _, line in self.samples]
        clocks, maxima, power, reasons = [], [], [], set()
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        for row in rows:
            parts = [p.strip() for p in row.split(',')]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0])); maxima.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(clocks) if clocks else None, 'sm_max_mhz': max(maxima) if maxima else None,
                'power_w_max': max(power) if power else None, 'samples': len(clocks), 'reasons': sorted(reasons)}


def use_all_host_threads() -> int:
    """Lets the BLAS behind NumPy use every host core (torchrun exports OMP_NUM_THREADS=1 to its workers).
    Returns the thread count in effect."""
    cores = os.cpu_count() or 1
    for name in ('OMP_NUM_THREADS', 'OPENBLAS_NUM_THREADS', 'MKL_NUM_THREADS'):
        os.environ[name] = str(cores)
    try:
        import threadpoolctl
        import numpy  # noqa: F401  (the pools exist once NumPy is loaded)
        threadpoolctl.threadpool_limits(limits=cores)
        pools = [pool.get('num_threads', 1) for pool in threadpoolctl.threadpool_info() if pool.get('user_api') == 'blas']
        return max(pools) if pools else cores
    except Exception:
        return cores


def cpu_gemm_sample(seconds_target: float = 12.0) -> dict:
    """The reference's CPU check of this path (float64 NumPy product of the FP32 operands,
    tests/test_tensor_copy.py:52) on a slab of A's rows sized to take roughly `seconds_target`."""
    cores = use_all_host_threads()
    import numpy as np
    from oracle import reference_math as oracle
    right = oracle.seeded_uniform(11, (K, N)).astype(np.float64)
    rows = 64
    probe = oracle.seeded_uniform(7, (rows, K))
    started = time.perf_counter()
    oracle.gemm_f64(probe, right)
    elapsed = time.perf_counter() - started
    rows = int(min(M, max(64, rows * seconds_target / max(elapsed, 1e-3)) // 64 * 64))
    left = oracle.seeded_uniform(7, (rows, K))
    started = time.perf_counter()
    oracle.gemm_f64(left, right)
    elapsed = time.perf_counter() - started
    return {'value': 2.0 * rows * N * K / elapsed / 1e12, 'unit': 'TFLOP/s', 'cores': cores, 'kind': 'port',
            'sample': f'float64 NumPy product of {rows} of the {M} rows of A with the full B ({elapsed:.1f} s)',
            'rows': rows, 'seconds': elapsed}


def _graph_latency_us(torch, stream, call, launches: int, samples: int = 7) -> float:
    """The reference's timing protocol (benchmark.py:244-268): a CUDA graph of `launches` launches, median of
    `samples` event timings, microseconds per launch."""
    with torch.cuda.stream(stream):
        for _ in range(min(launches, 20)):
            call()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                call()
        graph.replay()
        stream.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        timings = []
        for _ in range(samples):
            begin.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            timings.append(begin.elapsed_time(end) * 1000 / launches)
    return statistics.median(timings)


def reference_kernel_baseline(torch, ops) -> dict | None:
    """The second baseline beside the CPU one: the reference's own kernels on this GPU next to this build's kernels for
    the same problems, both timed as the reference times kernels. Two sets (oracle/build_ref.py): the tf32x3 PTX file
    the reference committed itself (128^3), and the kernels its unmodified compiler emits for sm_100 at 128^3, 512^3,
    2048^3 and 8192^3 in both compensated modes (mma.sync, 32 x 64 tiles, 512-thread CTAs: the schedule of its
    examples/tensor_matmul scaled up). Maximum errors are relative to max|exact|, exact = float64 product on the GPU
    (64 sampled rows above 2048). None when nothing was built."""
    from oracle import ref_kernel, reference_math as oracle
    if not ref_kernel.available():
        return None
    device = torch.device('cuda', 0)
    stream = torch.cuda.Stream(device)
    left = torch.from_numpy(oracle.seeded_normal(7, (128, 128))).to(device)
    right = torch.from_numpy(oracle.seeded_normal(11, (128, 128))).to(device)
    theirs, mine = torch.empty((128, 128), device=device), torch.empty((128, 128), device=device)
    reference = ref_kernel.ReferenceMatmul()
    try:
        with torch.cuda.stream(stream):
            reference_us = _graph_latency_us(torch, stream, lambda: reference.launch(right.data_ptr(), left.data_ptr(), theirs.data_ptr(), stream.cuda_stream), 200)
            ours_us = _graph_latency_us(torch, stream, lambda: ops.gemm(left, right, 'tf32x3', out=mine), 200)
        stream.synchronize()
        identical = bool(torch.equal(theirs, mine))
    finally:
        reference.close()
    out = {'workload': 'gemm_tf32x3_128x128x128 (examples/tensor_matmul)', 'reference_kernel': 'matmul_tiled_128, the reference\'s committed PTX '
           '(docs/video/demo/capture/kernel.ptx) assembled for sm_100a', 'reference_median_us': reference_us, 'ours_median_us': ours_us,
           'outputs_bit_identical': identical, 'timing': 'CUDA graph of 200 launches, median of 7'}
    compiled = []
    available = ref_kernel.manifest()
    generator = torch.Generator(device=device)
    for n, launches in ((128, 200), (512, 200), (2048, 20), (8192, 3)):
        generator.manual_seed(7)
        a = torch.rand((n, n), device=device, generator=generator) * 2 - 1
        generator.manual_seed(11)
        b = torch.rand((n, n), device=device, generator=generator) * 2 - 1
        rows = torch.arange(0, n, max(1, n // 64), device=device) if n > 2048 else torch.arange(n, device=device)
        exact = a[rows].double() @ b.double()
        scale = float(exact.abs().max().item())
        for mode in ('bf16x3', 'tf32x3'):
            name = f'gemm_{mode}_{n}'
            if name not in available:
                continue
            c_ref, c_mine = torch.zeros((n, n), device=device), torch.zeros((n, n), device=device)
            with ref_kernel.ReferenceKernel(name) as kernel:
                pointers = {'left': a.data_ptr(), 'right': b.data_ptr(), 'result': c_ref.data_ptr()}
                with torch.cuda.stream(stream):
                    their_us = _graph_latency_us(torch, stream, lambda: kernel.launch(pointers, stream.cuda_stream), launches, 5)
                    our_us = _graph_latency_us(torch, stream, lambda: ops.gemm(a, b, mode, out=c_mine), launches, 5)
                stream.synchronize()
            compiled.append({'workload': f'gemm_{mode}_{n}x{n}x{n}', 'reference_median_us': their_us, 'ours_median_us': our_us,
                             'reference_tflops': 2.0 * n ** 3 / their_us / 1e6, 'ours_tflops': 2.0 * n ** 3 / our_us / 1e6,
                             'reference_max_rel_error': float((c_ref[rows].double() - exact).abs().max().item()) / scale,
                             'ours_max_rel_error': float((c_mine[rows].double() - exact).abs().max().item()) / scale,
                             'outputs_bit_identical': bool(torch.equal(c_ref, c_mine)), 'launches_per_graph': launches,
                             'reference_registers': available[name].get('registers'), 'reference_grid': available[name]['grid'][0]})
        del a, b, exact
    if compiled:
        out['compiled_by_the_reference_for_sm_100'] = compiled
        out['compiled_how'] = 'unmodified reference compiler (arch sm_100, opt_level 3) with stand-ins for the absent emmy-ml IR classes; ptxas -arch=sm_100a'
    return out


def run_reference(args) -> None:
    """The reference arm: its CPU implementation of the path, on the host cores, rank 0 only."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cores = use_all_host_threads()
    import numpy as np
    from oracle import reference_math as oracle
    right = oracle.seeded_uniform(11, (K, N)).astype(np.float64)
    probe = oracle.seeded_uniform(7, (64, K))
    started = time.perf_counter()
    oracle.gemm_f64(probe, right)
    per_row = (time.perf_counter() - started) / 64
    total_steps = args.steps + args.warmup
    budget = 150.0 / max(total_steps, 1)                       # keep the whole run within a few minutes
    rows = int(min(M, max(64, budget / max(per_row, 1e-6)) // 64 * 64))
    left = oracle.seeded_uniform(7, (rows, K))
    for _ in range(args.warmup):
        oracle.gemm_f64(left, right)
    started = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_f64(left, right)
    elapsed = time.perf_counter() - started
    value = 2.0 * rows * N * K * args.steps / elapsed / 1e12
    sample = f'each step: float64 NumPy product of {rows} of the {M} rows of A with the full B'
    print(json.dumps({
        'impl': 'reference', 'metric': 'bf16x3_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': elapsed / args.steps * 1e3, 'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64', 'data': 'synthetic',
        'config': bench_config(args.gpus), 'sample': sample,
        'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }))


def timed(torch, fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call of fn on the current stream (CUDA events, after warm-up)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters


def reference_kernel_latency_us(torch, name: str, launches: int = 200, samples: int = 6, loaded=None) -> float | None:
    """Warm latency of one kernel the reference's compiler emitted for sm_100 (oracle/_ref), on this GPU, with the
    reference's protocol: its seeded inputs, `zero_outputs` cleared before every launch, a CUDA graph of `launches`
    launches, median of `samples`. None when that kernel was not built. `loaded`: the kernel, already loaded by the
    caller (who then also unloads it)."""
    from oracle import ref_kernel
    records = ref_kernel.manifest()
    if name not in records:
        return None
    from deuteron_b200 import argument_array, jit
    record = records[name]
    device = torch.device('cuda', 0)
    buffers = {arg['name']: torch.from_numpy(argument_array(arg)).to(device) for arg in record['args']}
    pointers = {key: value.data_ptr() for key, value in buffers.items()}
    stream = torch.cuda.Stream(device)

    def timed(kernel) -> float:
        def call():   # the reference's runner clears `zero_outputs` with cuMemsetD8Async before every launch
            for output in record.get('zero_outputs', []):
                jit.memset_zero(buffers[output].data_ptr(), buffers[output].numel() * buffers[output].element_size(), stream.cuda_stream)
            kernel.launch(pointers, stream.cuda_stream)
        with torch.cuda.stream(stream):
            return _graph_latency_us(torch, stream, call, launches, samples)

    if loaded is not None:
        return timed(loaded)
    with ref_kernel.ReferenceKernel(name) as kernel:
        return timed(kernel)


def open_workload_latencies() -> dict:
    """Warm latency of the reference's fifteen open workloads (the shapes of its README table), each compiled from
    scheduled IR and timed as the reference times them: a CUDA graph of 200 launches, median of 6 event timings
    (benchmark.py:244-268) -- of 60 here, on both sides, because a launch of a microsecond follows the clocks and
    these ramp for the first milliseconds of a measurement that starts on an idle GPU; output resets included where the
    launch has them. `reference_b200_us` is the kernel the
    reference's own compiler emits for the same IR, run on this GPU with the same protocol; `reference_rtx5090_us` is
    the reference's published number on other hardware."""
    import math
    import torch
    from deuteron_b200 import LocalRunner, compile_kernel, schedules as S
    published_us = {'p00_scalar_add': 2.976, 'p01_vector_add': 2.976, 'p02_scale_shift': 3.040, 'p03_relu_mul': 2.976, 'r01_array_sum': 2.960,
                    'r02_big_sum': 6.816, 'r03_mean': 4.784, 'r04_row_sum': 2.960, 'm01_matmul_512': 8.896, 'm02_matmul_rect': 3.144,
                    'f01_rmsnorm': 3.152, 'f02_row_softmax': 2.976, 'f03_l2norm': 2.976, 'a01_attention': 4.800, 'a02_attention_128': 4.800}
    cases = [(name, pair, published_us[name]) for name, pair in S.open_workloads().items()]
    out = {}
    # A workload's two kernels are timed one right after the other, each by the median of 60 graph replays. The
    # reference's kernels are all loaded before the first measurement and unloaded after the last. A launch of this
    # build measures 0.2 us shorter in a process that has used one stream only (0.92 against 1.15 us for the vector
    # add) than after another stream has run a graph; the reference's kernels, each on a stream of its own, are always
    # measured in the second state, so this build's are put there too.
    import contextlib
    from oracle import ref_kernel
    available = ref_kernel.manifest()
    with contextlib.ExitStack() as stack, LocalRunner(0) as runner:
        theirs_loaded = {name: stack.enter_context(ref_kernel.ReferenceKernel(f'open_{name}')) for name, _, _ in cases if f'open_{name}' in available}
        if theirs_loaded:   # every timed measurement, the first too, follows a measurement on another stream
            first = next(iter(theirs_loaded))
            reference_kernel_latency_us(torch, f'open_{first}', samples=6, loaded=theirs_loaded[first])
        for name, (graph, meta), published in cases:
            compiled = compile_kernel(graph, meta, arch='sm_100a', opt_level=3)
            result = runner.run_kernel(meta['kernels'][0], compiled, warmup=20, iters=200, samples=60)
            out[name] = {'median_us': result['median_us'], 'reference_rtx5090_us': published}
            if result.get('kernel_only_us') is not None:
                out[name]['kernel_only_us'] = result['kernel_only_us']
            if name in theirs_loaded:
                out[name]['reference_b200_us'] = reference_kernel_latency_us(torch, f'open_{name}', samples=60, loaded=theirs_loaded[name])
    mean = lambda key: math.exp(sum(math.log(v[key]) for v in out.values() if isinstance(v, dict) and key in v) / max(1, sum(1 for v in out.values() if isinstance(v, dict) and key in v)))
    summary = {'geometric_mean_us': mean('median_us'), 'reference_rtx5090_geometric_mean_us': 3.752}
    if all('reference_b200_us' in v for v in out.values()):
        summary['reference_b200_geometric_mean_us'] = mean('reference_b200_us')
    out.update(summary)
    return out


def extras(torch, ops, peaks: dict) -> dict:
    """Other hot kernels at their benchmark sizes (inputs larger than L2), resident inputs."""
    out = {}
    device = torch.device('cuda', torch.cuda.current_device())
    generator = torch.Generator(device=device).manual_seed(7)
    a = torch.rand((M, K), device=device, generator=generator) * 2 - 1
    b = torch.rand((K, N), device=device, generator=generator) * 2 - 1
    c = torch.empty((M, N), device=device)
    ms = timed(torch, lambda: ops.gemm(a, b, 'tf32x3', out=c), 5)
    out['gemm_tf32x3_8192'] = {'ms': ms, 'tflops': FLOPS_PER_GEMM / ms / 1e9}
    # The pool's measured peaks have no TF32 figure: time the library TF32 GEMM here as that denominator.
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    library_ms = timed(torch, lambda: torch.matmul(a, b, out=c), 5)
    torch.backends.cuda.matmul.allow_tf32 = previous
    tf32_peak = FLOPS_PER_GEMM / library_ms / 1e9
    out['gemm_tf32x3_8192'].update({'library_tf32_gemm_tflops': tf32_peak,
                                    'ratio_to_library_tf32_gemm_over_3': out['gemm_tf32x3_8192']['tflops'] / (tf32_peak / 3)})
    del a, b, c
    n = 1 << 28
    x = torch.randn(n, device=device, generator=generator)
    y = torch.randn(n, device=device, generator=generator)
    z = torch.empty_like(x)
    half = torch.empty(n, dtype=torch.float16, device=device)
    half2 = torch.empty_like(half)
    rows = torch.empty(65536, device=device)
    peak = peaks['hbm_gbs']
    for name, fn, nbytes in (
            ('add_f32_2^28', lambda: ops.add(x, y, z), 12 * n),
            ('f16_narrow_2^28', lambda: ops.f16_narrow(x, half), 6 * n),
            ('f16_widen_2^28', lambda: ops.f16_widen(half, z), 6 * n),
            ('f16_copy_2^28', lambda: ops.f16_copy(half, half2), 4 * n),
            ('row_sum_65536x4096', lambda: ops.row_reduce('sum', x.view(65536, 4096), rows), 4 * n + 4 * 65536),
            ('row_max_65536x4096', lambda: ops.row_reduce('max', x.view(65536, 4096), rows), 4 * n + 4 * 65536),
            ('row_softmax_65536x4096', lambda: ops.row_softmax(x.view(65536, 4096), z.view(65536, 4096)), 8 * n),
            ('rms_norm_65536x4096', lambda: ops.rms_norm(x.view(65536, 4096), y[:4096], 1e-5, z.view(65536, 4096)), 8 * n + 4 * 4096),
            ('l2_norm_65536x4096', lambda: ops.l2_norm(x.view(65536, 4096), z.view(65536, 4096)), 8 * n),
            ('row_softmax_16384x16384', lambda: ops.row_softmax(x.view(16384, 16384), z.view(16384, 16384)), 8 * n)):
        ms = timed(torch, fn, 10)
        out[name] = {'ms': ms, 'gbs': nbytes / ms / 1e6, 'frac_of_hbm_peak': nbytes / ms / 1e6 / peak}
        if name.startswith(('row_softmax', 'rms_norm', 'l2_norm')):
            # these run the kernel compiled for the one program (deuteron_b200/jit.py); the library kernel that takes the
            # program as an argument -- what a C-ABI caller of dtn_row_fused gets -- is timed beside it
            out[name]['kernel'] = 'per-program (NVRTC)'
            previous = os.environ.get('DTN_JIT')
            os.environ['DTN_JIT'] = '0'
            try:
                library_ms = timed(torch, fn, 10)
            finally:
                if previous is None:
                    del os.environ['DTN_JIT']
                else:
                    os.environ['DTN_JIT'] = previous
            out[name]['library_kernel'] = {'ms': library_ms, 'gbs': nbytes / library_ms / 1e6, 'frac_of_hbm_peak': nbytes / library_ms / 1e6 / peak}
    del x, y, z, half, half2
    batch, hq, hkv, s, d = 4, 32, 8, 4096, 128
    q = (torch.randn((batch, hq, s, d), device=device, generator=generator) / d ** 0.5).half()
    k = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
    v = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
    o = torch.empty((batch, hq, s, d), device=device)
    import time
    torch.cuda.synchronize()
    time.sleep(3.0)   # the kernel is timed alone (burst peak as denominator): let the clocks recover from the runs above
    ms = timed(torch, lambda: ops.gqa_attention(q, k, v, d ** -0.5, out=o), 10, warmup=3)
    flops = 4.0 * batch * hq * s * s * d
    out['gqa_fwd_b4_h32_kv8_s4096_d128_f16'] = {'ms': ms, 'tflops': flops / ms / 1e9,
                                               'frac_of_bf16_peak': flops / ms / 1e9 / peaks['bf16_tflops'],
                                               'note': '10 launches after 3 s of idle and 3 warm-up launches'}
    return out


def host_link_rate(torch, dist, device, world: int, h2d_bytes: int, d2h_bytes: int) -> dict:
    """The rate at which this job's ranks can move one step's bytes between host and device when all of them copy at
    once: the bound of the end-to-end figure. Plain page-locked copies, one per direction and rank (as many bytes as a
    step moves on that rank), both directions at the same time, three rounds, the fastest; maximum over ranks."""
    up_host = torch.empty(max(h2d_bytes, 1), dtype=torch.uint8, pin_memory=True)
    down_host = torch.empty(max(d2h_bytes, 1), dtype=torch.uint8, pin_memory=True)
    up_dev, down_dev = torch.empty_like(up_host, device=device), torch.empty_like(down_host, device=device)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    best = None
    for _ in range(4):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        begin = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        end = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        begin[0].record(up); begin[1].record(down)
        with torch.cuda.stream(up):
            up_dev.copy_(up_host, non_blocking=True)
        with torch.cuda.stream(down):
            down_host.copy_(down_dev, non_blocking=True)
        end[0].record(up); end[1].record(down)
        torch.cuda.synchronize()
        ms = max(begin[0].elapsed_time(end[0]), begin[1].elapsed_time(end[1]))
        if world > 1:
            gathered = torch.tensor([ms], device=device)
            dist.all_reduce(gathered, op=dist.ReduceOp.MAX)
            ms = float(gathered.item())
        best = ms if best is None else min(best, ms)
    total = torch.tensor([float(h2d_bytes + d2h_bytes)], device=device)
    if world > 1:
        dist.all_reduce(total)
    return {'aggregate_gbs_both_directions': float(total.item()) / best / 1e6, 'ms_for_one_step_bytes': best,
            'how': 'page-locked cudaMemcpyAsync, one copy per direction and rank of that rank\'s bytes of a step, all ranks and '
                   'both directions at once, best of 4, maximum over ranks'}


def sustained_leg(torch, ops, a, b, c, peaks: dict, index: int, seconds: float = 3.0) -> dict:
    """The same step back to back for about `seconds`: the figure of a long run under the power cap, with the clocks it
    ran at. Compared with the sustained library peak, which was taken the same way."""
    for _ in range(3):
        ops.gemm(a, b, 'bf16x3', out=c)
    torch.cuda.synchronize()
    probe_begin, probe_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    probe_begin.record()
    for _ in range(10):
        ops.gemm(a, b, 'bf16x3', out=c)
    probe_end.record()
    torch.cuda.synchronize()
    steps = int(max(50, min(5000, seconds * 1e3 / (probe_begin.elapsed_time(probe_end) / 10))))
    sampler = ClockSampler(index)
    sampler.start()
    time.sleep(0.2)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall_begin = time.perf_counter()
    begin.record()
    for _ in range(steps):
        ops.gemm(a, b, 'bf16x3', out=c)
    end.record()
    torch.cuda.synchronize()
    wall_end = time.perf_counter()
    clocks = sampler.stop(wall_begin, wall_end)
    ms = begin.elapsed_time(end) / steps
    flops = 2.0 * a.shape[0] * b.shape[1] * a.shape[1]
    tflops = flops / ms / 1e9
    out = {'steps': steps, 'seconds': (wall_end - wall_begin), 'ms_per_step': ms, 'tflops': tflops,
           'frac_of_sustained_bf16_peak_over_3': tflops / (peaks['bf16_tflops_sustained'] / 3.0),
           'peak': peaks['bf16_tflops_sustained'] / 3.0, 'clocks': clocks}
    if clocks.get('sm_mhz') and clocks.get('sm_max_mhz'):
        # the same work at the maximum clock, had the power cap not lowered it: step time x median MHz / maximum MHz
        out['tflops_scaled_to_max_clock'] = tflops * clocks['sm_max_mhz'] / clocks['sm_mhz']
    return out


def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    # Libraries (NCCL's version banner) write to stdout; keep stdout for the one JSON line.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the kernels have no CPU path')
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    from deuteron_b200 import LocalRunner, Options, compile_kernel, native, ops, schedules, sharding
    native.lib()
    peaks = measured_peaks()

    # ONE M x N x K product for the whole job (seeds 7 and 11 on every rank); rank r owns the r-th block of output
    # columns: it needs all of A and its own columns of B, and writes its own columns of C. No exchange.
    shards = args.as_rank_of if (world == 1 and args.as_rank_of > 1) else world
    # The microsecond launches of the open workloads are timed first, on a GPU that has done nothing yet: behind the
    # seconds of tensor-bound work below (1 kW, clocks and temperature still settling) the same launches measured
    # 0.2-0.4 us longer, this build's and the reference's alike.
    open_latency = open_workload_latencies() if (world == 1 and shards == 1 and not args.no_extras) else None
    blocks = sharding.column_blocks(N, shards)
    col0, col1 = blocks[rank]
    width = col1 - col0
    generator = torch.Generator(device=device)
    generator.manual_seed(7)
    a = torch.rand((M, K), device=device, generator=generator) * 2 - 1
    generator.manual_seed(11)
    b_full = torch.rand((K, N), device=device, generator=generator) * 2 - 1
    b = b_full[:, col0:col1].contiguous() if shards > 1 else b_full    # the rank's columns of B, as they arrive from its host
    c = torch.empty((M, width), device=device)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(value: float, op=None) -> float:
        if world == 1:
            return value
        gathered = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(gathered, op=op or dist.ReduceOp.MAX)
        return float(gathered.item())

    for _ in range(max(args.warmup, 3)):
        ops.gemm(a, b, 'bf16x3', out=c)
    ops.check_device_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    wall_begin = time.perf_counter()
    for step in range(args.steps):
        events[step][0].record()
        ops.gemm(a, b, 'bf16x3', out=c, phase=1 | 4)  # split of the rank's columns of B: 1 kernel
        events[step][1].record()
        ops.gemm(a, b, 'bf16x3', out=c, phase=3 | 8)  # product kernel, which splits A beside its products: 1 kernel
        events[step][2].record()
    barrier()
    wall_end = time.perf_counter()
    total_ms = over_ranks(events[0][0].elapsed_time(events[-1][2]))
    product_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in events)
    split_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in events)
    slowest_product_ms = over_ranks(product_ms)
    ops.check_device_status()
    clocks = sampler.stop(wall_begin, wall_end) if rank == 0 else None
    value = FLOPS_PER_GEMM * args.steps / total_ms / 1e9      # the one product's flops / the slowest rank's time

    # Parity spot check inside the bench: 32 sampled rows of this rank's columns against a float64 product of the
    # GPU's own data; the figure of the line is the worst rank's.
    sample_rows = torch.arange(0, M, M // 32, device=device)
    exact = a[sample_rows].double() @ b.double()
    rel_error = over_ranks(float(((c[sample_rows].double() - exact).abs().max() / exact.abs().max()).item()))
    del exact

    # Weak-scaling companion at N > 1: every rank multiplies a full 8192-wide block of its own (the previous form of
    # this line; no exchange either), for comparison with the strong figure.
    replicas = None
    if world > 1:
        c_wide = torch.empty((M, N), device=device)
        for _ in range(3):
            ops.gemm(a, b_full, 'bf16x3', out=c_wide)
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        replica_steps = max(3, min(args.steps, 10))
        begin.record()
        for _ in range(replica_steps):
            ops.gemm(a, b_full, 'bf16x3', out=c_wide)
        end.record()
        end.synchronize()
        replica_ms = over_ranks(begin.elapsed_time(end) / replica_steps)
        replicas = {'what': f'every rank multiplies its own {M} x {N} x {K} (weak scaling, no exchange)', 'ms_per_step': replica_ms,
                    'tflops_aggregate': FLOPS_PER_GEMM * world / replica_ms / 1e9, 'scaling': 'weak'}
        del c_wide

    # End to end, host buffers in, host buffers out. One GPU: compile_kernel + LocalRunner.execute. Several GPUs:
    # compile_kernel + sharding.ShardedHostProduct (every rank feeds its columns of B and 1/N of A's rows from its own
    # page-locked host memory, the rows of A are exchanged over NVLink, its columns of C return to its host).
    e2e = None
    if shards == world:
        graph, meta = schedules.matmul_example(M, N, K)
        compiled = compile_kernel(graph, meta, arch='sm_100a', opt_level=3, options=Options(contraction_precision='bf16x3'))
        e2e_steps = max(3, min(args.steps, 10))
        a_host_full, b_host_full = a.cpu().numpy(), b_full.cpu().numpy()
        with LocalRunner(local_rank) as runner:
            if world == 1:
                host = {'left': runner.pinned((M, K), np.float32), 'right': runner.pinned((K, N), np.float32)}
                host['left'][:] = a_host_full
                host['right'][:] = b_host_full
                result = {'result': runner.pinned((M, N), np.float32)}
                run_e2e = lambda: runner.execute(compiled, host, result, synchronize=True)
                h2d, d2h = 4 * (M * K + K * N), 4 * M * N
                produced = result['result']
                call = 'compile_kernel + LocalRunner.execute (pinned host buffers)'
                stream = runner.stream
            else:
                product = sharding.ShardedHostProduct(compiled, rank, world, device)
                rows_host = runner.pinned((product.owned_row_count, K), np.float32)
                rows_host[:] = product.pack_rows(a_host_full)
                cols_host = runner.pinned((K, width), np.float32)
                cols_host[:] = b_host_full[:, col0:col1]
                produced = runner.pinned((M, width), np.float32)
                run_e2e = lambda: product.execute(rows_host, cols_host, produced, synchronize=True)
                h2d, d2h = product.host_bytes()
                call = ('compile_kernel + sharding.ShardedHostProduct.execute (pinned host buffers; each rank feeds its columns of B and '
                        f'1/{world} of the rows of A, NCCL all-gather of the rows of A, {len(product.plan)} row blocks in flight)')
                stream = product.compute
            del a_host_full, b_host_full
            for _ in range(2):
                run_e2e()
            barrier()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            for _ in range(e2e_steps):
                run_e2e()
            end.record(stream)
            end.synchronize()
            e2e_ms = over_ranks(begin.elapsed_time(end))
            matches = over_ranks(float(np.array_equal(produced[::64], c[::64].cpu().numpy())), dist.ReduceOp.MIN if world > 1 else None)
            h2d_total, d2h_total = int(over_ranks(float(h2d), dist.ReduceOp.SUM if world > 1 else None)), \
                int(over_ranks(float(d2h), dist.ReduceOp.SUM if world > 1 else None))
            link = host_link_rate(torch, dist, device, world, h2d, d2h)
            e2e = {'value': FLOPS_PER_GEMM * e2e_steps / e2e_ms / 1e9, 'unit': 'TFLOP/s',
                   'h2d_bytes_per_step': h2d_total, 'd2h_bytes_per_step': d2h_total,
                   'h2d_bytes_per_step_rank0': h2d, 'd2h_bytes_per_step_rank0': d2h, 'steps': e2e_steps,
                   'ms_per_step': e2e_ms / e2e_steps, 'call': call, 'matches_resident_result': bool(matches),
                   'host_link': link, 'ms_per_step_over_host_link_ms': e2e_ms / e2e_steps / link['ms_for_one_step_bytes']}
            del produced

    # The second sharded path, at N > 1 only: one GQA forward (B=4, 32/8 heads, S=4096, D=128) split over the ranks by
    # (batch, kv-head) groups, no exchange; aggregate = the whole problem's flops / the slowest rank's time.
    gqa_sharded = None
    if world > 1 and not args.no_extras:
        # Every rank reaches every barrier and collective below whatever happens in between, so that a failure on
        # one rank can neither hang the others nor cost the line above.
        batch, hq, hkv, s, d = 4, 32, 8, 4096, 128
        groups = sharding.group_range(batch * hkv, world, rank)
        failed, local_ms, run = 0.0, 0.0, None
        try:
            del a, b, b_full
            torch.cuda.empty_cache()
            generator.manual_seed(7)
            q = (torch.randn((batch, hq, s, d), device=device, generator=generator) / d ** 0.5).half()
            kk = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
            vv = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
            o = torch.zeros((batch, hq, s, d), device=device)
            run = lambda: ops.gqa_attention(q, kk, vv, d ** -0.5, out=o, groups=groups)
            for _ in range(3):
                run()
        except Exception as error:   # noqa: BLE001 - reported in the line
            failed, run = 1.0, None
            print(f'rank {rank}: sharded attention set-up failed: {error}', file=sys.stderr)
        barrier()
        try:
            if run is not None:
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                for _ in range(10):
                    run()
                end.record()
                end.synchronize()
                local_ms = begin.elapsed_time(end) / 10
                ops.check_device_status()
        except Exception as error:   # noqa: BLE001
            failed = 1.0
            print(f'rank {rank}: sharded attention failed: {error}', file=sys.stderr)
        barrier()
        gathered = torch.tensor([local_ms, failed], device=device)
        dist.all_reduce(gathered, op=dist.ReduceOp.MAX)
        gqa_ms, any_failed = float(gathered[0].item()), float(gathered[1].item()) > 0
        flops = 4.0 * batch * hq * s * s * d
        if any_failed or gqa_ms <= 0:
            gqa_sharded = {'workload': 'gqa_fwd_b4_h32_kv8_s4096_d128_f16', 'error': 'a rank failed; see stderr'}
        else:
            gqa_sharded = {'workload': 'gqa_fwd_b4_h32_kv8_s4096_d128_f16', 'groups_per_rank': groups[1] - groups[0], 'ms': gqa_ms,
                           'tflops_aggregate': flops / gqa_ms / 1e9, 'scaling': 'strong',
                           'frac_of_bf16_peak_per_gpu': flops / gqa_ms / 1e9 / world / peaks['bf16_tflops']}
            # the optional exchange of this path: all-gather of the finished (batch, kv-head) groups
            try:
                ranges = [sharding.group_range(batch * hkv, world, r) for r in range(world)]
                for _ in range(2):
                    sharding.all_gather_groups(o, hq // hkv, ranges)
                barrier()
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                for _ in range(5):
                    sharding.all_gather_groups(o, hq // hkv, ranges)
                end.record()
                end.synchronize()
                gather_ms = over_ranks(begin.elapsed_time(end) / 5)
                gqa_sharded['all_gather_of_groups_ms'] = gather_ms
                gqa_sharded['all_gather_gbs_received_per_rank'] = (world - 1) / world * o.numel() * 4 / gather_ms / 1e6
            except Exception as error:   # noqa: BLE001
                print(f'rank {rank}: all-gather of attention groups failed: {error}', file=sys.stderr)
                barrier()

    if rank == 0:
        peak = peaks['bf16_tflops'] / 3.0
        flops_per_rank = 2.0 * M * width * K
        achieved = flops_per_rank / product_ms / 1e9
        algorithmic_bytes = 8 * M * K + 2 * 2 * (M * K + width * K) + 4 * M * width   # A read and its planes written; four planes read once; C written
        line = {
            'metric': 'bf16x3_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': total_ms / args.steps, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'bf16x3 (bf16 hi/lo operands, f32 accumulate, f32 in/out)', 'data': 'synthetic',
            'config': bench_config(shards),
            'step': f'split of the rank\'s {width} columns of B (1 kernel) + tcgen05 product kernel with the split of A running '
                    'inside it (1 kernel, preceded by a memset of its counters)',
            'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s', 'frac': achieved / peak,
                         'frac_of_nominal': achieved / (2250.0 / 3.0),
                         'traffic': PRODUCT_KERNEL_DRAM_BYTES if world == 1 else None,
                         'traffic_note': 'bytes per launch from the committed ncu capture of the 8192^3 launch; algorithmic '
                         f'bytes per launch of this rank {algorithmic_bytes:.3e}',
                         'kernel': 'gemm_x3_stream_kernel (products + split of A, rank 0)', 'ms_per_launch': product_ms,
                         'ms_per_launch_slowest_rank': slowest_product_ms, 'split_ms_per_step': split_ms,
                         'peak_source': f"{peaks['source']} dense bf16 burst peak {peaks['bf16_tflops']} TFLOP/s / 3 products; "
                                        'frac_of_nominal uses the nominal 2250 TFLOP/s / 3'},
            'clocks': clocks,
            'e2e': e2e,
            'gpu_launches': 2 * args.steps,
            'max_rel_error_vs_f64_sampled_rows': rel_error,
        }
        if line['roofline']['frac'] > 1.0:
            line['roofline']['note'] = 'above 1: the measured library peak is a lower bound of the hardware peak, see frac_of_nominal'
        extras_out = {}
        if replicas is not None:
            extras_out['replicas_weak_scaling'] = replicas
        if gqa_sharded is not None:
            extras_out['gqa_sharded_by_groups'] = gqa_sharded
        if shards > world:
            line['emulated'] = (f'one GPU timed the step of rank 0 of a {shards}-GPU run ({width} of the {N} columns); value = the whole '
                                'product over that time, what the job reaches if every rank takes as long; no end-to-end figure')
        if world == 1 and shards == 1 and not args.no_cpu_baseline:
            line['cpu_baseline'] = cpu_gemm_sample()
            reference_gpu = reference_kernel_baseline(torch, ops)
            if reference_gpu is not None:
                line['reference_kernel_baseline'] = reference_gpu
        if world == 1 and shards == 1 and not args.no_extras:
            line['sustained'] = sustained_leg(torch, ops, a, b, c, peaks, local_rank)
            del a, b, b_full, c
            torch.cuda.empty_cache()
            extras_out.update(extras(torch, ops, peaks))
            extras_out['open_workload_latency'] = open_latency
        if extras_out:
            line['extras'] = extras_out
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


SWEEP_GEMMS = ((16, 8192, 8192), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (16384, 16384, 16384))   # by work
SWEEP_ATTENTION = (512, 2048, 8192, 16384)      # batch 8, 64 query / 8 kv heads, head_dim 128, f16 storage


def run_sweep(args) -> None:
    """The mixed sweep of the largest configuration, each problem split over the ranks (strong scaling): a GEMM by
    output column blocks, an attention forward by (batch, kv-head) groups; N(0,1) inputs from fixed seeds.

    Every launch is timed with its own pair of events on the launching stream; a 512 MiB buffer is overwritten
    between launches so that no problem starts with its operands in L2. The figure of a problem is the median over
    its launches, maximum over ranks; rank 0 prints one JSON line.
    """
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the kernels have no CPU path')
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    from deuteron_b200 import native, ops, sharding
    native.lib()
    peaks = measured_peaks()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    # read after the write: the lines the write leaves in L2 are dirty, and a launch timed right behind it pays for
    # their write-back (126 MB beside its own traffic); a pass of reads over other memory leaves clean lines behind
    cold = torch.zeros(256 << 20, dtype=torch.uint8, device=device)
    generator = torch.Generator(device=device)

    def normal(seed: int, shape, scale: float = 1.0):
        generator.manual_seed(seed)
        return torch.randn(shape, device=device, generator=generator) * scale

    def measure(make, budget_ms: float) -> tuple[float, bool]:
        """Median milliseconds per launch of the callable `make()` builds (0 when this rank owns nothing), and whether
        anything failed on this rank. Never raises: every rank must reach the collectives that follow."""
        try:
            call = make()
            if call is None:
                return 0.0, False
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            # One call is up to three kernels; enqueued from Python the second reaches the GPU after the first has
            # finished when the problem is small, and the events would time the interpreter. The call is captured
            # once and replayed, as the reference's runner does with its launches (benchmark.py:246-262).
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                call()
            call = graph.replay
            call()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            call()
            end.record()
            end.synchronize()
            launches = int(max(3, min(30, budget_ms / max(begin.elapsed_time(end), 1e-3))))
            time.sleep(0.5)   # every problem starts from an idle GPU, whatever ran before it
            samples = []
            for _ in range(launches):
                flush.fill_(1)
                cold.max()
                begin.record()
                call()
                end.record()
                end.synchronize()
                samples.append(begin.elapsed_time(end))
            ops.check_device_status()
            return statistics.median(samples), False
        except Exception as error:   # noqa: BLE001 - reported in the line
            print(f'rank {rank}: sweep item failed: {error}', file=sys.stderr)
            return 0.0, True

    def over_ranks(ms: float, failed: bool) -> tuple[float, bool]:
        if world == 1:
            return ms, failed
        gathered = torch.tensor([ms, float(failed)], device=device)
        dist.all_reduce(gathered, op=dist.ReduceOp.MAX)
        return float(gathered[0].item()), float(gathered[1].item()) > 0

    sampler = ClockSampler(local_rank)
    wall_begin = time.perf_counter()
    if rank == 0:
        sampler.start()
    batch, hq, hkv, d = 8, 64, 8, 128
    jobs = [('gemm', 2.0 * m * n * k, (mode, m, n, k)) for mode in ('bf16x3', 'tf32x3') for m, n, k in SWEEP_GEMMS]
    jobs += [('attention', 4.0 * batch * hq * s * s * d, (s,)) for s in SWEEP_ATTENTION]
    jobs.sort(key=lambda job: job[1])   # ascending work: a small problem is not timed in the wake of a long one
    items = []
    for kind, flops, spec in jobs:
        holder = {}
        if kind == 'gemm':
            mode, m, n, k = spec
            begin_col, end_col = sharding.column_blocks(n, world)[rank]

            def make(m=m, k=k, width=end_col - begin_col, mode=mode, holder=holder):
                if width == 0:
                    return None
                holder['a'], holder['b'] = normal(7, (m, k)), normal(11 + rank, (k, width))
                holder['c'] = torch.empty((m, width), device=device)
                return lambda: ops.gemm(holder['a'], holder['b'], mode, out=holder['c'])

            item = {'kernel': f'gemm_{mode}', 'm': m, 'n': n, 'k': k, 'columns_per_rank': end_col - begin_col}
        else:
            (s,) = spec
            groups = sharding.group_range(batch * hkv, world, rank)

            def make(s=s, groups=groups, holder=holder):
                if groups[1] == groups[0]:
                    return None
                holder['q'] = normal(7, (batch, hq, s, d)).half()
                holder['k'] = normal(8, (batch, hkv, s, d)).half()
                holder['v'] = normal(9, (batch, hkv, s, d)).half()
                holder['o'] = torch.empty((batch, hq, s, d), device=device)
                return lambda: ops.gqa_attention(holder['q'], holder['k'], holder['v'], d ** -0.5, out=holder['o'], groups=groups)

            item = {'kernel': 'gqa_fwd_f16', 'batch': batch, 'q_heads': hq, 'kv_heads': hkv, 'seq_len': s, 'head_dim': d,
                    'groups_per_rank': groups[1] - groups[0]}
        ms, failed = over_ranks(*measure(make, 300.0 if kind == 'gemm' else 400.0))
        holder.clear()
        torch.cuda.empty_cache()
        if failed or ms <= 0:
            item['error'] = 'a rank failed; see stderr'
        else:
            tflops = flops / ms / 1e9
            item.update(ms=ms, tflops_aggregate=tflops)
            if kind == 'gemm' and spec[1] <= 16:
                item['b_gbs_aggregate'] = 4.0 * spec[2] * spec[3] / ms / 1e6
                item['frac_of_hbm_peak_per_gpu'] = item['b_gbs_aggregate'] / world / peaks['hbm_gbs']
            elif kind == 'gemm' and spec[0] == 'bf16x3':
                item['frac_of_bf16_peak_over_3_per_gpu'] = tflops / world / (peaks['bf16_tflops'] / 3.0)
                item['frac_of_sustained_bf16_peak_over_3_per_gpu'] = tflops / world / (peaks['bf16_tflops_sustained'] / 3.0)
            elif kind == 'attention':
                item['frac_of_bf16_peak_per_gpu'] = tflops / world / peaks['bf16_tflops']
                item['frac_of_sustained_bf16_peak_per_gpu'] = tflops / world / peaks['bf16_tflops_sustained']
        items.append(item)
    torch.cuda.synchronize()
    wall_end = time.perf_counter()
    if rank == 0:
        line = {'metric': 'mixed_sweep', 'n_gpus': world, 'scaling': 'strong', 'data': 'synthetic', 'unit': 'TFLOP/s',
                'config': {'workload': 'mixed_sweep_gemm_1024_2048_4096_16384_skinny16_attention_512_2048_8192_16384',
                           'inputs': 'N(0,1), seeds 7 / 11+rank (GEMM), 7 / 8 / 9 (attention, f16 storage)',
                           'parallelism': f'each problem split x{world}: GEMM by output column blocks, attention by (batch, kv-head) groups; no collective',
                           'l2': '512 MiB written, then 256 MiB of other memory read, between launches (cold L2 without dirty lines)',
                           'timing': 'problems in ascending order of work, 0.5 s idle before the timed launches of each; '
                                     'one call captured in a CUDA graph and replayed between CUDA events; '
                                     'median over launches, maximum over ranks'},
                'peaks': {'bf16_tflops': peaks['bf16_tflops'], 'bf16_tflops_sustained': peaks['bf16_tflops_sustained'],
                          'hbm_gbs': peaks['hbm_gbs'], 'source': peaks['source'],
                          'note': 'launches of tens of milliseconds run at the clocks of the power cap: compare them with the sustained peak'},
                'clocks': sampler.stop(wall_begin, wall_end), 'items': items}
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_all_gather(args) -> None:
    """Times the optional exchange that follows the sharded GEMM, two ways: the all-gather (NCCL) of the ranks' finished
    8192 x 8192 output blocks into the full 8192 x (8192 * N) product on every rank, after the GEMM; and
    `sharding.GatheredProduct`, which pushes finished row blocks into the peers' copies (symmetric memory, peer stores
    over NVLink) while the rest is multiplied. Opt-in (`--all-gather`), never part of the default line: the data path
    itself has no collective."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world < 2:
        raise SystemExit('--all-gather needs --gpus 2 or more')
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    dist.init_process_group('nccl', device_id=device)
    from deuteron_b200 import ops, sharding
    generator = torch.Generator(device=device)
    generator.manual_seed(7)
    a = torch.rand((M, K), device=device, generator=generator) * 2 - 1
    generator.manual_seed(11 + rank)
    b = torch.rand((K, N), device=device, generator=generator) * 2 - 1
    block = torch.empty((M, N), device=device)
    blocks = sharding.column_blocks(N * world, world)
    iters = max(3, min(args.steps, 10))

    def timed(call) -> float:
        for _ in range(2):
            call()
        dist.barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(iters):
            call()
        end.record()
        end.synchronize()
        gathered = torch.tensor([begin.elapsed_time(end) / iters], device=device)
        dist.all_reduce(gathered, op=dist.ReduceOp.MAX)
        return float(gathered.item())

    def gemm_then_gather():
        ops.gemm(a, b, 'bf16x3', out=block)
        return sharding.all_gather_columns(block, blocks)

    gemm_ms = timed(lambda: ops.gemm(a, b, 'bf16x3', out=block))
    gather_ms = timed(lambda: sharding.all_gather_columns(block, blocks))
    sequential_ms = timed(gemm_then_gather)
    expected = gemm_then_gather()
    overlapped_ms, identical, failure = None, None, None
    try:
        product = sharding.GatheredProduct(M, N * world, rank, world, device, row_blocks=args.row_blocks or None)
        overlapped_ms = timed(lambda: product.run(a, b, 'bf16x3'))
        full = product.run(a, b, 'bf16x3')
        torch.cuda.synchronize()
        same = torch.tensor([float(torch.equal(full, expected))], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        identical = bool(same.item())
    except Exception as error:   # noqa: BLE001 - symmetric memory may be unavailable; the NCCL figures stand
        failure = repr(error)[:200]
    ops.check_device_status()
    if rank == 0:
        received = (world - 1) * M * N * 4
        flops = FLOPS_PER_GEMM * world
        line = {'metric': 'gemm_with_all_gather_of_output_column_blocks', 'n_gpus': world, 'block_bytes': M * N * 4,
                'bytes_received_per_rank': received, 'gemm_ms': gemm_ms, 'all_gather_ms': gather_ms,
                'all_gather_gbs_received_per_rank': received / gather_ms / 1e6,
                'gemm_then_all_gather_ms': sequential_ms, 'gemm_then_all_gather_tflops': flops / sequential_ms / 1e9,
                'overlapped_ms': overlapped_ms, 'overlapped_tflops': flops / overlapped_ms / 1e9 if overlapped_ms else None,
                'overlapped_result_identical': identical, 'overlapped_failure': failure,
                'note': 'all_gather = torch.distributed all_gather (NCCL) plus the permute into row-major; overlapped = '
                        f'sharding.GatheredProduct ({len(product.rows) if identical is not None else 0} row blocks, dtn_push_block on a side stream, barrier at the end); max over ranks'}
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


PROFILE_CASES = ('gemm_bf16x3', 'gemm_tf32x3', 'gemm_bf16x3_8192', 'gemm_bf16x3_2048', 'gemm_skinny', 'attention', 'add', 'f16_narrow', 'f16_widen', 'f16_copy', 'row_sum', 'row_max',
                 'row_softmax', 'rms_norm', 'fused_affine')


def run_profile_case(name: str, launches: int) -> None:
    """A small, self-ending case of one kernel for a profiler capture: inputs larger than the L2 where
    the kernel is memory-bound, well under a GB on the device, `launches` launches, then exit."""
    import torch
    from deuteron_b200 import ops
    torch.cuda.set_device(0)
    device = torch.device('cuda', 0)
    generator = torch.Generator(device=device).manual_seed(7)
    if name == 'gemm_skinny':
        a = torch.rand((16, 8192), device=device, generator=generator) * 2 - 1
        b = torch.rand((8192, 8192), device=device, generator=generator) * 2 - 1
        c = torch.empty((16, 8192), device=device)
        call = lambda: ops.gemm(a, b, 'bf16x3', out=c)
    elif name == 'fused_affine':
        from deuteron_b200 import compile_kernel, native, schedules
        n = 1 << 26
        plan = compile_kernel(*schedules.pointwise_example('affine', n)).plan
        x = torch.randn(n, device=device, generator=generator)
        z = torch.empty_like(x)
        constants = {'mul_c1': torch.tensor([2.0], device=device), 'add_c1': torch.tensor([1.0], device=device), 'x': x}
        pointers = [constants[plan.buffers[f'in{i}'][0]].data_ptr() for i in range(len(plan.params['inputs']))]
        call = lambda: native.elementwise_program(plan.params, pointers, z.data_ptr(), torch.cuda.current_stream().cuda_stream)
    elif name.startswith('gemm_'):
        n = int(name.rsplit('_', 1)[1]) if name.rsplit('_', 1)[1].isdigit() else 4096
        name = name if not name.rsplit('_', 1)[1].isdigit() else name.rsplit('_', 1)[0]
        a = torch.rand((n, n), device=device, generator=generator) * 2 - 1
        b = torch.rand((n, n), device=device, generator=generator) * 2 - 1
        c = torch.empty((n, n), device=device)
        call = lambda: ops.gemm(a, b, name[5:], out=c)
    elif name == 'attention':
        batch, hq, hkv, s, d = 2, 16, 4, 4096, 128   # 512 work items of 256 queries: 3.5 per SM
        q = (torch.randn((batch, hq, s, d), device=device, generator=generator) / d ** 0.5).half()
        k = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
        v = (torch.randn((batch, hkv, s, d), device=device, generator=generator) / d ** 0.5).half()
        o = torch.empty((batch, hq, s, d), device=device)
        call = lambda: ops.gqa_attention(q, k, v, d ** -0.5, out=o)
    else:
        n = 1 << 26
        x = torch.randn(n, device=device, generator=generator)
        y = torch.randn(n, device=device, generator=generator)
        z = torch.empty_like(x)
        half = torch.empty(n, dtype=torch.float16, device=device)
        half2 = torch.empty_like(half)
        rows = torch.empty(16384, device=device)
        call = {'add': lambda: ops.add(x, y, z), 'f16_narrow': lambda: ops.f16_narrow(x, half),
                'f16_widen': lambda: ops.f16_widen(half, z), 'f16_copy': lambda: ops.f16_copy(half, half2),
                'row_sum': lambda: ops.row_reduce('sum', x.view(16384, 4096), rows),
                'row_max': lambda: ops.row_reduce('max', x.view(16384, 4096), rows),
                'row_softmax': lambda: ops.row_softmax(x.view(16384, 4096), z.view(16384, 4096)),
                'rms_norm': lambda: ops.rms_norm(x.view(16384, 4096), y[:4096], 1e-5, z.view(16384, 4096))}[name]
    for _ in range(launches):
        call()
    torch.cuda.synchronize()
    ops.check_device_status()
    print(json.dumps({'profile_case': name, 'launches': launches}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument('--profile-case', choices=PROFILE_CASES, help='run a small case of one kernel and exit')
    parser.add_argument('--launches', type=int, default=3)
    parser.add_argument('--gpus', type=int, default=1)
    parser.add_argument('--steps', type=int, default=200)
    parser.add_argument('--warmup', type=int, default=3)
    parser.add_argument('--impl', choices=('ours', 'reference'), default='ours')
    parser.add_argument('--as-rank-of', type=int, default=0, metavar='N',
                        help='on one GPU, time the step rank 0 of an N-GPU run would do (its block of columns); the value is '
                             'what the N-GPU job reaches if every rank takes that long. The line says so; end to end is skipped')
    parser.add_argument('--no-cpu-baseline', action='store_true')
    parser.add_argument('--no-extras', action='store_true')
    parser.add_argument('--row-blocks', type=int, default=0, help='row blocks of the overlapped exchange (--all-gather); 0 = automatic')
    parser.add_argument('--all-gather', action='store_true', help='time the optional all-gather of the output column blocks (N > 1)')
    parser.add_argument('--sweep', action='store_true', help='time the mixed sweep of GEMM and attention sizes, each split over the ranks')
    args = parser.parse_args()
    if args.steps < 1 or args.warmup < 0:
        raise SystemExit('steps must be positive and warmup nonnegative')
    if args.profile_case:
        run_profile_case(args.profile_case, max(args.launches, 1))
        return
    if args.impl == 'reference':
        run_reference(args)
        return
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun when called directly with --gpus N
        command = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={args.gpus}',
                   '--master-addr', '127.0.0.1', '--master-port', '29511', __file__, *sys.argv[1:]]
        raise SystemExit(subprocess.call(command))
    if args.all_gather:
        run_all_gather(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    run_ours(args)


if __name__ == '__main__':
    main()
