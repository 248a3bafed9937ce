"""Per-program kernels for small fused elementwise and row programs, row reductions and the attention example.

The library's kernels for these plans take the register program as an argument, which is what a memory-bound launch
wants (one kernel, any program, the decode paid once per eight elements). A latency-bound launch -- a few thousand
elements, one wave of threads -- is as long as one thread's instruction chain, and there the decode is most of the
chain: four to nine times the instructions of a kernel written for the one program. The reference is a compiler and
emits such a kernel for every workload (compiler/codegen/lower.py). This module does the same for the plan kinds
where it matters (KINDS): it writes the program out as CUDA C++ with every operator inlined, in the operator table's
own arithmetic (csrc/program.cuh: one rounding per operator, never contracted into fma, the approximate exp / sqrt /
rsqrt / reciprocal instructions), has NVRTC compile it for sm_100a and launches it through the driver API. The
reference-layout attention of a few hundred rows gets a kernel unrolled for its shape in the same way, with the
library kernel's order of operations.

Used by LocalRunner and by the row operators of ops.py; every program this module does not take (rows longer than
32 768 columns or not a multiple of four, misaligned buffers, long plain reductions) runs the library's kernels, and so
does everything when NVRTC is missing. `DTN_JIT=0` turns it off. Nothing here needs a GPU to generate or compile (NVRTC targets an
architecture, not a device); loading and launching need the current CUDA context.
"""
from __future__ import annotations

import ctypes as ct
import hashlib
import os
import threading
from typing import Any

PRELUDE = r'''
typedef long long i64;
__device__ __forceinline__ float dtn_ex2(float x) { float y; asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float dtn_exp(float x) { return dtn_ex2(__fmul_rn(x, 1.4426950408889634f)); }
__device__ __forceinline__ float dtn_sqrt(float x) { float y; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float dtn_rsqrt(float x) { float y; asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float dtn_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float dtn_h2f(unsigned short h) { float y; asm("cvt.f32.f16 %0, %1;" : "=f"(y) : "h"(h)); return y; }
__device__ __forceinline__ unsigned short dtn_f2h(float x) { unsigned short h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(x)); return h; }
'''

# operator code (native.ELEMENTWISE_OPS) -> expression over `a` and `b`, in the arithmetic of csrc/program.cuh::prog_apply
_OPERATORS = {
    0: '__fadd_rn({a}, {b})', 1: '__fsub_rn({a}, {b})', 2: '__fmul_rn({a}, {b})', 3: '__fdividef({a}, {b})',
    4: 'fmaxf({a}, {b})', 5: 'fminf({a}, {b})', 6: 'fmaxf({a}, 0.0f)', 7: 'dtn_exp({a})', 8: 'dtn_sqrt({a})',
    9: 'dtn_rsqrt({a})', 10: 'dtn_rcp({a})', 11: '(-{a})', 12: 'fabsf({a})', 13: '({a})',
}
KINDS = ('elementwise_program', 'row_fused', 'row_reduce', 'attention')   # plan kinds this module may take
SMALL_ELEMENTS = 1 << 16      # plain reductions above this many elements go to the library's kernels
_COMPONENTS = 'xyzw'


def enabled() -> bool:
    return os.environ.get('DTN_JIT', '1') != '0'


def apply(op: int, a: str, b: str) -> str:
    return _OPERATORS[op].format(a=a, b=b)


# ------------------------------------------------------------------------------------------------
# elementwise programs (classify._program_plan / dtn_elementwise_program)
# ------------------------------------------------------------------------------------------------
def elementwise_source(params: dict, buffers: dict) -> dict | None:
    """CUDA source of one kernel for the register program `params`, or None when this module does not take it:
    a multiple of four elements, every vector buffer at a multiple of four elements from its start (so that its
    vector accesses are aligned). f16 buffers are widened exactly on load and the result is rounded to nearest even
    on store, as in csrc/elementwise_program.cu; a thread takes eight elements when there is an f16 buffer and the
    count allows, four otherwise. Any size: with nothing to decode the kernel also streams faster than the library's
    (x * a + b over 2^26 FP32 elements: 6.5 against 5.6 TB/s)."""
    inputs, n = params['inputs'], params['n']
    if n < 4 or n % 4 or any(op not in _OPERATORS for op in params['ops']):
        return None
    vector_offsets = [buffers['out'][1]] + [buffers[f'in{i}'][1] for i, spec in enumerate(inputs) if not spec['scalar']]
    if any(offset % 4 for offset in vector_offsets):
        return None
    halves = params['out_f16'] or any(spec['f16'] for spec in inputs)
    width = 8 if halves and n % 8 == 0 and not any(offset % 8 for offset in vector_offsets) else 4
    registers = max([params['out_reg'], len(inputs) - 1, *params['dst'], *params['a'], *params['b']]) + 1
    lines = ['__device__ __forceinline__ float dtn_element(' + ', '.join(f'float in{i}' for i in range(len(inputs))) + ') {']
    lines.append('  float ' + ', '.join(f'r{k} = {"in%d" % k if k < len(inputs) else "0.0f"}' for k in range(registers)) + ';')
    for op, dst, a, b in zip(params['ops'], params['dst'], params['a'], params['b']):
        lines.append(f'  r{dst} = {apply(op, f"r{a}", f"r{b}")};')
    lines += [f'  return r{params["out_reg"]};', '}']
    arguments = ', '.join(f'const void* __restrict__ p{i}' for i in range(len(inputs)))
    lines.append(f'extern "C" __global__ void __launch_bounds__(256) dtn_jit_kernel({arguments}{", " if inputs else ""}void* __restrict__ out, i64 pieces) {{')
    lines.append('  const i64 v = (i64)blockIdx.x * 256 + threadIdx.x;')
    for i, spec in enumerate(inputs):   # scalars are read before the bounds check: their latency overlaps the vector loads
        if spec['scalar']:
            value = f'dtn_h2f(__ldg(static_cast<const unsigned short*>(p{i})))' if spec['f16'] else f'__ldg(static_cast<const float*>(p{i}))'
            lines.append(f'  const float s{i} = {value};')
    lines.append('  if (v >= pieces) return;')
    vector_type = 'uint4' if width == 8 else 'uint2'
    for i, spec in enumerate(inputs):
        if spec['scalar']:
            continue
        lines.append(f'  float x{i}[{width}];')
        if spec['f16']:
            lines.append(f'  {{ const {vector_type} w = __ldg(static_cast<const {vector_type}*>(p{i}) + v);')
            for e, word in enumerate(_COMPONENTS[:width // 2]):
                lines.append(f'    x{i}[{2 * e}] = dtn_h2f((unsigned short)(w.{word} & 0xffffu)); x{i}[{2 * e + 1}] = dtn_h2f((unsigned short)(w.{word} >> 16));')
            lines.append('  }')
        else:
            for part in range(width // 4):
                lines.append(f'  {{ const float4 w = __ldg(static_cast<const float4*>(p{i}) + v * {width // 4} + {part});'
                             f' x{i}[{4 * part}] = w.x; x{i}[{4 * part + 1}] = w.y; x{i}[{4 * part + 2}] = w.z; x{i}[{4 * part + 3}] = w.w; }}')
    lines.append(f'  float y[{width}];')
    for e in range(width):
        operands = ', '.join(f's{i}' if spec['scalar'] else f'x{i}[{e}]' for i, spec in enumerate(inputs))
        lines.append(f'  y[{e}] = dtn_element({operands});')
    if params['out_f16']:
        words = ', '.join(f'(unsigned)dtn_f2h(y[{2 * e}]) | ((unsigned)dtn_f2h(y[{2 * e + 1}]) << 16)' for e in range(width // 2))
        lines.append(f'  static_cast<{vector_type}*>(out)[v] = make_{vector_type}({words});')
    else:
        for part in range(width // 4):
            lines.append(f'  static_cast<float4*>(out)[v * {width // 4} + {part}] = make_float4(y[{4 * part}], y[{4 * part + 1}], y[{4 * part + 2}], y[{4 * part + 3}]);')
    lines.append('}')
    pieces = n // width
    return {'source': PRELUDE + '\n'.join(lines) + '\n', 'entry': 'dtn_jit_kernel', 'grid': (pieces + 255) // 256, 'block': 256,
            'pointers': [f'in{i}' for i in range(len(inputs))] + ['out'], 'scalars': [('i64', pieces)]}


# ------------------------------------------------------------------------------------------------
# row programs (classify_rows._row_program / dtn_row_fused)
# ------------------------------------------------------------------------------------------------
ROW_PRELUDE = r'''
// One value per thread -> the row's value in every thread: xor tree inside a warp, then the warps' results through
// shared memory, added (or compared) in warp order.
template <bool MAX>
__device__ __forceinline__ float dtn_warp_combine(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, w) : v + w;
  }
  return v;
}
template <bool MAX, int WARPS>
__device__ __forceinline__ float dtn_combine(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, w) : v + w;
  }
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  v = scratch[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) v = MAX ? fmaxf(v, scratch[w]) : v + scratch[w];
  return v;
}
'''
ROW_THREADS = 128
ROW_MAX_VECTORS = 8           # 128-bit vectors of the row one thread keeps in registers
_ROW_REGISTERS = 12


def row_source(params: dict, buffers: dict) -> dict | None:
    """CUDA source of one kernel for a fused row program: 128 threads per row (a warp per row, four rows per CTA, for
    rows of at most 512 columns; 256 to 1024 threads for rows of 4096 to 32 768 columns), the row in registers (one
    global read), the reduction(s), the scalar stage and the elementwise stage written out operator by operator. Register numbering as in csrc/row_fused.cu: r0, r1 = the
    reduced values, r2 = the element, r3 + i = input i.

    Rows that get an elementwise stage are taken at any number of rows: with no program to decode and every load of
    a row requested before the first use, these kernels also stream faster than the library's (65 536 x 4096: RMS norm
    6.9 against 5.8 TB/s, softmax 6.9 against 6.0, L2 norm 6.8 against 6.2)."""
    rows, cols, inputs = params['rows'], params['cols'], params['inputs']
    # A row that is only reduced need not stay in registers: it is streamed by as many threads as give each at most
    # eight vectors (up to 1024: one row of 32 768 values is a CTA's work, and its loads should all be in flight).
    streamed = params['per_row'] and params['reduce'] != 'softmax'
    if streamed:
        threads = min(1024, max(ROW_THREADS, (cols // 4 + 7) // 8 + 31 & ~31))
    else:   # the row stays in registers, at most eight vectors a thread: 128 threads up to 4096 columns, 1024 up to 32 768
        threads = ROW_THREADS
        while threads < 1024 and cols > threads * 4 * ROW_MAX_VECTORS:
            threads *= 2
    lanes = 32 if (not streamed and cols <= 512) else threads   # threads that share a row
    if rows < 1 or rows > 0x7fffffff or cols < 4 or cols % 4 or (streamed and rows * cols > SMALL_ELEMENTS):
        return None
    if not streamed and cols > threads * 4 * ROW_MAX_VECTORS:
        return None
    if any(op not in _OPERATORS for op in params['ops']) or params['reduce'] not in ('sum', 'sumsq', 'max', 'softmax'):
        return None
    if buffers['x'][1] % 4 or (not params['per_row'] and buffers['out'][1] % 4):
        return None
    if any(buffers[f'in{i}'][1] % 4 for i, item in enumerate(inputs) if item['kind'] == 'columns'):
        return None
    reduce, n_scalar, out_reg = params['reduce'], params['n_scalar'], params['out_reg']
    program = list(zip(params['ops'], params['dst'], params['a'], params['b']))
    if max([out_reg, *params['dst'], *params['a'], *params['b'], 2 + len(inputs)]) >= _ROW_REGISTERS:
        return None
    is_max = reduce in ('max', 'softmax')
    identity = '-__int_as_float(0x7f800000)' if is_max else '0.0f'
    vectors = (cols // 4 + lanes - 1) // lanes
    rows_per_cta = threads // lanes
    pointer_inputs = [i for i, item in enumerate(inputs) if item['kind'] != 'immediate']
    fold = {'sum': '__fadd_rn({acc}, {v})', 'sumsq': 'fmaf({v}, {v}, {acc})', 'max': 'fmaxf({acc}, {v})', 'softmax': 'fmaxf({acc}, {v})'}[reduce]
    lines = []
    # elementwise stage as a function of the registers' values at its start
    lines.append('__device__ __forceinline__ float dtn_element(' + ', '.join(f'float a{k}' for k in range(_ROW_REGISTERS)) + ') {')
    lines.append('  float ' + ', '.join(f'e{k} = a{k}' for k in range(_ROW_REGISTERS)) + ';')
    for op, dst, a, b in program[n_scalar:]:
        lines.append(f'  e{dst} = {apply(op, f"e{a}", f"e{b}")};')
    lines += [f'  return e{out_reg};', '}']
    arguments = ['const float* __restrict__ x'] + [f'const float* __restrict__ p{i}' for i in pointer_inputs] + ['float* __restrict__ out', 'int cols', 'int rows']
    lines.append(f'extern "C" __global__ void __launch_bounds__({threads}) dtn_jit_kernel({", ".join(arguments)}) {{')
    if rows_per_cta > 1:   # a warp per row: the lanes combine by shuffles alone, so a warp without a row may leave
        lines += [f'  const int row = blockIdx.x * {rows_per_cta} + (threadIdx.x >> 5), tid = threadIdx.x & 31;',
                  '  if (row >= rows) return;']
    else:
        lines += [f'  __shared__ float scratch[2][{threads // 32}];',
                  '  const int row = blockIdx.x, tid = threadIdx.x;']
    lines.append('  const float4* xr = reinterpret_cast<const float4*>(x + (i64)row * cols);')
    for i, item in enumerate(inputs):
        if item['kind'] == 'scalar':
            lines.append(f'  const float c{i} = __ldg(p{i});')
        elif item['kind'] == 'immediate':
            lines.append(f'  const float c{i} = __int_as_float({_float_bits(item.get("value", 0.0))});')
    lines.append(f'  const float identity = {identity};')
    columns = [] if params['per_row'] else [i for i, item in enumerate(inputs) if item['kind'] == 'columns']
    # Per-column inputs are requested with the row, although the elementwise stage uses them: one trip to memory, not
    # two. Not in CTAs of 512 threads and more, where the registers they take cost a resident CTA: there they are read where they are used.
    early = columns if threads <= 256 else []
    lines.append(f'  float4 v[{vectors}];')
    for i in early:
        lines.append(f'  float4 q{i}[{vectors}];')
    lines.append('#pragma unroll')
    lines.append(f'  for (int u = 0; u < {vectors}; ++u) {{')
    lines.append(f'    const int j = u * {lanes} + tid;')
    lines.append('    v[u] = j * 4 < cols ? __ldg(xr + j) : make_float4(identity, identity, identity, identity);')
    for i in early:
        lines.append(f'    q{i}[u] = j * 4 < cols ? __ldg(reinterpret_cast<const float4*>(p{i}) + j) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);')
    lines.append('  }')
    lines.append('  float first = identity;')
    lines.append('#pragma unroll')
    lines.append(f'  for (int u = 0; u < {vectors}; ++u) {{')
    for c in _COMPONENTS:
        lines.append('    first = ' + fold.format(acc='first', v=f'v[u].{c}') + ';')
    lines.append('  }')
    combine = (lambda name, maximum, slot: f'  {name} = dtn_warp_combine<{"true" if maximum else "false"}>({name});') if rows_per_cta > 1 else \
              (lambda name, maximum, slot: f'  {name} = dtn_combine<{"true" if maximum else "false"}, {threads // 32}>({name}, scratch[{slot}]);')
    lines.append(combine('first', is_max, 0))
    lines.append('  float second = 0.0f;')
    if reduce == 'softmax':
        lines.append('#pragma unroll')
        lines.append(f'  for (int u = 0; u < {vectors}; ++u)')
        lines.append('    second += (dtn_exp(__fsub_rn(v[u].x, first)) + dtn_exp(__fsub_rn(v[u].y, first))) + '
                     '(dtn_exp(__fsub_rn(v[u].z, first)) + dtn_exp(__fsub_rn(v[u].w, first)));')
        lines.append(combine('second', False, 1))
    # scalar stage
    initial = {0: 'first', 1: 'second'}
    for i, item in enumerate(inputs):
        if item['kind'] != 'columns':
            initial[3 + i] = f'c{i}'
    lines.append('  float ' + ', '.join(f'r{k} = {initial.get(k, "0.0f")}' for k in range(_ROW_REGISTERS)) + ';')
    for op, dst, a, b in program[:n_scalar]:
        lines.append(f'  r{dst} = {apply(op, f"r{a}", f"r{b}")};')
    if params['per_row']:
        lines.append(f'  if (tid == 0) out[row] = r{out_reg};')
    else:
        lines.append('  float4* out_row = reinterpret_cast<float4*>(out + (i64)row * cols);')
        lines.append('#pragma unroll')
        lines.append(f'  for (int u = 0; u < {vectors}; ++u) {{')
        lines.append(f'    const int j = u * {lanes} + tid;')
        lines.append('    if (j * 4 >= cols) continue;')
        for i in columns:
            if i not in early:
                lines.append(f'    const float4 late{i} = __ldg(reinterpret_cast<const float4*>(p{i}) + j);')
        lines.append('    float4 result;')
        for c in _COMPONENTS:
            values = []
            for k in range(_ROW_REGISTERS):
                if k == 2:
                    values.append(f'v[u].{c}')
                elif k - 3 in columns:
                    values.append(f'q{k - 3}[u].{c}' if k - 3 in early else f'late{k - 3}.{c}')
                else:
                    values.append(f'r{k}')
            lines.append(f'    result.{c} = dtn_element({", ".join(values)});')
        lines.append('    out_row[j] = result;')
        lines.append('  }')
    lines.append('}')
    return {'source': PRELUDE + ROW_PRELUDE + '\n'.join(lines) + '\n', 'entry': 'dtn_jit_kernel', 'grid': (rows + rows_per_cta - 1) // rows_per_cta, 'block': threads,
            'pointers': ['x'] + [f'in{i}' for i in pointer_inputs] + ['out'], 'scalars': [('i32', cols), ('i32', rows)]}


def _float_bits(value: float) -> str:
    import struct
    return hex(struct.unpack('<I', struct.pack('<f', float(value)))[0])


# ------------------------------------------------------------------------------------------------
# small attention (classify._classify_attention / dtn_attention_f32)
# ------------------------------------------------------------------------------------------------
ATTENTION_MAX_ROWS = 1024


def attention_source(params: dict, buffers: dict) -> dict | None:
    """CUDA source of the reference-layout attention (q[rows, depth], kt[depth, keys], v[keys, cols]) for one shape:
    a warp per query row and a CTA per warp, every extent a constant, so that the loads of a row's keys and values are
    all independent and in flight together instead of staged through shared memory behind two barriers. For a few
    hundred rows of at most 256 keys, where the launch is one warp's chain. The arithmetic and its order are those of
    csrc/attention_f32.cu's one-stage case (scores by sequential fma over the depth, weights ex2.approx((s - max) *
    log2 e), mass by the same butterfly, weighted sum by sequential fma over the keys, one approximate reciprocal),
    so the bits are the library kernel's."""
    rows, keys, depth, cols = params['rows'], params['keys'], params['depth'], params['cols']
    if not (1 <= rows <= ATTENTION_MAX_ROWS and 32 <= keys <= 256 and keys % 32 == 0 and 1 <= depth <= 128 and cols in (32, 64)):
        return None
    rounds, groups = keys // 32, cols // 32
    scale = f'__int_as_float({_float_bits(params["scale"])})'
    # The values are not needed before the weights exist: where they fit, they are requested into shared memory as
    # asynchronous copies before the first score is computed and arrive behind the scores and the softmax.
    staged = keys * cols * 4 <= 48 * 1024 and buffers['v'][1] % 4 == 0
    request = f'''
  __shared__ __align__(16) float vs[KEYS * COLS];
#pragma unroll
  for (int i = 0; i < KEYS * COLS / 128; ++i)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(vs + 4 * (lane + 32 * i))),
                 "l"(v + 4 * (lane + 32 * i)) : "memory");
  asm volatile("cp.async.commit_group;" ::: "memory");''' if staged else ''
    arrive = '''
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();''' if staged else ''
    value = 'vs[k * COLS + lane + 32 * c]' if staged else '__ldg(v + k * COLS + lane + 32 * c)'
    source = PRELUDE + f'''
extern "C" __global__ void __launch_bounds__(32) dtn_jit_kernel(const float* __restrict__ q, const float* __restrict__ kt,
                                                                const float* __restrict__ v, float* __restrict__ out) {{
  constexpr int KEYS = {keys}, DEPTH = {depth}, COLS = {cols}, ROUNDS = {rounds}, GROUPS = {groups};
  const int row = blockIdx.x, lane = threadIdx.x;
  const float* qr = q + row * DEPTH;{request}
  float s[ROUNDS];
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) s[r] = 0.0f;
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {{
    const float qv = __ldg(qr + d);
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) s[r] = fmaf(qv, __ldg(kt + d * KEYS + lane + 32 * r), s[r]);
  }}
  float peak = -__int_as_float(0x7f800000);
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {{
    s[r] = __fmul_rn(s[r], {scale});
    peak = fmaxf(peak, s[r]);
  }}
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  float mass = 0.0f;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {{
    s[r] = dtn_ex2(__fmul_rn(__fsub_rn(s[r], peak), 1.4426950408889634f));
    mass = __fadd_rn(mass, s[r]);
  }}
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mass = __fadd_rn(mass, __shfl_xor_sync(0xffffffffu, mass, o));
  float acc[GROUPS];
#pragma unroll
  for (int c = 0; c < GROUPS; ++c) acc[c] = 0.0f;{arrive}
#pragma unroll
  for (int k = 0; k < KEYS; ++k) {{
    const float w = __shfl_sync(0xffffffffu, s[k / 32], k % 32);
#pragma unroll
    for (int c = 0; c < GROUPS; ++c) acc[c] = fmaf(w, {value}, acc[c]);
  }}
  const float inverse = dtn_rcp(mass);
#pragma unroll
  for (int c = 0; c < GROUPS; ++c) out[row * COLS + lane + 32 * c] = __fmul_rn(acc[c], inverse);
}}
'''
    return {'source': source, 'entry': 'dtn_jit_kernel', 'grid': rows, 'block': 32, 'pointers': ['q', 'kt', 'v', 'out'], 'scalars': []}


def specialized_source(plan: Any) -> dict | None:
    """The per-program kernel of a plan (source, entry, launch geometry, argument roles), or None."""
    if not enabled():
        return None
    try:
        if plan.kind == 'elementwise_program':
            return elementwise_source(plan.params, plan.buffers)
        if plan.kind == 'row_fused':
            return row_source(plan.params, plan.buffers)
        if plan.kind == 'attention':
            return attention_source(plan.params, plan.buffers)
        if plan.kind == 'row_reduce' and plan.params['op'] in ('sum', 'max', 'sumsq'):   # a row program with no operators
            reduction = {'rows': plan.params['rows'], 'cols': plan.params['cols'], 'reduce': plan.params['op'], 'inputs': [], 'n_scalar': 0,
                         'out_reg': 0, 'ops': [], 'dst': [], 'a': [], 'b': [], 'per_row': True}
            return row_source(reduction, plan.buffers)
    except (KeyError, ValueError, TypeError):
        return None
    return None


# ------------------------------------------------------------------------------------------------
# NVRTC and the driver API
# ------------------------------------------------------------------------------------------------
_lock = threading.RLock()   # compile_source is entered from kernel_for, which holds it
_cubins: dict[str, bytes | None] = {}
_modules: dict[tuple[int, str], Any] = {}
_libraries: dict[str, Any] = {}


def _library(name: str):
    if name not in _libraries:
        try:
            _libraries[name] = ct.CDLL(name)
        except OSError:
            _libraries[name] = None
    return _libraries[name]


def _nvrtc():
    """NVRTC from the loader's path, the CUDA toolkit's usual place, or the copy the PyTorch wheels depend on."""
    candidates = ['libnvrtc.so.12', 'libnvrtc.so', '/usr/local/cuda/lib64/libnvrtc.so.12']
    try:
        import importlib.util
        found = importlib.util.find_spec('nvidia.cuda_nvrtc')
        candidates += [os.path.join(place, 'lib', 'libnvrtc.so.12') for place in (found.submodule_search_locations if found else [])]
    except (ImportError, ValueError):
        pass
    for name in candidates:
        library = _library(name)
        if library is not None:
            return library
    return None


def compile_source(source: str, arch: str = 'sm_100a') -> bytes | None:
    """NVRTC: CUDA C++ -> cubin for `arch`. None when NVRTC is not there or rejects the source (the caller then runs
    the library's kernel). No contraction into fma: a program computes what its operators compute one by one."""
    key = hashlib.sha256((arch + '\0' + source).encode()).hexdigest()
    with _lock:
        if key in _cubins:
            return _cubins[key]
        cubin = _stored_cubin(key)
        nvrtc = _nvrtc() if cubin is None else None
        if nvrtc is not None:
            program = ct.c_void_p()
            if nvrtc.nvrtcCreateProgram(ct.byref(program), source.encode(), b'dtn_jit.cu', 0, None, None) == 0:
                options = [f'--gpu-architecture={arch}'.encode(), b'--std=c++17', b'--fmad=false']
                array = (ct.c_char_p * len(options))(*options)
                if nvrtc.nvrtcCompileProgram(program, len(options), array) == 0:
                    size = ct.c_size_t()
                    if nvrtc.nvrtcGetCUBINSize(program, ct.byref(size)) == 0 and size.value:
                        buffer = ct.create_string_buffer(size.value)
                        if nvrtc.nvrtcGetCUBIN(program, buffer) == 0:
                            cubin = buffer.raw
                nvrtc.nvrtcDestroyProgram(ct.byref(program))
            if cubin is not None:
                _store_cubin(key, cubin)
        _cubins[key] = cubin
        return cubin


def _cubin_path(key: str) -> str | None:
    """Where a compiled kernel is kept between processes: beside the compile records, under DEUTERON_CACHE
    (compiler/build.py:99-104 keeps the reference's PTX there)."""
    root = os.environ.get('DEUTERON_CACHE')
    return os.path.join(root, f'jit-{key}.cubin') if root else None


def _stored_cubin(key: str) -> bytes | None:
    path = _cubin_path(key)
    try:
        if path is not None:
            with open(path, 'rb') as handle:
                data = handle.read()
            if data[:4] == b'\x7fELF':   # anything else is not a record of ours: compile again
                return data
    except OSError:
        pass
    return None


def _store_cubin(key: str, cubin: bytes) -> None:
    path = _cubin_path(key)
    if path is None:
        return
    try:   # written under another name and renamed, so that a reader never sees half a file
        os.makedirs(os.path.dirname(path), exist_ok=True)
        temporary = f'{path}.{os.getpid()}.{threading.get_ident()}.tmp'
        with open(temporary, 'wb') as handle:
            handle.write(cubin)
        os.replace(temporary, path)
    except OSError:
        pass


class Kernel:
    """A compiled per-program kernel loaded into the current CUDA context."""

    def __init__(self, cubin: bytes, entry: str) -> None:
        driver = _library('libcuda.so.1')
        if driver is None:
            raise OSError('libcuda.so.1 is not available')
        self._driver = driver
        self._module, self._function = ct.c_void_p(), ct.c_void_p()
        if driver.cuModuleLoadData(ct.byref(self._module), cubin) != 0:
            raise OSError('cuModuleLoadData failed')
        if driver.cuModuleGetFunction(ct.byref(self._function), self._module, entry.encode()) != 0:
            raise OSError('cuModuleGetFunction failed')

    def attributes(self) -> tuple[int, int]:
        """(registers per thread, static shared memory in bytes) of the loaded kernel."""
        registers, shared = ct.c_int(0), ct.c_int(0)
        self._driver.cuFuncGetAttribute(ct.byref(registers), 4, self._function)    # CU_FUNC_ATTRIBUTE_NUM_REGS
        self._driver.cuFuncGetAttribute(ct.byref(shared), 1, self._function)       # CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES
        return registers.value, shared.value

    def launch(self, grid: int, block: int, values: list, stream: int) -> None:
        params = (ct.c_void_p * len(values))(*[ct.cast(ct.byref(v), ct.c_void_p) for v in values])
        status = self._driver.cuLaunchKernel(self._function, grid, 1, 1, block, 1, 1, 0, ct.c_void_p(stream), params, None)
        if status != 0:
            raise OSError(f'cuLaunchKernel failed with CUresult {status}')


def memset_zero(address: int, nbytes: int, stream: int) -> None:
    """cuMemsetD8Async of zeros on `stream` (a memset node when the stream is being captured)."""
    driver = _library('libcuda.so.1')
    if driver is None:
        raise OSError('libcuda.so.1 is not available')
    status = driver.cuMemsetD8Async(ct.c_uint64(address), ct.c_ubyte(0), ct.c_size_t(nbytes), ct.c_void_p(stream))
    if status != 0:
        raise OSError(f'cuMemsetD8Async failed with CUresult {status}')


def kernel_for(spec: dict, device: int, arch: str = 'sm_100a') -> Kernel | None:
    """The loaded kernel of a specialised source on `device` (whose context must be current), or None."""
    key = (device, hashlib.sha256(spec['source'].encode()).hexdigest())
    with _lock:
        if key in _modules:
            return _modules[key]
        cubin = compile_source(spec['source'], arch)
        kernel = None
        if cubin is not None:
            try:
                kernel = Kernel(cubin, spec['entry'])
            except OSError:
                kernel = None
        _modules[key] = kernel
        return kernel


def launch(spec: dict, kernel: Kernel, pointer_of: Any, stream: int) -> None:
    """One launch: `pointer_of(role)` gives the device address of a buffer role of the plan."""
    values: list = [ct.c_uint64(pointer_of(role)) for role in spec['pointers']]
    for kind, value in spec['scalars']:
        values.append({'i64': ct.c_longlong, 'i32': ct.c_int, 'f32': ct.c_float}[kind](value))
    kernel.launch(spec['grid'], spec['block'], values, stream)
