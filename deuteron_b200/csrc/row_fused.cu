// Fused row kernels: one reduction over every row of x[rows, cols], a scalar stage on the reduced
// value, and an elementwise stage over the same row -- row softmax, RMS norm, L2 norm and mean in
// one launch and (for rows of up to 8192 values) one trip through memory.
//
// The reference reaches the same fusion by rewriting the scheduled IR: load forwarding keeps the row
// in registers between the reduction loop and the consumer loop (compiler/passes/regforward.py:150-269)
// and the softmax normaliser replaces the online (max, sum) pair by a max pass followed by a sum of
// exponentials over cached values (compiler/passes/hybrid_normalizer.py:139-183). Here a group of
// 8 to 256 threads owns a row: the row is read once with 128-bit loads into eight vectors per thread,
// reduced by a butterfly shuffle (plus one shared-memory round when the group spans warps), and
// written once; longer rows take the same code chunk by chunk and re-read the row (mostly from L2).
//
// The two stages arrive as one short register program: instructions [0, n_scalar) run once per row
// on the reduced value and the one-element inputs, the rest run per element. Register 0 holds the
// reduced value, register 1 the sum of exp(x - max) for the softmax reduction, register 2 the row
// element, registers 3.. the extra inputs in order; the others are temporaries.
//
// Chain form. In the workloads this kernel exists for, the elementwise stage is a chain: every
// instruction combines the running value with a per-row scalar, a per-column input, the row element
// or itself (softmax: x - max, exp, * 1/sum; RMS norm: x * scale, * w). A chain needs no register
// file per element: the operator is decoded once per row and step, outside the loop over the
// thread's 32 cached elements, so the cost per element is the arithmetic alone. Programs that are
// not chains run on a per-element interpreter (correct for any program, several times slower).
#include <math.h>

#include "dtn_common.cuh"
#include "program.cuh"

namespace dtn {

constexpr int kRowRegs = 12;
constexpr int kRowMaxInstr = 32;
constexpr int kRowMaxInputs = 5;
constexpr int kRowCacheVecs = 8;   // 128-bit vectors of the row one thread keeps in registers
constexpr int kChainMax = 16;
enum { CHAIN_SCALAR = 0, CHAIN_COLUMNS = 1, CHAIN_ELEMENT = 2, CHAIN_SELF = 3 };

struct RowProgram {
  int reduce, n_inputs, n_scalar, n_instr, out_reg;
  const float* input[kRowMaxInputs];
  float immediate[kRowMaxInputs];
  unsigned char kind[kRowMaxInputs];
  unsigned char op[kRowMaxInstr], dst[kRowMaxInstr], a[kRowMaxInstr], b[kRowMaxInstr];
};

// The scalar stage's registers: a plain array indexed at run time. It lives in local memory (L1-resident, a few dozen
// bytes per thread); one load per operand is far cheaper here than the twelve-way compare chains a register-resident
// file needs, and the scalar stage runs once per row, not per element.
struct ScalarFile {
  float r[kRowRegs];
};

struct RowChain {
  int n;
  int cached_exp;   // 1: the chain opens with (x - max), exp and the softmax sum pass leaves exactly those values in the row cache
  unsigned char op[kChainMax], kind[kChainMax], index[kChainMax], swap[kChainMax];   // index: register (scalar) or input (columns)
};

// Combines one value per thread over the TPR threads that share a row (TPR lanes of a warp, or all warps of the CTA).
// Across warps: every warp leaves its partial in one of two scratch rows (alternating from call to call, so one barrier
// per call is enough: a row is rewritten only after the barrier of the call in between) and every thread folds them all.
template <int TPR, bool MAX>
__device__ __forceinline__ float row_combine(float v, float* scratch, int& parity) {
  constexpr int kLanes = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, w) : v + w;
  }
  if constexpr (TPR > 32) {
    float* mine = scratch + parity * 8;
    parity ^= 1;
    if ((threadIdx.x & 31) == 0) mine[threadIdx.x >> 5] = v;
    __syncthreads();
    v = mine[0];
#pragma unroll
    for (int w = 1; w < TPR / 32; ++w) v = MAX ? fmaxf(v, mine[w]) : v + mine[w];
  }
  return v;
}

__device__ __forceinline__ float fold_first(int reduce, float acc, float v) {
  if (reduce == DTN_REDUCE_SUM) return acc + v;
  if (reduce == DTN_REDUCE_SUMSQ) return fmaf(v, v, acc);
  return fmaxf(acc, v);   // max and softmax
}

// The one-element inputs and the literals of a program: the same for every row, so they are read once per thread,
// before the first row is touched (their latency hides behind the loads of the row).
struct RowConstants {
  float v[kRowMaxInputs];
};
__device__ __forceinline__ RowConstants row_constants(const RowProgram& prog) {
  RowConstants c;
#pragma unroll
  for (int i = 0; i < kRowMaxInputs; ++i) {
    c.v[i] = 0.0f;
    if (i < prog.n_inputs && prog.kind[i] != DTN_ROW_INPUT_COLUMNS)
      c.v[i] = prog.kind[i] == DTN_ROW_INPUT_IMMEDIATE ? prog.immediate[i] : __ldg(prog.input[i]);
  }
  return c;
}

// Scalar stage: the reduced values and the constants go into registers, then instructions [0, n_scalar) run.
// Every thread of the row computes the same values.
__device__ __forceinline__ void scalar_stage(const RowProgram& prog, const RowConstants& constants, float first, float second,
                                             ScalarFile& scalars) {
#pragma unroll
  for (int k = 0; k < kRowRegs; ++k) scalars.r[k] = 0.0f;
  scalars.r[0] = first;
  scalars.r[1] = second;
#pragma unroll
  for (int i = 0; i < kRowMaxInputs; ++i) scalars.r[3 + i] = constants.v[i];
  for (int n = 0; n < prog.n_scalar; ++n) scalars.r[prog.dst[n]] = prog_apply(prog.op[n], scalars.r[prog.a[n]], scalars.r[prog.b[n]]);
}

template <int OP>
__device__ __forceinline__ float chain_op(float a, float o, bool swap) {
  if constexpr (OP == DTN_EW_ADD) return __fadd_rn(a, o);
  if constexpr (OP == DTN_EW_SUB) return swap ? __fsub_rn(o, a) : __fsub_rn(a, o);
  if constexpr (OP == DTN_EW_MUL) return __fmul_rn(a, o);
  if constexpr (OP == DTN_EW_DIV) return swap ? __fdividef(o, a) : __fdividef(a, o);
  if constexpr (OP == DTN_EW_MAX) return fmaxf(a, o);
  if constexpr (OP == DTN_EW_MIN) return fminf(a, o);
  return prog_apply(OP, a, a);   // unary operators (constant-folded switch)
}

// Unit u of a thread's chunk covers four consecutive columns of one 128-bit vector (VEC) or four
// columns TPR apart (scalar accesses). Columns are 32-bit: a buffer holds fewer than 2^31 elements.
template <int TPR, bool VEC>
__device__ __forceinline__ int chain_column(int chunk_base, int rank, int u, int lane) {
  if constexpr (VEC) return chunk_base + (rank + u * TPR) * 4 + lane;
  return chunk_base + rank + (u * 4 + lane) * TPR;
}

// One step of the chain over the thread's 32 cached elements. OP and KIND are compile-time: the two uniform
// switches in chain_run pick the instantiation once per row and step.
template <int OP, int KIND, int TPR, bool VEC, int NV>
__device__ __forceinline__ void chain_step(float4 (&acc)[NV], const float4 (&kept)[NV], float scalar,
                                           const float* __restrict__ columns, bool swap, int chunk_base, int rank, int cols) {
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    float o[4];
    if constexpr (KIND == CHAIN_SCALAR) {
      o[0] = o[1] = o[2] = o[3] = scalar;
    } else if constexpr (KIND == CHAIN_ELEMENT) {
      o[0] = kept[u].x; o[1] = kept[u].y; o[2] = kept[u].z; o[3] = kept[u].w;
    } else if constexpr (KIND == CHAIN_SELF) {
      o[0] = acc[u].x; o[1] = acc[u].y; o[2] = acc[u].z; o[3] = acc[u].w;
    } else if constexpr (VEC) {
      const int col = chain_column<TPR, VEC>(chunk_base, rank, u, 0);
      const float4 q = col < cols ? __ldg(reinterpret_cast<const float4*>(columns + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
      o[0] = q.x; o[1] = q.y; o[2] = q.z; o[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = chain_column<TPR, VEC>(chunk_base, rank, u, e);
        o[e] = col < cols ? __ldg(columns + col) : 0.0f;
      }
    }
    acc[u].x = chain_op<OP>(acc[u].x, o[0], swap);
    acc[u].y = chain_op<OP>(acc[u].y, o[1], swap);
    acc[u].z = chain_op<OP>(acc[u].z, o[2], swap);
    acc[u].w = chain_op<OP>(acc[u].w, o[3], swap);
  }
}

template <int OP, int TPR, bool VEC, int NV>
__device__ __forceinline__ void chain_binary(float4 (&acc)[NV], const float4 (&kept)[NV], int kind, float scalar,
                                             const float* __restrict__ columns, bool swap, int chunk_base, int rank, int cols) {
  switch (kind) {
    case CHAIN_SCALAR: chain_step<OP, CHAIN_SCALAR, TPR, VEC>(acc, kept, scalar, columns, swap, chunk_base, rank, cols); break;
    case CHAIN_COLUMNS: chain_step<OP, CHAIN_COLUMNS, TPR, VEC>(acc, kept, scalar, columns, swap, chunk_base, rank, cols); break;
    case CHAIN_ELEMENT: chain_step<OP, CHAIN_ELEMENT, TPR, VEC>(acc, kept, scalar, columns, swap, chunk_base, rank, cols); break;
    default: chain_step<OP, CHAIN_SELF, TPR, VEC>(acc, kept, scalar, columns, swap, chunk_base, rank, cols); break;
  }
}

template <int TPR, bool VEC, int NV>
__device__ __forceinline__ void chain_load(float4 (&cache)[NV], const float* __restrict__ xr, int chunk_base, int rank,
                                           int cols, float fill) {
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    if constexpr (VEC) {
      const int col = chain_column<TPR, VEC>(chunk_base, rank, u, 0);
      cache[u] = col < cols ? ld_stream_f4(reinterpret_cast<const float4*>(xr + col)) : make_float4(fill, fill, fill, fill);
    } else {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = chain_column<TPR, VEC>(chunk_base, rank, u, e);
        v[e] = col < cols ? __ldg(xr + col) : fill;
      }
      cache[u] = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

// Folds the thread's cached elements into four partial reductions; the reduction operator is a uniform branch
// taken once per chunk, not per element.
template <int NV>
__device__ __forceinline__ void chain_fold(int reduce, const float4 (&cache)[NV], float (&part)[4]) {
  if (reduce == DTN_REDUCE_SUM) {
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      part[0] += cache[u].x; part[1] += cache[u].y; part[2] += cache[u].z; part[3] += cache[u].w;
    }
  } else if (reduce == DTN_REDUCE_SUMSQ) {
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      part[0] = fmaf(cache[u].x, cache[u].x, part[0]); part[1] = fmaf(cache[u].y, cache[u].y, part[1]);
      part[2] = fmaf(cache[u].z, cache[u].z, part[2]); part[3] = fmaf(cache[u].w, cache[u].w, part[3]);
    }
  } else {
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      part[0] = fmaxf(part[0], cache[u].x); part[1] = fmaxf(part[1], cache[u].y);
      part[2] = fmaxf(part[2], cache[u].z); part[3] = fmaxf(part[3], cache[u].w);
    }
  }
}

template <int TPR, bool VEC, int NV>
__device__ __forceinline__ void chain_run(const RowProgram& prog, const RowChain& chain, const ScalarFile& scalars,
                                          float4 (&acc)[NV], const float4 (&kept)[NV], int chunk_base, int rank,
                                          int cols, int first_step = 0) {
  for (int s = first_step; s < chain.n; ++s) {
    const int kind = chain.kind[s];
    const bool swap = chain.swap[s] != 0;
    const float scalar = kind == CHAIN_SCALAR ? scalars.r[chain.index[s]] : 0.0f;
    const float* columns = nullptr;
    if (kind == CHAIN_COLUMNS) columns = prog.input[chain.index[s]];
#define DTN_CHAIN_BINARY(OP) \
  case OP: chain_binary<OP, TPR, VEC>(acc, kept, kind, scalar, columns, swap, chunk_base, rank, cols); break;
#define DTN_CHAIN_UNARY(OP) \
  case OP: chain_step<OP, CHAIN_SELF, TPR, VEC>(acc, kept, 0.0f, nullptr, false, chunk_base, rank, cols); break;
    switch (chain.op[s]) {
      DTN_CHAIN_BINARY(DTN_EW_ADD) DTN_CHAIN_BINARY(DTN_EW_SUB) DTN_CHAIN_BINARY(DTN_EW_MUL) DTN_CHAIN_BINARY(DTN_EW_DIV)
      DTN_CHAIN_BINARY(DTN_EW_MAX) DTN_CHAIN_BINARY(DTN_EW_MIN) DTN_CHAIN_UNARY(DTN_EW_RELU) DTN_CHAIN_UNARY(DTN_EW_EXP)
      DTN_CHAIN_UNARY(DTN_EW_SQRT) DTN_CHAIN_UNARY(DTN_EW_RSQRT) DTN_CHAIN_UNARY(DTN_EW_RCP) DTN_CHAIN_UNARY(DTN_EW_NEG)
      DTN_CHAIN_UNARY(DTN_EW_ABS)
      default: break;   // copy
    }
#undef DTN_CHAIN_BINARY
#undef DTN_CHAIN_UNARY
  }
}

// TPR threads per row (8, 16, 32 lanes of a warp, or a CTA of 64, 128 or 256 threads). KEEPX: a later step of the
// chain reads the row element again, so the running values need registers of their own. NV: 128-bit vectors of the row
// a thread keeps (1, 2, 4 or 8): short rows get the instantiation that holds them and no more, which is an eighth of
// the code of the 8-vector form (a small launch spends most of its time fetching instructions otherwise).
template <int TPR, bool VEC, bool KEEPX, int NV>
__global__ void __launch_bounds__(TPR <= 32 ? 128 : TPR, (KEEPX ? 512 : 640) / (TPR <= 32 ? 128 : TPR))
row_chain_kernel(const RowProgram prog, const RowChain chain, const float* __restrict__ x, float* __restrict__ out, int64_t rows,
                 int cols, int64_t ldx, int64_t ldo) {
  constexpr int kThreads = TPR <= 32 ? 128 : TPR;
  constexpr int RPB = kThreads / TPR;                                // rows per CTA
  constexpr int kChunkCols = TPR * NV * 4;   // columns one pass of the group covers
  __shared__ float scratch[16];
  int parity = 0;
  const int rank = threadIdx.x % TPR, sub = threadIdx.x / TPR;
  const int reduce = prog.reduce;
  const bool is_max = reduce == DTN_REDUCE_MAX || reduce == DTN_REDUCE_SOFTMAX;
  const bool one_chunk = cols <= kChunkCols;
  const float identity = is_max ? -INFINITY : 0.0f;
  const RowConstants constants = row_constants(prog);
  if constexpr (VEC) {
    // per-column inputs are read only in the elementwise stage, after the reduction: start fetching this thread's
    // part of them now so that the first row does not wait for them
    for (int s = 0; s < chain.n; ++s) {
      if (chain.kind[s] != CHAIN_COLUMNS) continue;
      const float* columns = prog.input[chain.index[s]];
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        const int col = chain_column<TPR, VEC>(0, rank, u, 0);
        if (col < cols) asm volatile("prefetch.global.L1 [%0];" ::"l"(columns + col));
      }
    }
  }
  for (int64_t row0 = (int64_t)blockIdx.x * RPB; row0 < rows; row0 += (int64_t)gridDim.x * RPB) {
    int64_t row = row0 + sub;
    const bool live = row < rows;   // uniform over the lanes that share a row; a CTA-wide group always has a live row
    if (!live) row = rows - 1;      // idle groups of the last CTA repeat the last row and store nothing
    const float* xr = x + row * ldx;
    float4 cache[NV];
    float part[4] = {identity, identity, identity, identity};
    if (one_chunk) {
      chain_load<TPR, VEC>(cache, xr, 0, rank, cols, identity);
      chain_fold(reduce, cache, part);
    } else {
      // longer rows: the reduction streams the row chunk by chunk, eight loads in flight per thread
      for (int chunk_base = 0; chunk_base < cols; chunk_base += kChunkCols) {
        chain_load<TPR, VEC>(cache, xr, chunk_base, rank, cols, identity);
        chain_fold(reduce, cache, part);
      }
    }
    float first = is_max ? fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) : (part[0] + part[1]) + (part[2] + part[3]);
    first = is_max ? row_combine<TPR, true>(first, scratch, parity) : row_combine<TPR, false>(first, scratch, parity);

    float second = 0.0f;
    if (reduce == DTN_REDUCE_SOFTMAX) {
      if (one_chunk) {   // padding holds -inf, whose exponential is 0
        // the exponentials stay in the row cache: when the elementwise stage opens with the same (x - max), exp
        // (chain.cached_exp) it continues from them instead of computing each a second time
#pragma unroll
        for (int u = 0; u < NV; ++u) {
          const float4 e = make_float4(exp_ref(__fsub_rn(cache[u].x, first)), exp_ref(__fsub_rn(cache[u].y, first)),
                                       exp_ref(__fsub_rn(cache[u].z, first)), exp_ref(__fsub_rn(cache[u].w, first)));
          second += (e.x + e.y) + (e.z + e.w);
          if constexpr (!KEEPX) cache[u] = e;
        }
      } else {
        for (int chunk_base = 0; chunk_base < cols; chunk_base += kChunkCols) {
          chain_load<TPR, VEC>(cache, xr, chunk_base, rank, cols, -INFINITY);
#pragma unroll
          for (int u = 0; u < NV; ++u)
            second += (exp_ref(cache[u].x - first) + exp_ref(cache[u].y - first)) + (exp_ref(cache[u].z - first) + exp_ref(cache[u].w - first));
        }
      }
      second = row_combine<TPR, false>(second, scratch, parity);
    }

    ScalarFile scalars;
    scalar_stage(prog, constants, first, second, scalars);
    if (ldo == 0) {
      if (live && rank == 0) {
        out[row] = scalars.r[prog.out_reg];
      }
      continue;
    }
    if (!live) continue;
    float* out_row = out + row * ldo;
    for (int chunk_base = 0; chunk_base < cols; chunk_base += kChunkCols) {
      if (!one_chunk) chain_load<TPR, VEC>(cache, xr, chunk_base, rank, cols, 0.0f);
      if constexpr (KEEPX) {
        float4 acc[NV];
#pragma unroll
        for (int u = 0; u < NV; ++u) acc[u] = cache[u];
        chain_run<TPR, VEC>(prog, chain, scalars, acc, cache, chunk_base, rank, cols);
#pragma unroll
        for (int u = 0; u < NV; ++u) cache[u] = acc[u];
      } else if (reduce == DTN_REDUCE_SOFTMAX && one_chunk) {
        // the cache holds exp(x - max) already; a chain that does not open with those two steps starts from x again
        if (!chain.cached_exp) chain_load<TPR, VEC>(cache, xr, 0, rank, cols, 0.0f);
        chain_run<TPR, VEC>(prog, chain, scalars, cache, cache, chunk_base, rank, cols, chain.cached_exp ? 2 : 0);
      } else {
        chain_run<TPR, VEC>(prog, chain, scalars, cache, cache, chunk_base, rank, cols);
      }
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        if constexpr (VEC) {
          const int col = chain_column<TPR, VEC>(chunk_base, rank, u, 0);
          if (col < cols) st_stream_f4(reinterpret_cast<float4*>(out_row + col), cache[u]);
        } else {
          const float v[4] = {cache[u].x, cache[u].y, cache[u].z, cache[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = chain_column<TPR, VEC>(chunk_base, rank, u, e);
            if (col < cols) out_row[col] = v[e];
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Interpreter for programs whose elementwise stage is not a chain: a CTA per row, the row streamed
// three times (reduction, softmax sum, elementwise stage), every element run through the register
// program two lanes at a time.
// ---------------------------------------------------------------------------------------
template <int W>
__device__ __forceinline__ void element_compute(const RowProgram& prog, const ScalarFile& scalars, const float (&xv)[W],
                                                int64_t col, float (&result)[W]) {
  RegFile<kRowRegs, W> regs;
#pragma unroll
  for (int k = 0; k < kRowRegs; ++k)
#pragma unroll
    for (int e = 0; e < W; ++e) regs.r[k][e] = scalars.r[k];
#pragma unroll
  for (int e = 0; e < W; ++e) regs.r[2][e] = xv[e];
#pragma unroll
  for (int i = 0; i < kRowMaxInputs; ++i) {
    if (i < prog.n_inputs && prog.kind[i] == DTN_ROW_INPUT_COLUMNS) {
      float v[W];
      if constexpr (W == 2) {
        const float2 q = __ldg(reinterpret_cast<const float2*>(prog.input[i] + col));
        v[0] = q.x; v[1] = q.y;
      } else {
        v[0] = __ldg(prog.input[i] + col);
      }
      regs.put(3 + i, v);
    }
  }
  for (int n = prog.n_scalar; n < prog.n_instr; ++n) {
    float a[W], b[W], d[W];
    regs.get(prog.a[n], a);
    regs.get(prog.b[n], b);
    const int op = prog.op[n];
#pragma unroll
    for (int e = 0; e < W; ++e) d[e] = prog_apply(op, a[e], b[e]);
    regs.put(prog.dst[n], d);
  }
  regs.get(prog.out_reg, result);
}

template <bool VEC>
__global__ void __launch_bounds__(256, 2)
row_interpreter_kernel(const RowProgram prog, const float* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t cols,
                       int64_t ldx, int64_t ldo) {
  constexpr int TPR = 256;
  __shared__ float scratch[16];
  int parity = 0;
  const int rank = threadIdx.x;
  const int reduce = prog.reduce;
  const bool is_max = reduce == DTN_REDUCE_MAX || reduce == DTN_REDUCE_SOFTMAX;
  const int64_t units = VEC ? (cols >> 2) : cols;
  const RowConstants constants = row_constants(prog);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * ldx;
    float first = is_max ? -INFINITY : 0.0f;
    for (int64_t j = rank; j < units; j += TPR) {
      if constexpr (VEC) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + j);
        first = fold_first(reduce, fold_first(reduce, fold_first(reduce, fold_first(reduce, first, v.x), v.y), v.z), v.w);
      } else {
        first = fold_first(reduce, first, __ldg(xr + j));
      }
    }
    first = is_max ? row_combine<TPR, true>(first, scratch, parity) : row_combine<TPR, false>(first, scratch, parity);
    float second = 0.0f;
    if (reduce == DTN_REDUCE_SOFTMAX) {
      for (int64_t j = rank; j < units; j += TPR) {
        if constexpr (VEC) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + j);
          second += (exp_ref(v.x - first) + exp_ref(v.y - first)) + (exp_ref(v.z - first) + exp_ref(v.w - first));
        } else {
          second += exp_ref(__ldg(xr + j) - first);
        }
      }
      second = row_combine<TPR, false>(second, scratch, parity);
    }
    ScalarFile scalars;
    scalar_stage(prog, constants, first, second, scalars);
    if (ldo == 0) {
      if (rank == 0) {
        out[row] = scalars.r[prog.out_reg];
      }
      continue;
    }
    float* out_row = out + row * ldo;
    for (int64_t j = rank; j < units; j += TPR) {
      if constexpr (VEC) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + j);
        const float lo[2] = {v.x, v.y}, hi[2] = {v.z, v.w};
        float r0[2], r1[2];
        element_compute<2>(prog, scalars, lo, j * 4, r0);
        element_compute<2>(prog, scalars, hi, j * 4 + 2, r1);
        st_stream_f4(reinterpret_cast<float4*>(out_row) + j, make_float4(r0[0], r0[1], r1[0], r1[1]));
      } else {
        const float xv[1] = {__ldg(xr + j)};
        float result[1];
        element_compute<1>(prog, scalars, xv, j, result);
        out_row[j] = result[0];
      }
    }
  }
}

// Chain form of the elementwise stage of `prog`, if it has one. Register 2 (the element) starts as the running value;
// every instruction must read the running value and write the next one, and its other operand must be a value the
// elementwise stage has not overwritten. *keep_x: a step after the first reads the row element.
static bool row_chain_of(const RowProgram& prog, RowChain* chain, bool* keep_x, bool per_row) {
  chain->n = 0;
  chain->cached_exp = 0;
  *keep_x = false;
  int running = 2;
  bool written[kRowRegs] = {false};
  bool is_columns[kRowRegs] = {false};
  for (int i = 0; i < prog.n_inputs; ++i)
    if (prog.kind[i] == DTN_ROW_INPUT_COLUMNS) is_columns[3 + i] = true;
  for (int n = prog.n_scalar; n < prog.n_instr; ++n) {
    if (chain->n >= kChainMax) return false;
    const int op = prog.op[n], a = prog.a[n], b = prog.b[n];
    const bool binary = op <= DTN_EW_MIN;
    int other = -1;
    bool swap = false;
    if (!binary) {
      if (a != running) return false;
    } else if (a == running) {
      other = b;
    } else if (b == running) {
      other = a;
      swap = true;
    } else {
      return false;
    }
    int kind = CHAIN_SELF, index = 0;
    if (binary) {
      if (other == running) {
        kind = CHAIN_SELF;
      } else if (written[other]) {
        return false;
      } else if (other == 2) {
        kind = CHAIN_ELEMENT;
        if (chain->n > 0) *keep_x = true;
      } else if (is_columns[other]) {
        kind = CHAIN_COLUMNS;
        index = other - 3;
      } else {
        kind = CHAIN_SCALAR;
        index = other;
      }
    }
    chain->op[chain->n] = (unsigned char)op;
    chain->kind[chain->n] = (unsigned char)kind;
    chain->index[chain->n] = (unsigned char)index;
    chain->swap[chain->n] = swap ? 1 : 0;
    ++chain->n;
    running = prog.dst[n];
    written[running] = true;
  }
  // softmax: (x - max), exp are what the sum pass computed; the scalar stage must have left the maximum in register 0
  bool max_intact = true;
  for (int n = 0; n < prog.n_scalar; ++n) max_intact = max_intact && prog.dst[n] != 0;
  chain->cached_exp = prog.reduce == DTN_REDUCE_SOFTMAX && !*keep_x && max_intact && chain->n >= 2 && chain->op[0] == DTN_EW_SUB &&
                      chain->kind[0] == CHAIN_SCALAR && chain->index[0] == 0 && chain->swap[0] == 0 && chain->op[1] == DTN_EW_EXP;
  return per_row || prog.out_reg == running;   // a per-row result is read from the scalar registers
}

template <int TPR, int NV>
static int row_chain_launch_nv(const RowProgram& prog, const RowChain& chain, bool keep_x, const float* x, float* out, int64_t rows,
                               int64_t cols, int64_t ldx, int64_t ldo, bool aligned, cudaStream_t s) {
  constexpr int kThreads = TPR <= 32 ? 128 : TPR;
  constexpr int RPB = kThreads / TPR;
  int64_t blocks = (rows + RPB - 1) / RPB;
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  const unsigned grid = (unsigned)blocks;
  if (aligned && keep_x)
    row_chain_kernel<TPR, true, true, NV><<<grid, kThreads, 0, s>>>(prog, chain, x, out, rows, (int)cols, ldx, ldo);
  else if (aligned)
    row_chain_kernel<TPR, true, false, NV><<<grid, kThreads, 0, s>>>(prog, chain, x, out, rows, (int)cols, ldx, ldo);
  else if (keep_x)
    row_chain_kernel<TPR, false, true, 8><<<grid, kThreads, 0, s>>>(prog, chain, x, out, rows, (int)cols, ldx, ldo);
  else
    row_chain_kernel<TPR, false, false, 8><<<grid, kThreads, 0, s>>>(prog, chain, x, out, rows, (int)cols, ldx, ldo);
  DTN_LAUNCH_CHECK("row_chain_kernel");
  return DTN_OK;
}

// The number of vectors a thread keeps: the smallest of 1, 2, 4, 8 that holds the row (aligned rows only; the scalar
// form always keeps eight).
template <int TPR>
static int row_chain_launch(const RowProgram& prog, const RowChain& chain, bool keep_x, const float* x, float* out, int64_t rows,
                            int64_t cols, int64_t ldx, int64_t ldo, bool aligned, cudaStream_t s) {
  if (aligned && cols <= (int64_t)TPR * 4) return row_chain_launch_nv<TPR, 1>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
  if (aligned && cols <= (int64_t)TPR * 8) return row_chain_launch_nv<TPR, 2>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
  if (aligned && cols <= (int64_t)TPR * 16) return row_chain_launch_nv<TPR, 4>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
  return row_chain_launch_nv<TPR, 8>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
}

// Threads per row: the smallest group whose eight vectors per thread hold the whole row, widened while the
// device would otherwise be left mostly idle (few rows) and every thread still gets at least one vector.
static int row_group_size(int64_t rows, int64_t cols) {
  int tpr = 8;
  while (tpr < 256 && (int64_t)tpr * kRowCacheVecs * 4 < cols) tpr *= 2;
  const int64_t wanted = (int64_t)sm_count() * 1024;
  while (tpr < 256 && rows * tpr < wanted && (int64_t)tpr * 2 * 4 <= cols) tpr *= 2;
  return tpr;
}

static int row_fused_launch(const RowProgram& prog, const float* x, float* out, int64_t rows, int64_t cols, int64_t ldx, int64_t ldo,
                            bool aligned, cudaStream_t s) {
  RowChain chain;
  bool keep_x = false;
  if (cols < (1LL << 30) && row_chain_of(prog, &chain, &keep_x, ldo == 0)) {
    switch (row_group_size(rows, cols)) {
      case 8: return row_chain_launch<8>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
      case 16: return row_chain_launch<16>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
      case 32: return row_chain_launch<32>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
      case 64: return row_chain_launch<64>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
      case 128: return row_chain_launch<128>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
      default: return row_chain_launch<256>(prog, chain, keep_x, x, out, rows, cols, ldx, ldo, aligned, s);
    }
  }
  int64_t blocks = rows;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (aligned)
    row_interpreter_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(prog, x, out, rows, cols, ldx, ldo);
  else
    row_interpreter_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(prog, x, out, rows, cols, ldx, ldo);
  DTN_LAUNCH_CHECK("row_interpreter_kernel");
  return DTN_OK;
}

}  // namespace dtn

extern "C" int dtn_row_fused(int reduce_op, const float* x, int64_t rows, int64_t cols, int64_t ldx, const void* const* inputs,
                             const unsigned char* input_kind, const float* input_immediate, int n_inputs,
                             const unsigned char* ops, const unsigned char* dsts, const unsigned char* as,
                             const unsigned char* bs, int n_scalar_instr, int n_instr, int out_reg, float* out, int64_t ldo,
                             void* stream) {
  using namespace dtn;
  DTN_REQUIRE(rows >= 0 && cols >= 0, DTN_ERR_INVALID, "row_fused: negative extent");
  DTN_REQUIRE(reduce_op >= DTN_REDUCE_SUM && reduce_op <= DTN_REDUCE_SOFTMAX, DTN_ERR_INVALID, "row_fused: unknown reduction %d",
              reduce_op);
  DTN_REQUIRE(n_inputs >= 0 && n_inputs <= kRowMaxInputs, DTN_ERR_UNSUPPORTED, "row_fused: at most %d extra inputs",
              kRowMaxInputs);
  DTN_REQUIRE(n_instr >= 0 && n_instr <= kRowMaxInstr && n_scalar_instr >= 0 && n_scalar_instr <= n_instr, DTN_ERR_UNSUPPORTED,
              "row_fused: at most %d instructions, scalar stage first", kRowMaxInstr);
  DTN_REQUIRE(out_reg >= 0 && out_reg < kRowRegs, DTN_ERR_INVALID, "row_fused: bad output register");
  if (rows == 0 || (cols == 0 && ldo != 0)) return DTN_OK;
  DTN_REQUIRE(out != nullptr && (x != nullptr || cols == 0), DTN_ERR_INVALID, "row_fused: null pointer");
  DTN_REQUIRE(ldx >= cols && (ldo == 0 || ldo >= cols), DTN_ERR_INVALID, "row_fused: leading dimension below cols");
  DTN_REQUIRE(ldo != 0 || n_scalar_instr == n_instr, DTN_ERR_INVALID,
              "row_fused: a per-row result takes no elementwise stage");
  DTN_REQUIRE(aligned_to(x, 4) && aligned_to(out, 4), DTN_ERR_INVALID, "row_fused: pointers must be 4-byte aligned");
  DTN_REQUIRE(n_inputs == 0 || (inputs && input_kind && input_immediate), DTN_ERR_INVALID, "row_fused: null input table");
  DTN_REQUIRE(n_instr == 0 || (ops && dsts && as && bs), DTN_ERR_INVALID, "row_fused: null program");
  RowProgram prog = {};
  prog.reduce = reduce_op;
  prog.n_inputs = n_inputs;
  prog.n_scalar = n_scalar_instr;
  prog.n_instr = n_instr;
  prog.out_reg = out_reg;
  bool aligned = aligned_to(x, 16) && ldx % 4 == 0 && cols % 4 == 0 && (ldo == 0 || (aligned_to(out, 16) && ldo % 4 == 0));
  for (int i = 0; i < n_inputs; ++i) {
    DTN_REQUIRE(input_kind[i] <= DTN_ROW_INPUT_IMMEDIATE, DTN_ERR_INVALID, "row_fused: input %d has an unknown kind", i);
    prog.kind[i] = input_kind[i];
    prog.immediate[i] = input_immediate[i];
    if (input_kind[i] != DTN_ROW_INPUT_IMMEDIATE) {
      DTN_REQUIRE(inputs[i] != nullptr && aligned_to(inputs[i], 4), DTN_ERR_INVALID, "row_fused: input %d is null or misaligned", i);
      prog.input[i] = static_cast<const float*>(inputs[i]);
      if (input_kind[i] == DTN_ROW_INPUT_COLUMNS) aligned = aligned && aligned_to(inputs[i], 16);
    }
  }
  for (int k = 0; k < n_instr; ++k) {
    DTN_REQUIRE(ops[k] <= DTN_EW_COPY && dsts[k] < kRowRegs && as[k] < kRowRegs && bs[k] < kRowRegs, DTN_ERR_INVALID,
                "row_fused: instruction %d is malformed", k);
    prog.op[k] = ops[k];
    prog.dst[k] = dsts[k];
    prog.a[k] = as[k];
    prog.b[k] = bs[k];
  }
  return row_fused_launch(prog, x, out, rows, cols, ldx, ldo, aligned, as_stream(stream));
}
