// Fused row kernels: one reduction over every row of x[rows, cols], a scalar stage on the reduced
// value, and an elementwise stage over the same row -- row softmax, RMS norm, L2 norm and mean in
// one launch and (for rows of up to 8192 values) one trip through memory.
//
// The reference reaches the same fusion by rewriting the scheduled IR: load forwarding keeps the row
// in registers between the reduction loop and the consumer loop (compiler/passes/regforward.py:150-269)
// and the softmax normaliser replaces the online (max, sum) pair by a max pass followed by a sum of
// exponentials over cached values (compiler/passes/hybrid_normalizer.py:139-183). Here the row is
// read once with 128-bit loads into at most eight vectors per thread, reduced by a butterfly shuffle
// (and one shared-memory round when a whole CTA shares the row), and written once; longer or
// unaligned rows take the same code through loops that re-read the row (mostly from L2).
//
// The two stages arrive as one short register program: instructions [0, n_scalar) run once per row
// on the reduced value and the one-element inputs, the rest run per element. Register 0 holds the
// reduced value, register 1 the sum of exp(x - max) for the softmax reduction, register 2 the row
// element, registers 3.. the extra inputs in order; the others are temporaries.
#include <math.h>

#include "dtn_common.cuh"
#include "program.cuh"

namespace dtn {

constexpr int kRowRegs = 12;
constexpr int kRowMaxInstr = 32;
constexpr int kRowMaxInputs = 5;
constexpr int kRowCacheVecs = 8;   // 128-bit vectors of the row one thread keeps in registers

struct RowProgram {
  int n_inputs, n_scalar, n_instr, out_reg;
  const float* input[kRowMaxInputs];
  float immediate[kRowMaxInputs];
  unsigned char kind[kRowMaxInputs];
  unsigned char op[kRowMaxInstr], dst[kRowMaxInstr], a[kRowMaxInstr], b[kRowMaxInstr];
};

// Combines one value per thread over the TPR threads that share a row.
template <int TPR, bool MAX>
__device__ __forceinline__ float row_combine(float v, float* scratch) {
  v = MAX ? warp_max(v) : warp_sum(v);
  if constexpr (TPR > 32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float w = lane < TPR / 32 ? scratch[lane] : (MAX ? -INFINITY : 0.0f);
    v = MAX ? warp_max(w) : warp_sum(w);
    __syncthreads();
  }
  return v;
}

template <int RED>
__device__ __forceinline__ float fold_first(float acc, float v) {
  if constexpr (RED == DTN_REDUCE_SUM) return acc + v;
  if constexpr (RED == DTN_REDUCE_SUMSQ) return fmaf(v, v, acc);
  return fmaxf(acc, v);   // max and softmax
}

// The elementwise stage on W consecutive elements starting at column `col` (W = 2 needs col even and the
// column inputs 8-byte aligned there, which the aligned modes guarantee).
template <int W>
__device__ __forceinline__ void element_compute(const RowProgram& prog, const RegFile<kRowRegs, 1>& scalars, const float (&xv)[W],
                                                int64_t col, float (&result)[W]) {
  RegFile<kRowRegs, W> regs;
#pragma unroll
  for (int k = 0; k < kRowRegs; ++k)
#pragma unroll
    for (int e = 0; e < W; ++e) regs.r[k][e] = scalars.r[k][0];
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

// One 128-bit vector of the row: two interpreter passes of two elements (a narrow register file keeps the
// kernel at two CTAs per SM), one 128-bit store.
__device__ __forceinline__ void element_vector(const RowProgram& prog, const RegFile<kRowRegs, 1>& scalars, const float4 v,
                                               int64_t col, float* __restrict__ out_row) {
  const float lo[2] = {v.x, v.y}, hi[2] = {v.z, v.w};
  float r0[2], r1[2];
  element_compute<2>(prog, scalars, lo, col, r0);
  element_compute<2>(prog, scalars, hi, col + 2, r1);
  st_stream_f4(reinterpret_cast<float4*>(out_row + col), make_float4(r0[0], r0[1], r1[0], r1[1]));
}

// MODE 0: aligned row of at most TPR * kRowCacheVecs vectors, kept in registers. MODE 1: aligned, streamed.
// MODE 2: scalar accesses (any alignment, any cols).
template <int RED, int TPR, int MODE>
__global__ void __launch_bounds__(256, 2)
row_fused_kernel(const RowProgram prog, const float* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t cols,
                 int64_t ldx, int64_t ldo) {
  constexpr int RPB = 256 / TPR;   // rows per CTA
  constexpr bool kMax = RED == DTN_REDUCE_MAX || RED == DTN_REDUCE_SOFTMAX;
  __shared__ float scratch[8];
  const int rank = threadIdx.x % TPR, sub = threadIdx.x / TPR;
  const int64_t nvec = cols >> 2;
  for (int64_t row0 = (int64_t)blockIdx.x * RPB; row0 < rows; row0 += (int64_t)gridDim.x * RPB) {
    int64_t row = row0 + sub;
    const bool live = row < rows;   // uniform over a warp (TPR == 32) or over the CTA (TPR == 256, RPB == 1)
    if (!live) row = rows - 1;      // idle warps of the last CTA repeat the last row and store nothing
    const float* xr = x + row * ldx;
    float4 cache[kRowCacheVecs];
    float first = kMax ? -INFINITY : 0.0f;
    if constexpr (MODE == 0) {
#pragma unroll
      for (int u = 0; u < kRowCacheVecs; ++u) {
        const int64_t j = rank + (int64_t)u * TPR;
        if (j < nvec) cache[u] = ld_stream_f4(reinterpret_cast<const float4*>(xr) + j);
      }
      float part[4] = {first, first, first, first};
#pragma unroll
      for (int u = 0; u < kRowCacheVecs; ++u) {
        if (rank + (int64_t)u * TPR < nvec) {
          part[0] = fold_first<RED>(part[0], cache[u].x);
          part[1] = fold_first<RED>(part[1], cache[u].y);
          part[2] = fold_first<RED>(part[2], cache[u].z);
          part[3] = fold_first<RED>(part[3], cache[u].w);
        }
      }
      first = kMax ? fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) : (part[0] + part[1]) + (part[2] + part[3]);
    } else if constexpr (MODE == 1) {
      float part[4] = {first, first, first, first};
      for (int64_t j = rank; j < nvec; j += TPR) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + j);
        part[0] = fold_first<RED>(part[0], v.x);
        part[1] = fold_first<RED>(part[1], v.y);
        part[2] = fold_first<RED>(part[2], v.z);
        part[3] = fold_first<RED>(part[3], v.w);
      }
      first = kMax ? fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) : (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (int64_t j = rank; j < cols; j += TPR) first = fold_first<RED>(first, xr[j]);
    }
    first = row_combine<TPR, kMax>(first, scratch);

    float second = 0.0f;
    if constexpr (RED == DTN_REDUCE_SOFTMAX) {
      if constexpr (MODE == 0) {
#pragma unroll
        for (int u = 0; u < kRowCacheVecs; ++u) {
          if (rank + (int64_t)u * TPR < nvec)
            second += (exp_ref(cache[u].x - first) + exp_ref(cache[u].y - first)) +
                      (exp_ref(cache[u].z - first) + exp_ref(cache[u].w - first));
        }
      } else if constexpr (MODE == 1) {
        for (int64_t j = rank; j < nvec; j += TPR) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + j);
          second += (exp_ref(v.x - first) + exp_ref(v.y - first)) + (exp_ref(v.z - first) + exp_ref(v.w - first));
        }
      } else {
        for (int64_t j = rank; j < cols; j += TPR) second += exp_ref(xr[j] - first);
      }
      second = row_combine<TPR, false>(second, scratch);
    }

    // scalar stage (every thread of the row computes the same values)
    RegFile<kRowRegs, 1> scalars;
#pragma unroll
    for (int k = 0; k < kRowRegs; ++k) scalars.r[k][0] = 0.0f;
    scalars.r[0][0] = first;
    scalars.r[1][0] = second;
#pragma unroll
    for (int i = 0; i < kRowMaxInputs; ++i) {
      if (i < prog.n_inputs && prog.kind[i] != DTN_ROW_INPUT_COLUMNS) {
        const float v[1] = {prog.kind[i] == DTN_ROW_INPUT_IMMEDIATE ? prog.immediate[i] : __ldg(prog.input[i])};
        scalars.put(3 + i, v);
      }
    }
    for (int n = 0; n < prog.n_scalar; ++n) {
      float a[1], b[1], d[1];
      scalars.get(prog.a[n], a);
      scalars.get(prog.b[n], b);
      d[0] = prog_apply(prog.op[n], a[0], b[0]);
      scalars.put(prog.dst[n], d);
    }
    if (ldo == 0) {   // one value per row
      if (live && rank == 0) {
        float result[1];
        scalars.get(prog.out_reg, result);
        out[row] = result[0];
      }
      continue;
    }
    if (!live) continue;
    float* out_row = out + row * ldo;
    if constexpr (MODE == 0) {
#pragma unroll
      for (int u = 0; u < kRowCacheVecs; ++u) {
        const int64_t j = rank + (int64_t)u * TPR;
        if (j < nvec) element_vector(prog, scalars, cache[u], j * 4, out_row);
      }
    } else if constexpr (MODE == 1) {
      for (int64_t j = rank; j < nvec; j += TPR) {
        element_vector(prog, scalars, __ldg(reinterpret_cast<const float4*>(xr) + j), j * 4, out_row);
      }
    } else {
      for (int64_t j = rank; j < cols; j += TPR) {
        const float xv[1] = {xr[j]};
        float result[1];
        element_compute<1>(prog, scalars, xv, j, result);
        out_row[j] = result[0];
      }
    }
  }
}

template <int RED, int TPR>
static int row_fused_launch_mode(const RowProgram& prog, const float* x, float* out, int64_t rows, int64_t cols, int64_t ldx,
                                 int64_t ldo, int mode, cudaStream_t s) {
  constexpr int RPB = 256 / TPR;
  int64_t blocks = (rows + RPB - 1) / RPB;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const unsigned grid = (unsigned)blocks;
  if (mode == 0)
    row_fused_kernel<RED, TPR, 0><<<grid, 256, 0, s>>>(prog, x, out, rows, cols, ldx, ldo);
  else if (mode == 1)
    row_fused_kernel<RED, TPR, 1><<<grid, 256, 0, s>>>(prog, x, out, rows, cols, ldx, ldo);
  else
    row_fused_kernel<RED, TPR, 2><<<grid, 256, 0, s>>>(prog, x, out, rows, cols, ldx, ldo);
  DTN_LAUNCH_CHECK("row_fused_kernel");
  return DTN_OK;
}

template <int RED>
static int row_fused_launch(const RowProgram& prog, const float* x, float* out, int64_t rows, int64_t cols, int64_t ldx,
                            int64_t ldo, bool aligned, cudaStream_t s) {
  // A warp per row while a lane holds at most two vectors of it, or when there are rows enough to fill the
  // device with warps; a whole CTA per row otherwise.
  const bool warp_rows = cols <= 256 || (cols <= 1024 && rows >= (int64_t)sm_count() * 64);
  const int tpr = warp_rows ? 32 : 256;
  const int mode = !aligned ? 2 : ((cols >> 2) <= (int64_t)tpr * kRowCacheVecs ? 0 : 1);
  if (warp_rows) return row_fused_launch_mode<RED, 32>(prog, x, out, rows, cols, ldx, ldo, mode, s);
  return row_fused_launch_mode<RED, 256>(prog, x, out, rows, cols, ldx, ldo, mode, s);
}

}  // namespace dtn

extern "C" int dtn_row_fused(int reduce_op, const float* x, int64_t rows, int64_t cols, int64_t ldx, const void* const* inputs,
                             const unsigned char* input_kind, const float* input_immediate, int n_inputs,
                             const unsigned char* ops, const unsigned char* dsts, const unsigned char* as,
                             const unsigned char* bs, int n_scalar_instr, int n_instr, int out_reg, float* out, int64_t ldo,
                             void* stream) {
  using namespace dtn;
  DTN_REQUIRE(rows >= 0 && cols >= 0, DTN_ERR_INVALID, "row_fused: negative extent");
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
  cudaStream_t s = as_stream(stream);
  switch (reduce_op) {
    case DTN_REDUCE_SUM: return row_fused_launch<DTN_REDUCE_SUM>(prog, x, out, rows, cols, ldx, ldo, aligned, s);
    case DTN_REDUCE_MAX: return row_fused_launch<DTN_REDUCE_MAX>(prog, x, out, rows, cols, ldx, ldo, aligned, s);
    case DTN_REDUCE_SUMSQ: return row_fused_launch<DTN_REDUCE_SUMSQ>(prog, x, out, rows, cols, ldx, ldo, aligned, s);
    case DTN_REDUCE_SOFTMAX: return row_fused_launch<DTN_REDUCE_SOFTMAX>(prog, x, out, rows, cols, ldx, ldo, aligned, s);
    default:
      set_error("row_fused: unknown reduction %d", reduce_op);
      return DTN_ERR_INVALID;
  }
}
