// Register programs shared by the fused elementwise and fused row kernels: a small register file held
// in real registers (every index is resolved by a compare chain, so nothing spills to local memory)
// and the operator table. Arithmetic is FP32 with one rounding per operator, never contracted into
// fma, so a program computes what the reference computes operator by operator; exp, sqrt, rsqrt and
// reciprocal are the approximate instructions the reference emits by default
// (compiler/codegen/lower.py:259-289).
#pragma once
#include "dtn_common.cuh"

namespace dtn {

template <int NREG, int W>
struct RegFile {
  float r[NREG][W];
  __device__ __forceinline__ void get(int idx, float (&out)[W]) const {
#pragma unroll
    for (int k = 0; k < NREG; ++k)
      if (idx == k) {
#pragma unroll
        for (int e = 0; e < W; ++e) out[e] = r[k][e];
      }
  }
  __device__ __forceinline__ void put(int idx, const float (&in)[W]) {
#pragma unroll
    for (int k = 0; k < NREG; ++k)
      if (idx == k) {
#pragma unroll
        for (int e = 0; e < W; ++e) r[k][e] = in[e];
      }
  }
};

__device__ __forceinline__ float prog_apply(int op, float a, float b) {
  switch (op) {
    case DTN_EW_ADD: return __fadd_rn(a, b);
    case DTN_EW_SUB: return __fsub_rn(a, b);
    case DTN_EW_MUL: return __fmul_rn(a, b);
    case DTN_EW_DIV: return __fdividef(a, b);
    case DTN_EW_MAX: return fmaxf(a, b);
    case DTN_EW_MIN: return fminf(a, b);
    case DTN_EW_RELU: return fmaxf(a, 0.0f);
    case DTN_EW_EXP: return exp_ref(a);
    case DTN_EW_SQRT: {
      float y;
      asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a));
      return y;
    }
    case DTN_EW_RSQRT: {
      float y;
      asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a));
      return y;
    }
    case DTN_EW_RCP: return rcp_approx(a);
    case DTN_EW_NEG: return -a;
    case DTN_EW_ABS: return fabsf(a);
    default: return a;
  }
}

}  // namespace dtn
