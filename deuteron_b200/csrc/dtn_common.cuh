// Shared host/device helpers for the deuteron_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/deuteron_b200.h"

namespace dtn {

// ---------------------------------------------------------------------------------------
// Host-side error plumbing: one message per host thread, read back by dtn_last_error().
// ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
const char* get_error();

// Device status word written by kernels whose bounded waits run out. One per process.
int* device_status_word();  // device pointer, allocated lazily (returns nullptr on failure)

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

#define DTN_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      ::dtn::set_error("%s failed: %s (%s)", #expr, cudaGetErrorName(_e),                 \
                       cudaGetErrorString(_e));                                           \
      return DTN_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

#define DTN_LAUNCH_CHECK(what)                                                            \
  do {                                                                                    \
    cudaError_t _e = cudaGetLastError();                                                  \
    if (_e != cudaSuccess) {                                                              \
      ::dtn::set_error("launch of %s failed: %s (%s)", what, cudaGetErrorName(_e),        \
                       cudaGetErrorString(_e));                                           \
      return DTN_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

#define DTN_REQUIRE(cond, code, ...)                                                      \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      ::dtn::set_error(__VA_ARGS__);                                                      \
      return code;                                                                        \
    }                                                                                     \
  } while (0)

static inline bool aligned_to(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

int sm_count();  // multiprocessors of the current device (cached)

// ---------------------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Streaming 128-bit global load that does not allocate in L1, and streaming store.
__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_f4(float4* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream_u4(uint4* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// exp(x) as the reference lowers it: ex2.approx(x * log2(e)), log2(e) an FP32 constant.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Flush-to-zero form: one MUFU instruction, no range fix-up around it. Results below 2^-126 become 0; used where such
// values cannot matter (attention probabilities, which are summed with values near 1).
__device__ __forceinline__ float ex2_approx_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float exp_ref(float x) { return ex2_approx(x * 1.4426950408889634f); }
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#endif  // __CUDACC__

}  // namespace dtn
