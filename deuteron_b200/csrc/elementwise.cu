// Bandwidth-bound elementwise kernels: FP32 elementwise operators and the f16 storage
// kernels (copy / widen / narrow). Every kernel moves 128-bit vectors per thread, keeps
// several independent loads in flight, and uses streaming loads/stores because each byte
// is touched once. Unaligned origins are handled by a scalar head and tail around the
// vector body; if the buffers' misalignments cannot be reconciled the scalar kernel runs.
#include "dtn_common.cuh"

namespace dtn {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;  // 128-bit vectors per thread per array

template <int OP>
__device__ __forceinline__ float ew_apply(float a, float b) {
  if constexpr (OP == DTN_EW_ADD) return __fadd_rn(a, b);
  if constexpr (OP == DTN_EW_SUB) return __fsub_rn(a, b);
  if constexpr (OP == DTN_EW_MUL) return __fmul_rn(a, b);
  if constexpr (OP == DTN_EW_DIV) return __fdividef(a, b);
  if constexpr (OP == DTN_EW_MAX) return fmaxf(a, b);
  if constexpr (OP == DTN_EW_MIN) return fminf(a, b);
  if constexpr (OP == DTN_EW_RELU) return fmaxf(a, 0.0f);
  if constexpr (OP == DTN_EW_EXP) return exp_ref(a);
  if constexpr (OP == DTN_EW_SQRT) {
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a));
    return y;
  }
  if constexpr (OP == DTN_EW_RSQRT) {
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a));
    return y;
  }
  if constexpr (OP == DTN_EW_RCP) return rcp_approx(a);
  if constexpr (OP == DTN_EW_NEG) return -a;
  if constexpr (OP == DTN_EW_ABS) return fabsf(a);
  return a;  // copy
}

template <int OP>
constexpr bool ew_is_binary() {
  return OP == DTN_EW_ADD || OP == DTN_EW_SUB || OP == DTN_EW_MUL || OP == DTN_EW_DIV ||
         OP == DTN_EW_MAX || OP == DTN_EW_MIN;
}

// Vector body: x, y, out are 16-byte aligned here; nvec = number of float4.
template <int OP>
__global__ void __launch_bounds__(kEwThreads)
ew_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ y, float4* __restrict__ out,
              int64_t nvec) {
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * kEwUnroll) + threadIdx.x;
  float4 a[kEwUnroll], b[kEwUnroll];
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec) {
      a[u] = ld_stream_f4(x + i);
      if constexpr (ew_is_binary<OP>()) b[u] = ld_stream_f4(y + i);
    }
  }
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec) {
      float4 r;
      if constexpr (ew_is_binary<OP>()) {
        r.x = ew_apply<OP>(a[u].x, b[u].x);
        r.y = ew_apply<OP>(a[u].y, b[u].y);
        r.z = ew_apply<OP>(a[u].z, b[u].z);
        r.w = ew_apply<OP>(a[u].w, b[u].w);
      } else {
        r.x = ew_apply<OP>(a[u].x, 0.f);
        r.y = ew_apply<OP>(a[u].y, 0.f);
        r.z = ew_apply<OP>(a[u].z, 0.f);
        r.w = ew_apply<OP>(a[u].w, 0.f);
      }
      st_stream_f4(out + i, r);
    }
  }
}

// Scalar kernel for heads, tails and irreconcilable alignments.
template <int OP>
__global__ void __launch_bounds__(kEwThreads)
ew_scalar_kernel(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ out,
                 int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float b = 0.f;
    if constexpr (ew_is_binary<OP>()) b = y[i];
    out[i] = ew_apply<OP>(x[i], b);
  }
}

// Smallest head h (in elements, < 16) that brings every pointer to a 16-byte boundary,
// or -1 when no such h exists. sizes[i] = element size of pointer i.
static int common_head(const void* const* ptrs, const int* sizes, int count) {
  for (int h = 0; h < 16; ++h) {
    bool ok = true;
    for (int i = 0; i < count && ok; ++i)
      ok = ((reinterpret_cast<uintptr_t>(ptrs[i]) + (uintptr_t)h * sizes[i]) & 15) == 0;
    if (ok) return h;
  }
  return -1;
}

static inline unsigned scalar_grid(int64_t n) {
  int64_t blocks = (n + kEwThreads - 1) / kEwThreads;
  int64_t cap = (int64_t)sm_count() * 8;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <int OP>
static int ew_launch(const float* x, const float* y, float* out, int64_t n, cudaStream_t s) {
  const void* ptrs[3] = {x, out, y};
  const int sizes[3] = {4, 4, 4};
  const int count = ew_is_binary<OP>() ? 3 : 2;
  int head = common_head(ptrs, sizes, count);
  if (head < 0 || n < 64) {
    ew_scalar_kernel<OP><<<scalar_grid(n), kEwThreads, 0, s>>>(x, y, out, n);
    DTN_LAUNCH_CHECK("ew_scalar_kernel");
    return DTN_OK;
  }
  if (head > n) head = (int)n;
  const int64_t nvec = (n - head) / 4;
  const int64_t tail_start = head + nvec * 4;
  if (head > 0) {
    ew_scalar_kernel<OP><<<1, 32, 0, s>>>(x, y, out, head);
    DTN_LAUNCH_CHECK("ew_scalar_kernel(head)");
  }
  if (nvec > 0) {
    const int64_t per_block = kEwThreads * kEwUnroll;
    const int64_t blocks = (nvec + per_block - 1) / per_block;
    DTN_REQUIRE(blocks < (int64_t)2147483647, DTN_ERR_UNSUPPORTED, "elementwise: n too large");
    ew_vec_kernel<OP><<<(unsigned)blocks, kEwThreads, 0, s>>>(
        reinterpret_cast<const float4*>(x + head),
        ew_is_binary<OP>() ? reinterpret_cast<const float4*>(y + head) : nullptr,
        reinterpret_cast<float4*>(out + head), nvec);
    DTN_LAUNCH_CHECK("ew_vec_kernel");
  }
  if (tail_start < n) {
    ew_scalar_kernel<OP><<<1, 32, 0, s>>>(x + tail_start, ew_is_binary<OP>() ? y + tail_start : nullptr,
                                          out + tail_start, n - tail_start);
    DTN_LAUNCH_CHECK("ew_scalar_kernel(tail)");
  }
  return DTN_OK;
}

// ------------------------------- f16 storage ------------------------------------------

// narrow: 8 floats (two float4) -> 8 halves (one uint4) per step.
__global__ void __launch_bounds__(kEwThreads)
f16_narrow_vec_kernel(const float4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec8) {
  constexpr int U = 2;
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * U) + threadIdx.x;
  float4 a[U], b[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) {
      a[u] = ld_stream_f4(src + 2 * i);
      b[u] = ld_stream_f4(src + 2 * i + 1);
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) {
      __half2 h0 = __floats2half2_rn(a[u].x, a[u].y);
      __half2 h1 = __floats2half2_rn(a[u].z, a[u].w);
      __half2 h2 = __floats2half2_rn(b[u].x, b[u].y);
      __half2 h3 = __floats2half2_rn(b[u].z, b[u].w);
      uint4 r;
      r.x = *reinterpret_cast<uint32_t*>(&h0);
      r.y = *reinterpret_cast<uint32_t*>(&h1);
      r.z = *reinterpret_cast<uint32_t*>(&h2);
      r.w = *reinterpret_cast<uint32_t*>(&h3);
      st_stream_u4(dst + i, r);
    }
  }
}

__global__ void __launch_bounds__(kEwThreads)
f16_widen_vec_kernel(const uint4* __restrict__ src, float4* __restrict__ dst, int64_t nvec8) {
  constexpr int U = 2;
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * U) + threadIdx.x;
  uint4 a[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) a[u] = ld_stream_u4(src + i);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) {
      float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&a[u].x));
      float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&a[u].y));
      float2 f2 = __half22float2(*reinterpret_cast<__half2*>(&a[u].z));
      float2 f3 = __half22float2(*reinterpret_cast<__half2*>(&a[u].w));
      st_stream_f4(dst + 2 * i, make_float4(f0.x, f0.y, f1.x, f1.y));
      st_stream_f4(dst + 2 * i + 1, make_float4(f2.x, f2.y, f3.x, f3.y));
    }
  }
}

__global__ void __launch_bounds__(kEwThreads)
f16_copy_vec_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec8) {
  constexpr int U = 4;
  const int64_t base = (int64_t)blockIdx.x * (kEwThreads * U) + threadIdx.x;
  uint4 a[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) a[u] = ld_stream_u4(src + i);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = base + (int64_t)u * kEwThreads;
    if (i < nvec8) st_stream_u4(dst + i, a[u]);
  }
}

// mode 0 = copy, 1 = widen, 2 = narrow
template <int MODE>
__global__ void __launch_bounds__(kEwThreads)
f16_scalar_kernel(const void* __restrict__ src, void* __restrict__ dst, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if constexpr (MODE == 0) {
      static_cast<uint16_t*>(dst)[i] = static_cast<const uint16_t*>(src)[i];
    } else if constexpr (MODE == 1) {
      static_cast<float*>(dst)[i] = __half2float(static_cast<const __half*>(src)[i]);
    } else {
      static_cast<__half*>(dst)[i] = __float2half_rn(static_cast<const float*>(src)[i]);
    }
  }
}

template <int MODE>
static int f16_launch(const void* src, void* dst, int64_t n, cudaStream_t s) {
  constexpr int src_size = (MODE == 2) ? 4 : 2;
  constexpr int dst_size = (MODE == 1) ? 4 : 2;
  const void* ptrs[2] = {src, dst};
  const int sizes[2] = {src_size, dst_size};
  const char* sp = static_cast<const char*>(src);
  char* dp = static_cast<char*>(dst);
  int head = common_head(ptrs, sizes, 2);
  if (head < 0 || n < 64) {
    f16_scalar_kernel<MODE><<<scalar_grid(n), kEwThreads, 0, s>>>(src, dst, n);
    DTN_LAUNCH_CHECK("f16_scalar_kernel");
    return DTN_OK;
  }
  const int64_t nvec8 = (n - head) / 8;
  const int64_t tail_start = head + nvec8 * 8;
  if (head > 0) {
    f16_scalar_kernel<MODE><<<1, 32, 0, s>>>(src, dst, head);
    DTN_LAUNCH_CHECK("f16_scalar_kernel(head)");
  }
  if (nvec8 > 0) {
    const void* vs = sp + (int64_t)head * src_size;
    void* vd = dp + (int64_t)head * dst_size;
    constexpr int U = (MODE == 0) ? 4 : 2;
    const int64_t per_block = kEwThreads * U;
    const int64_t blocks = (nvec8 + per_block - 1) / per_block;
    DTN_REQUIRE(blocks < (int64_t)2147483647, DTN_ERR_UNSUPPORTED, "f16: n too large");
    if constexpr (MODE == 0)
      f16_copy_vec_kernel<<<(unsigned)blocks, kEwThreads, 0, s>>>(static_cast<const uint4*>(vs),
                                                                  static_cast<uint4*>(vd), nvec8);
    else if constexpr (MODE == 1)
      f16_widen_vec_kernel<<<(unsigned)blocks, kEwThreads, 0, s>>>(static_cast<const uint4*>(vs),
                                                                   static_cast<float4*>(vd), nvec8);
    else
      f16_narrow_vec_kernel<<<(unsigned)blocks, kEwThreads, 0, s>>>(static_cast<const float4*>(vs),
                                                                    static_cast<uint4*>(vd), nvec8);
    DTN_LAUNCH_CHECK("f16 vector kernel");
  }
  if (tail_start < n) {
    f16_scalar_kernel<MODE><<<1, 32, 0, s>>>(sp + tail_start * src_size, dp + tail_start * dst_size,
                                             n - tail_start);
    DTN_LAUNCH_CHECK("f16_scalar_kernel(tail)");
  }
  return DTN_OK;
}

}  // namespace dtn

extern "C" {

int dtn_elementwise_f32(int op, const float* x, const float* y, float* out, int64_t n, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(n >= 0, DTN_ERR_INVALID, "elementwise: negative n");
  if (n == 0) return DTN_OK;
  DTN_REQUIRE(x && out, DTN_ERR_INVALID, "elementwise: null pointer");
  DTN_REQUIRE(aligned_to(x, 4) && aligned_to(out, 4) && (!y || aligned_to(y, 4)), DTN_ERR_INVALID,
              "elementwise: pointers must be 4-byte aligned");
  cudaStream_t s = as_stream(stream);
#define DTN_EW_CASE(OP, NEEDS_Y)                                                        \
  case OP:                                                                              \
    if (NEEDS_Y) DTN_REQUIRE(y != nullptr, DTN_ERR_INVALID, "elementwise: y is null");   \
    return ew_launch<OP>(x, y, out, n, s);
  switch (op) {
    DTN_EW_CASE(DTN_EW_ADD, true)
    DTN_EW_CASE(DTN_EW_SUB, true)
    DTN_EW_CASE(DTN_EW_MUL, true)
    DTN_EW_CASE(DTN_EW_DIV, true)
    DTN_EW_CASE(DTN_EW_MAX, true)
    DTN_EW_CASE(DTN_EW_MIN, true)
    DTN_EW_CASE(DTN_EW_RELU, false)
    DTN_EW_CASE(DTN_EW_EXP, false)
    DTN_EW_CASE(DTN_EW_SQRT, false)
    DTN_EW_CASE(DTN_EW_RSQRT, false)
    DTN_EW_CASE(DTN_EW_RCP, false)
    DTN_EW_CASE(DTN_EW_NEG, false)
    DTN_EW_CASE(DTN_EW_ABS, false)
    DTN_EW_CASE(DTN_EW_COPY, false)
    default:
      set_error("elementwise: unknown operator %d", op);
      return DTN_ERR_INVALID;
  }
#undef DTN_EW_CASE
}

int dtn_add_f32(const float* x, const float* y, float* out, int64_t n, void* stream) {
  return dtn_elementwise_f32(DTN_EW_ADD, x, y, out, n, stream);
}

static int f16_check(const void* src, void* dst, int64_t n, int sa, int da) {
  using namespace dtn;
  DTN_REQUIRE(n >= 0, DTN_ERR_INVALID, "f16: negative n");
  if (n == 0) return DTN_OK;
  DTN_REQUIRE(src && dst, DTN_ERR_INVALID, "f16: null pointer");
  DTN_REQUIRE(aligned_to(src, sa) && aligned_to(dst, da), DTN_ERR_INVALID,
              "f16: pointers must have their natural alignment");
  return DTN_OK;
}

int dtn_f16_copy(const uint16_t* src, uint16_t* dst, int64_t n, void* stream) {
  int rc = f16_check(src, dst, n, 2, 2);
  if (rc || n == 0) return rc;
  return dtn::f16_launch<0>(src, dst, n, dtn::as_stream(stream));
}
int dtn_f16_widen(const uint16_t* src, float* dst, int64_t n, void* stream) {
  int rc = f16_check(src, dst, n, 2, 4);
  if (rc || n == 0) return rc;
  return dtn::f16_launch<1>(src, dst, n, dtn::as_stream(stream));
}
int dtn_f16_narrow(const float* src, uint16_t* dst, int64_t n, void* stream) {
  int rc = f16_check(src, dst, n, 4, 2);
  if (rc || n == 0) return rc;
  return dtn::f16_launch<2>(src, dst, n, dtn::as_stream(stream));
}

}  // extern "C"
