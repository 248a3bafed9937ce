// Bandwidth-bound row reductions: out[r] = sum / max / sum of squares over a row of FP32.
//
// Short and medium rows: one warp per row. Each lane walks the row in 128-bit vectors at a
// stride of 32 vectors, eight independent loads (32 FP32 accumulators) in flight per lane,
// then a butterfly shuffle combines the lanes. Long rows with few of them: one CTA per row,
// shuffle per warp and one shared-memory round for the warp partials.
#include <math.h>

#include "dtn_common.cuh"

namespace dtn {

template <int OP>
__device__ __forceinline__ float red_identity() {
  if constexpr (OP == DTN_REDUCE_MAX) return -INFINITY;
  return 0.0f;
}
template <int OP>
__device__ __forceinline__ float red_fold(float acc, float v) {
  if constexpr (OP == DTN_REDUCE_MAX) return fmaxf(acc, v);  // NaN-suppressing maxnum
  if constexpr (OP == DTN_REDUCE_SUMSQ) return fmaf(v, v, acc);
  return acc + v;
}
template <int OP>
__device__ __forceinline__ float red_merge(float a, float b) {
  if constexpr (OP == DTN_REDUCE_MAX) return fmaxf(a, b);
  return a + b;
}
template <int OP>
__device__ __forceinline__ float red_warp(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_merge<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Partial of one row seen by one thread of a group of `width` threads with rank `rank`.
template <int OP, bool VEC>
__device__ __forceinline__ float row_partial(const float* __restrict__ row, int64_t cols, int rank,
                                             int width) {
  constexpr int U = 8;
  float acc[U][4];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[u][c] = red_identity<OP>();
  int64_t done = 0;
  if constexpr (VEC) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int64_t nvec = cols >> 2;
    int64_t j = rank;
    for (; j + (int64_t)(U - 1) * width < nvec; j += (int64_t)U * width) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = ld_stream_f4(row4 + j + (int64_t)u * width);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u][0] = red_fold<OP>(acc[u][0], v[u].x);
        acc[u][1] = red_fold<OP>(acc[u][1], v[u].y);
        acc[u][2] = red_fold<OP>(acc[u][2], v[u].z);
        acc[u][3] = red_fold<OP>(acc[u][3], v[u].w);
      }
    }
    for (; j < nvec; j += width) {
      float4 v = ld_stream_f4(row4 + j);
      acc[0][0] = red_fold<OP>(acc[0][0], v.x);
      acc[0][1] = red_fold<OP>(acc[0][1], v.y);
      acc[0][2] = red_fold<OP>(acc[0][2], v.z);
      acc[0][3] = red_fold<OP>(acc[0][3], v.w);
    }
    done = nvec << 2;
  }
  for (int64_t j = done + rank; j < cols; j += width) acc[1][0] = red_fold<OP>(acc[1][0], row[j]);
  // pairwise tree over the 32 accumulators
#pragma unroll
  for (int u = 0; u < U; ++u) {
    acc[u][0] = red_merge<OP>(acc[u][0], acc[u][1]);
    acc[u][2] = red_merge<OP>(acc[u][2], acc[u][3]);
    acc[u][0] = red_merge<OP>(acc[u][0], acc[u][2]);
  }
#pragma unroll
  for (int d = U / 2; d > 0; d >>= 1)
#pragma unroll
    for (int u = 0; u < d; ++u) acc[u][0] = red_merge<OP>(acc[u][0], acc[u + d][0]);
  return acc[0][0];
}

template <int OP, bool VEC>
__global__ void __launch_bounds__(256)
row_reduce_warp_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows,
                       int64_t cols, int64_t ldx) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v = row_partial<OP, VEC>(x + row * ldx, cols, lane, 32);
  v = red_warp<OP>(v);
  if (lane == 0) out[row] = v;
}

template <int OP, bool VEC>
__global__ void __launch_bounds__(512)
row_reduce_block_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows,
                        int64_t cols, int64_t ldx) {
  __shared__ float partial[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float v = row_partial<OP, VEC>(x + row * ldx, cols, threadIdx.x, blockDim.x);
    v = red_warp<OP>(v);
    if (lane == 0) partial[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float w = lane < (blockDim.x >> 5) ? partial[lane] : red_identity<OP>();
      w = red_warp<OP>(w);
      if (lane == 0) out[row] = w;
    }
    __syncthreads();
  }
}

template <int OP>
static int reduce_launch(const float* x, float* out, int64_t rows, int64_t cols, int64_t ldx,
                         cudaStream_t s) {
  const bool vec = aligned_to(x, 16) && (ldx % 4 == 0);
  const bool few_long_rows = rows < (int64_t)sm_count() * 4 && cols >= 8192;
  if (few_long_rows) {
    unsigned grid = (unsigned)rows;
    if (vec)
      row_reduce_block_kernel<OP, true><<<grid, 512, 0, s>>>(x, out, rows, cols, ldx);
    else
      row_reduce_block_kernel<OP, false><<<grid, 512, 0, s>>>(x, out, rows, cols, ldx);
    DTN_LAUNCH_CHECK("row_reduce_block_kernel");
    return DTN_OK;
  }
  const int warps = 8;
  const int64_t blocks = (rows + warps - 1) / warps;
  DTN_REQUIRE(blocks < (int64_t)2147483647, DTN_ERR_UNSUPPORTED, "row_reduce: too many rows");
  if (vec)
    row_reduce_warp_kernel<OP, true><<<(unsigned)blocks, warps * 32, 0, s>>>(x, out, rows, cols, ldx);
  else
    row_reduce_warp_kernel<OP, false><<<(unsigned)blocks, warps * 32, 0, s>>>(x, out, rows, cols, ldx);
  DTN_LAUNCH_CHECK("row_reduce_warp_kernel");
  return DTN_OK;
}

}  // namespace dtn

extern "C" int dtn_row_reduce_f32(int op, const float* x, float* out, int64_t rows, int64_t cols,
                                  int64_t ldx, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(rows >= 0 && cols >= 0, DTN_ERR_INVALID, "row_reduce: negative extent");
  if (rows == 0) return DTN_OK;
  DTN_REQUIRE(out != nullptr && (x != nullptr || cols == 0), DTN_ERR_INVALID, "row_reduce: null pointer");
  DTN_REQUIRE(ldx >= cols, DTN_ERR_INVALID, "row_reduce: ldx < cols");
  DTN_REQUIRE(aligned_to(x, 4) && aligned_to(out, 4), DTN_ERR_INVALID,
              "row_reduce: pointers must be 4-byte aligned");
  cudaStream_t s = as_stream(stream);
  switch (op) {
    case DTN_REDUCE_SUM: return reduce_launch<DTN_REDUCE_SUM>(x, out, rows, cols, ldx, s);
    case DTN_REDUCE_MAX: return reduce_launch<DTN_REDUCE_MAX>(x, out, rows, cols, ldx, s);
    case DTN_REDUCE_SUMSQ: return reduce_launch<DTN_REDUCE_SUMSQ>(x, out, rows, cols, ldx, s);
    default:
      set_error("row_reduce: unknown operator %d", op);
      return DTN_ERR_INVALID;
  }
}
