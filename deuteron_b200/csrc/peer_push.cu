// Pushes a finished block of a row-major FP32 matrix into the same place of up to seven other copies of that
// matrix -- the copies of the other GPUs of a column-sharded GEMM, addressed through peer mappings (symmetric
// memory). The block is read once and every 16-byte piece is stored to each destination; a warp writes 512
// contiguous bytes of a row per destination. One copy per peer reaches the same rate to a single peer (626-650
// against 678 GB/s on B200); with seven peers one launch that reads the block once was the faster form (4.83
// against 5.1 ms for the whole overlapped product on 8 GPUs). The kernel is meant to run on a side stream next to
// the product kernel: few CTAs, no shared memory, so that it fits on the SMs the persistent GEMM occupies.
#include <stdlib.h>

#include "dtn_common.cuh"

namespace dtn {

constexpr int kPushMaxDst = 7;

struct PushTargets {
  float* dst[kPushMaxDst];
};

template <bool VEC>
__global__ void __launch_bounds__(256)
push_block_kernel(const float* __restrict__ src, int64_t lds, PushTargets targets, int n_dst, int64_t ldd, int64_t rows,
                  int64_t cols) {
  const int64_t per_row = VEC ? cols / 4 : cols;
  const int64_t total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / per_row, piece = i - row * per_row;
    if constexpr (VEC) {
      const float4 v = ld_stream_f4(reinterpret_cast<const float4*>(src + row * lds) + piece);
#pragma unroll
      for (int d = 0; d < kPushMaxDst; ++d)
        if (d < n_dst) reinterpret_cast<float4*>(targets.dst[d] + row * ldd)[piece] = v;
    } else {
      const float v = src[row * lds + piece];
#pragma unroll
      for (int d = 0; d < kPushMaxDst; ++d)
        if (d < n_dst) targets.dst[d][row * ldd + piece] = v;
    }
  }
}

}  // namespace dtn

extern "C" int dtn_push_block(const float* src, int64_t lds, float* const* dsts, int n_dst, int64_t ldd, int64_t rows,
                              int64_t cols, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(rows >= 0 && cols >= 0, DTN_ERR_INVALID, "push_block: negative extent");
  DTN_REQUIRE(n_dst >= 0 && n_dst <= kPushMaxDst, DTN_ERR_INVALID, "push_block: between 0 and %d destinations, got %d", kPushMaxDst,
              n_dst);
  if (rows == 0 || cols == 0 || n_dst == 0) return DTN_OK;
  DTN_REQUIRE(src != nullptr && dsts != nullptr, DTN_ERR_INVALID, "push_block: null pointer");
  DTN_REQUIRE(lds >= cols && ldd >= cols, DTN_ERR_INVALID, "push_block: leading dimension smaller than the row");
  PushTargets targets = {};
  bool vec = aligned_to(src, 16) && lds % 4 == 0 && ldd % 4 == 0 && cols % 4 == 0;
  for (int d = 0; d < n_dst; ++d) {
    DTN_REQUIRE(dsts[d] != nullptr, DTN_ERR_INVALID, "push_block: destination %d is null", d);
    DTN_REQUIRE(aligned_to(dsts[d], 4) && dsts[d] != src, DTN_ERR_INVALID, "push_block: destination %d misaligned or equal to the source", d);
    targets.dst[d] = dsts[d];
    vec = vec && aligned_to(dsts[d], 16);
  }
  DTN_REQUIRE(aligned_to(src, 4), DTN_ERR_INVALID, "push_block: source must be 4-byte aligned");
  const int64_t pieces = rows * (vec ? cols / 4 : cols);
  // two CTAs per SM at most: the kernel shares the SMs with a running GEMM and is bound by the links, not by issue slots
  int64_t ctas = (pieces + 255) / 256;
  static const int per_sm = [] {
    const char* text = getenv("DTN_PUSH_CTAS_PER_SM");   // tuning aid
    const int value = text ? atoi(text) : 0;
    return value >= 1 && value <= 8 ? value : 2;
  }();
  const int64_t cap = (int64_t)sm_count() * per_sm;
  if (ctas > cap) ctas = cap;
  cudaStream_t s = as_stream(stream);
  if (vec)
    push_block_kernel<true><<<(unsigned)ctas, 256, 0, s>>>(src, lds, targets, n_dst, ldd, rows, cols);
  else
    push_block_kernel<false><<<(unsigned)ctas, 256, 0, s>>>(src, lds, targets, n_dst, ldd, rows, cols);
  DTN_LAUNCH_CHECK("push_block_kernel");
  return DTN_OK;
}
