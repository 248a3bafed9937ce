// Compensated FP32 GEMM on the sm_100a tensor cores: C = A*B with every FP32 operand split
// into a rounded high part and a rounded residual (bf16 or tf32) and the three products
// lo*hi, hi*lo, hi*hi accumulated in FP32 in tensor memory.
//
// Two passes:
//   1. split kernels turn A[M,K] and B[K,N] into K-major planes in the caller's workspace:
//      A_hi, A_lo [M, Kp] and (B transposed) Bt_hi, Bt_lo [N, Kp]. The split costs one read
//      of each operand and is not repeated per tile.
//   2. a persistent, warp-specialised kernel: one thread issues TMA tile loads of the four
//      planes into a shared-memory ring (128-byte swizzle), one thread issues the
//      tcgen05.mma instructions (three per k-step) into a double-buffered tensor-memory
//      accumulator, four warps drain finished accumulators with tcgen05.ld and store C
//      while the next tile's products run.
// Variants: one CTA per 128xBN tile (BN = 128 or 256) or a CTA pair per 256x256 tile
// (cta_group::2: each CTA loads its own 128 rows of A and its own half of B; no load is
// shared between CTAs by multicast).
#include <cuda.h>

#include <stdlib.h>

#include <mutex>
#include <type_traits>
#include <algorithm>
#include <vector>

#include "dtn_common.cuh"
#include "sm100_ptx.cuh"

namespace dtn {

int gemm_f32_launch(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t s, bool split_k_allowed);
int gemm_skinny_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                       int64_t ldc, void* workspace, cudaStream_t s);
bool gemm_skinny_supported(const float* A, const float* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb);
size_t gemm_skinny_workspace_bytes(int64_t N, int64_t K);
int gemm_skinny_plan(int64_t N, int64_t K, int workers, int64_t* unit_begin_out, int* first_out, int* last_out);
int gemm_small_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, cudaStream_t s);
bool gemm_fused_supported(int mode, const float* A, const float* B, int64_t N, int64_t K, int64_t lda, int64_t ldb);
int gemm_fused_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, cudaStream_t s, int bn);

// Problems for which the single-kernel path (operand split inside the kernel, no workspace) is
// faster than split pass + tcgen05 kernel: so little work that launches and set-up dominate
// (measured on B200: 3.1 vs 9.9 us at 128^3, 5.2 vs 11.8 us at 256^3, 10.4 vs 11.7 us at 512^3).
static bool prefers_small_kernel(int64_t M, int64_t N, int64_t K) {
  if (M <= 16) return true;   // skinny: bound by one pass over B, which only the single-kernel path achieves
  return (double)M * (double)N * (double)K <= 520.0 * 520.0 * 520.0;
}

// ---------------------------------------------------------------------------------------
// Operand split
// ---------------------------------------------------------------------------------------
struct Bf16Kind {
  using elem = __nv_bfloat16;
  static constexpr int kElemBytes = 2;
  static constexpr int kBlockK = 64;  // elements per 128-byte row
  __device__ static __forceinline__ void split(float v, elem& hi, elem& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  __device__ static __forceinline__ elem zero() { return __float2bfloat16_rn(0.f); }
};
struct Tf32Kind {
  using elem = float;  // tf32 value held in an FP32 container (low 13 mantissa bits zero)
  static constexpr int kElemBytes = 4;
  static constexpr int kBlockK = 32;
  __device__ static __forceinline__ float rna(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
  }
  // The high part is rounded with integer arithmetic: half a tf32 unit added to the bit pattern, thirteen low bits
  // cleared. That is round-to-nearest with ties away from zero and equals cvt.rna.tf32.f32 on all 2^32 inputs but NaNs,
  // without the conversion pipe. A NaN may come out of it as a zero; the residual, NaN whenever v is NaN or infinite,
  // keeps the conversion instruction, so the NaN still reaches every product of the element.
  __device__ static __forceinline__ void split(float v, elem& hi, elem& lo) {
    hi = __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xFFFFE000u);
    lo = rna(v - hi);
  }
  __device__ static __forceinline__ elem zero() { return 0.f; }
};

// A[rows, cols] (ld = ldx) -> hi/lo [rows, colsP]; columns >= cols are written as zero. One thread converts
// kSplitRowElems<KIND> consecutive elements: 16 bytes per store for either kind.
template <class KIND>
constexpr int kSplitRowElems = 16 / KIND::kElemBytes;   // 8 (bf16) or 4 (tf32)

template <class KIND>
__device__ __forceinline__ void split_rows_body(const float* __restrict__ X, int64_t ldx, int cols, int colsP,
                                                typename KIND::elem* __restrict__ hi,
                                                typename KIND::elem* __restrict__ lo, int vec_ok, int row, int block_x) {
  using E = typename KIND::elem;
  constexpr int EPT = kSplitRowElems<KIND>;
  const int c0 = (block_x * 256 + (int)threadIdx.x) * EPT;
  if (c0 >= colsP) return;
  const float* xr = X + (int64_t)row * ldx;
  float v[EPT];
#pragma unroll
  for (int j = 0; j < EPT; ++j) v[j] = 0.f;
  if (vec_ok && c0 + EPT - 1 < cols) {
#pragma unroll
    for (int q = 0; q < EPT / 4; ++q) {
      const float4 t = ld_stream_f4(reinterpret_cast<const float4*>(xr + c0) + q);
      v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < EPT; ++j)
      if (c0 + j < cols) v[j] = xr[c0 + j];
  }
  __align__(16) E h[EPT];
  __align__(16) E l[EPT];
#pragma unroll
  for (int j = 0; j < EPT; ++j) KIND::split(v[j], h[j], l[j]);
  *reinterpret_cast<uint4*>(hi + (int64_t)row * colsP + c0) = *reinterpret_cast<uint4*>(h);
  *reinterpret_cast<uint4*>(lo + (int64_t)row * colsP + c0) = *reinterpret_cast<uint4*>(l);
}

template <class KIND>
__global__ void __launch_bounds__(256)
split_rows_kernel(const float* __restrict__ X, int64_t ldx, int rows, int cols, int colsP,
                  typename KIND::elem* __restrict__ hi, typename KIND::elem* __restrict__ lo, int vec_ok) {
  ptx::launch_dependents();   // a product kernel launched behind this grid may begin its set-up; it waits for the grid before it loads
  split_rows_body<KIND>(X, ldx, cols, colsP, hi, lo, vec_ok, (int)blockIdx.y, (int)blockIdx.x);
}

// B[K, N] (ld = ldb) -> transposed hi/lo [N, Kp]; k >= K written as zero.
// 256 threads (`tid` 0..255) transpose a kBlockK x 64 tile through `scratch` (kTransposeScratchBytes of shared
// memory); `sync()` is a barrier over exactly those threads. The scratch may be reused after a further sync().
constexpr int kTransposeScratchBytes = 2 * 64 * 66 * 2;   // the larger of the layouts below (bf16 padded: 16 896 bytes)

struct CtaSync {
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

template <class KIND, class SYNC>
__device__ __forceinline__ void split_transpose_body(const float* __restrict__ B, int64_t ldb, int K, int N, int Kp,
                                                     typename KIND::elem* __restrict__ hi,
                                                     typename KIND::elem* __restrict__ lo, int block_x, int block_y,
                                                     uint8_t* scratch, int tid, SYNC sync) {
  using E = typename KIND::elem;
  constexpr int TK = KIND::kBlockK;          // 64 (bf16) or 32 (tf32): 128 bytes of k per row
  constexpr int PAD = (KIND::kElemBytes == 2) ? 2 : 1;
  constexpr int ROW = TK + PAD;
  static_assert(2 * 64 * ROW * (int)sizeof(E) <= kTransposeScratchBytes, "transposition scratch too small");
  E* s_hi = reinterpret_cast<E*>(scratch);
  E* s_lo = s_hi + 64 * ROW;
  const int k0 = block_x * TK, n0 = block_y * 64;
  {
    const int nn = tid & 63, kr = tid >> 6;  // 4 k-rows per pass
#pragma unroll 4
    for (int p = 0; p < TK / 4; ++p) {
      const int k = k0 + p * 4 + kr, n = n0 + nn;
      float v = 0.f;
      if (k < K && n < N) v = B[(int64_t)k * ldb + n];
      E h, l;
      KIND::split(v, h, l);
      s_hi[nn * ROW + p * 4 + kr] = h;
      s_lo[nn * ROW + p * 4 + kr] = l;
    }
  }
  sync();
  {
    // each thread writes 4 bytes of k; 32 threads cover one 128-byte row; 8 rows per pass
    constexpr int EPT = 4 / KIND::kElemBytes;  // elements per thread (2 bf16 or 1 tf32)
    const int kk = (tid & 31) * EPT, nr = tid >> 5;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int nn = p * 8 + nr, n = n0 + nn;
      if (n < N && k0 + kk < Kp) {
        const int64_t o = (int64_t)n * Kp + k0 + kk;
        *reinterpret_cast<uint32_t*>(hi + o) = *reinterpret_cast<const uint32_t*>(&s_hi[nn * ROW + kk]);
        *reinterpret_cast<uint32_t*>(lo + o) = *reinterpret_cast<const uint32_t*>(&s_lo[nn * ROW + kk]);
      }
    }
  }
}

// bf16 form with 128-bit global accesses: a thread loads a 4 (k) x 4 (n) block of B with four 16-byte loads, packs
// four consecutive k of each column into 8 bytes and stores them to a [64 n][64 k] shared tile whose 8-byte chunks are
// XOR-swizzled with the column group (conflict-free on both sides); the tile leaves as 16-byte pieces of whole
// 128-byte k-rows. Needs B 16-byte aligned with ldb % 4 == 0; edges fall back to guarded scalar loads.
template <class SYNC>
__device__ __forceinline__ void split_transpose_bf16_vec(const float* __restrict__ B, int64_t ldb, int K, int N, int Kp,
                                                         __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                                         int block_x, int block_y, uint8_t* scratch, int tid, SYNC sync) {
  static_assert(2 * 64 * 64 * 2 <= kTransposeScratchBytes, "transposition scratch too small");
  __nv_bfloat16* t_hi = reinterpret_cast<__nv_bfloat16*>(scratch);   // 16-byte aligned: the scratch is
  __nv_bfloat16* t_lo = t_hi + 64 * 64;
  const int k0 = block_x * 64, n0 = block_y * 64;
  {
    const int n4 = tid & 15, kc = tid >> 4;
    const int n = n0 + 4 * n4;
    float v[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int k = k0 + 4 * kc + r;
      if (k < K && n + 3 < N) {
        const float4 t = ld_stream_f4(reinterpret_cast<const float4*>(B + (int64_t)k * ldb + n));
        v[r][0] = t.x; v[r][1] = t.y; v[r][2] = t.z; v[r][3] = t.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[r][j] = (k < K && n + j < N) ? B[(int64_t)k * ldb + n + j] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __align__(8) __nv_bfloat16 h[4];
      __align__(8) __nv_bfloat16 l[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) Bf16Kind::split(v[r][j], h[r], l[r]);
      const int at = (4 * n4 + j) * 64 + 4 * (kc ^ n4);
      *reinterpret_cast<uint2*>(t_hi + at) = *reinterpret_cast<uint2*>(h);
      *reinterpret_cast<uint2*>(t_lo + at) = *reinterpret_cast<uint2*>(l);
    }
  }
  sync();
#pragma unroll
  for (int q = tid; q < 512; q += 256) {
    const int nn = q >> 3, pr = q & 7;          // row of the tile, pair of 4-element chunks (2 pr, 2 pr + 1)
    const int group = (nn >> 2) & 15;
    const int at = nn * 64 + 8 * (pr ^ (group >> 1));
    uint4 a = *reinterpret_cast<const uint4*>(t_hi + at);
    uint4 b = *reinterpret_cast<const uint4*>(t_lo + at);
    if (group & 1) {                            // the two chunks of the pair sit in swapped order
      a = make_uint4(a.z, a.w, a.x, a.y);
      b = make_uint4(b.z, b.w, b.x, b.y);
    }
    const int n = n0 + nn;
    if (n < N) {
      const int64_t o = (int64_t)n * Kp + k0 + 8 * pr;
      *reinterpret_cast<uint4*>(hi + o) = a;
      *reinterpret_cast<uint4*>(lo + o) = b;
    }
  }
}

// One kBlockK x 64 tile of B by either form.
template <class KIND, class SYNC>
__device__ __forceinline__ void split_transpose_tile(const float* __restrict__ B, int64_t ldb, int K, int N, int Kp,
                                                     typename KIND::elem* __restrict__ hi, typename KIND::elem* __restrict__ lo,
                                                     int block_x, int block_y, int b_vec_ok, uint8_t* scratch, int tid, SYNC sync) {
  if constexpr (KIND::kElemBytes == 2) {
    if (b_vec_ok) {
      split_transpose_bf16_vec(B, ldb, K, N, Kp, hi, lo, block_x, block_y, scratch, tid, sync);
      return;
    }
  }
  split_transpose_body<KIND>(B, ldb, K, N, Kp, hi, lo, block_x, block_y, scratch, tid, sync);
}

template <class KIND>
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ B, int64_t ldb, int K, int N, int Kp,
                       typename KIND::elem* __restrict__ hi, typename KIND::elem* __restrict__ lo, int b_vec_ok,
                       int* __restrict__ zero_words, int zero_count) {
  ptx::launch_dependents();
  // the product kernel behind this grid claims split items from a counter and publishes flags: start them at zero
  if (zero_words != nullptr && blockIdx.x == 0 && blockIdx.y == 0)
    for (int i = threadIdx.x; i < zero_count; i += blockDim.x) zero_words[i] = 0;
  __shared__ __align__(16) uint8_t scratch[kTransposeScratchBytes];
  split_transpose_tile<KIND>(B, ldb, K, N, Kp, hi, lo, (int)blockIdx.x, (int)blockIdx.y, b_vec_ok, scratch, (int)threadIdx.x, CtaSync());
}

// Both splits in one launch (one launch less on the latency of small and medium problems): the first
// a_blocks CTAs split rows of A, the rest transpose-split tiles of B.
template <class KIND>
__global__ void __launch_bounds__(256)
split_both_kernel(const float* __restrict__ A, int64_t lda, int K, int Kp, typename KIND::elem* __restrict__ a_hi,
                  typename KIND::elem* __restrict__ a_lo, int a_vec_ok, int a_blocks_x, int a_blocks,
                  const float* __restrict__ B, int64_t ldb, int N, typename KIND::elem* __restrict__ b_hi,
                  typename KIND::elem* __restrict__ b_lo, int b_blocks_x, int b_vec_ok) {
  ptx::launch_dependents();   // the product kernel may begin its set-up; it waits for this grid before it loads
  const int id = blockIdx.x;
  if (id < a_blocks) {
    split_rows_body<KIND>(A, lda, K, Kp, a_hi, a_lo, a_vec_ok, id / a_blocks_x, id % a_blocks_x);
  } else {
    const int b = id - a_blocks;
    __shared__ __align__(16) uint8_t scratch[kTransposeScratchBytes];
    split_transpose_tile<KIND>(B, ldb, K, N, Kp, b_hi, b_lo, b % b_blocks_x, b / b_blocks_x, b_vec_ok, scratch, (int)threadIdx.x, CtaSync());
  }
}

// ---------------------------------------------------------------------------------------
// Tensor-core kernel
// ---------------------------------------------------------------------------------------
constexpr int kGemmThreads = 192;  // warp 0: TMA, warp 1: MMA + tensor-memory owner, warps 2-5: epilogue
constexpr int kTileRowBytes = 128; // one swizzle row = one k-block of either kind
constexpr int kDefaultGroupM = 8;  // m-tiles per raster group (L2 reuse of the B planes)

template <int CTAS, int BN>
struct GemmCfg {
  static constexpr int kBnLoad = BN / CTAS;                       // B rows this CTA loads
  static constexpr int kABytes = 128 * kTileRowBytes;             // one A plane tile
  static constexpr int kBBytes = kBnLoad * kTileRowBytes;         // one B plane tile
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;   // hi+lo of both
  static constexpr int kStages = (200 * 1024) / kStageBytes;      // ring depth
  static constexpr int kTmemCols = 2 * BN;                        // double-buffered accumulator
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
  static_assert(kStages >= 2, "ring too shallow");
  static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "tensor memory columns must be a power of two");
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first = g * group_m;
  const int gsize = min(group_m, tiles_m - first);
  const int r = t - g * per_group;
  tm = first + r % gsize;
  tn = r / gsize;
}

template <int KIND /*0 = bf16, 1 = tf32*/, int CTAS, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_x3_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
               const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
               float* __restrict__ C, int64_t ldc, int M, int N, int num_kb, int tiles_m, int tiles_n,
               int group_m, int c_vec_ok, int* __restrict__ status) {
  using Cfg = GemmCfg<CTAS, BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBlockKElems = (KIND == 0) ? 64 : 32;
  constexpr uint32_t kIdesc = ptx::umma_idesc(KIND == 0 ? 1 : 2, 128 * CTAS, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  uint8_t* bar_ptr = tiles_ptr + kStages * Cfg::kStageBytes;
  const uint32_t bar_addr = tiles_addr + kStages * Cfg::kStageBytes;
  // barrier block layout (8-byte slots): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_addr + 8u * s; };
  auto empty_bar = [&](int s) { return bar_addr + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_addr + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_addr + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = (CTAS == 2) ? ptx::cluster_ctarank() : 0u;
  const int unit = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;        // tile worker index
  const int num_units = (CTAS == 2) ? (gridDim.x >> 1) : gridDim.x;
  const int num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4 * CTAS);
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
    ptx::tma_prefetch_desc(&tm_a_hi);
    ptx::tma_prefetch_desc(&tm_a_lo);
    ptx::tma_prefetch_desc(&tm_b_hi);
    ptx::tma_prefetch_desc(&tm_b_lo);
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTAS>(smem_u32(tmem_holder), Cfg::kTmemCols);
    ptx::tmem_relinquish<CTAS>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // Everything above touched only this CTA's shared and tensor memory; the operand planes are written by
  // the kernel before this one in the stream.
  ptx::grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------- TMA producer --------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t leader_full0 = (CTAS == 2) ? ptx::map_to_cta(full_bar(0), 0) : full_bar(0);
      for (int t = unit; t < num_tiles && ok; t += num_units) {
        int tm, tn;
        tile_coords(t, tiles_m, tiles_n, group_m, tm, tn);
        const int row_a = tm * (128 * CTAS) + (int)rank * 128;
        const int row_b = tn * BN + (int)rank * Cfg::kBnLoad;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            atomicExch(status, 0x100 | (int)(blockIdx.x & 0xff));
            ok = false;
            break;
          }
          const uint32_t sa_hi = tiles_addr + stage * Cfg::kStageBytes;
          const uint32_t sa_lo = sa_hi + Cfg::kABytes;
          const uint32_t sb_hi = sa_lo + Cfg::kABytes;
          const uint32_t sb_lo = sb_hi + Cfg::kBBytes;
          const int kx = kb * kBlockKElems;
          if constexpr (CTAS == 1) {
            ptx::mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
            ptx::tma_load_2d(sa_hi, &tm_a_hi, kx, row_a, full_bar(stage));
            ptx::tma_load_2d(sa_lo, &tm_a_lo, kx, row_a, full_bar(stage));
            ptx::tma_load_2d(sb_hi, &tm_b_hi, kx, row_b, full_bar(stage));
            ptx::tma_load_2d(sb_lo, &tm_b_lo, kx, row_b, full_bar(stage));
          } else {
            // Both CTAs' loads are counted on the leader CTA's barrier; the leader posts the
            // byte count of the pair.
            const uint32_t fb = leader_full0 + 8u * stage;
            if (rank == 0) ptx::mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
            ptx::tma_load_2d_pair(sa_hi, &tm_a_hi, kx, row_a, fb);
            ptx::tma_load_2d_pair(sa_lo, &tm_a_lo, kx, row_a, fb);
            ptx::tma_load_2d_pair(sb_hi, &tm_b_hi, kx, row_b, fb);
            ptx::tma_load_2d_pair(sb_lo, &tm_b_lo, kx, row_b, fb);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------
    // All 32 lanes walk the loop and wait on the barriers; an elected lane issues, so that the descriptors stay in
    // uniform registers (issued from a one-lane branch they go through vector registers, and a 128 x 64 tile's twelve
    // products of a k-block take no longer to execute than that takes to issue).
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int t = unit; t < num_tiles && ok; t += num_units, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag))) {
          if (lane == 0) atomicExch(status, 0x200 | (int)(blockIdx.x & 0xff));
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(full_bar(stage), phase, abort_flag))) {
            if (lane == 0) atomicExch(status, 0x300 | (int)(blockIdx.x & 0xff));
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa_hi = tiles_addr + stage * Cfg::kStageBytes;
          const uint32_t sa_lo = sa_hi + Cfg::kABytes;
          const uint32_t sb_hi = sa_lo + Cfg::kABytes;
          const uint32_t sb_lo = sb_hi + Cfg::kBBytes;
          ptx::umma_x3_kblock<KIND, CTAS>(d_tmem, ptx::desc_lo_sw128(sa_hi), ptx::desc_lo_sw128(sa_lo), ptx::desc_lo_sw128(sb_hi),
                                          ptx::desc_lo_sw128(sb_lo), kIdesc, kb != 0 ? 1u : 0u);
          ptx::umma_commit_elected<CTAS>(empty_bar(stage));  // frees this ring slot once the MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit_elected<CTAS>(tfull_bar(acc));  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue ------------------------------------------
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, +32) belong to this warp
    const uint32_t leader_tempty0 = (CTAS == 2) ? ptx::map_to_cta(tempty_bar(0), 0) : tempty_bar(0);
    int iter = 0;
    for (int t = unit; t < num_tiles; t += num_units, ++iter) {
      const int acc = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, group_m, tm, tn);
      const bool ready = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {  // leave together: the loads below are warp-wide
        if (lane == 0) atomicExch(status, 0x400 | (int)(blockIdx.x & 0xff));
        break;
      }
      ptx::tc_fence_after();
      const int row = tm * (128 * CTAS) + (int)rank * 128 + quarter * 32 + lane;
      const int col0 = tn * BN;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      float* crow = C + (int64_t)row * ldc + col0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
        if (row < M) {
          if (c_vec_ok && col0 + c * 32 + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(crow + c * 32 + 4 * j) =
                  make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + c * 32 + j < N) crow[c * 32 + j] = __uint_as_float(r[j]);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2)
          ptx::mbar_arrive_cluster(leader_tempty0 + 8u * acc);
        else
          ptx::mbar_arrive(tempty_bar(acc));
      }
    }
  }

  // ------------------------------- teardown --------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out: give copies already in flight time to land before the CTA's shared
    // memory and tensor memory are released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (CTAS == 2) ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CTAS>(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Stream kernel: CTA-pair tiles 256 rows tall and 64..256 columns wide from a host-made schedule,
// with the split of A running inside the kernel beside the products.
//
//  * Schedule. A persistent grid of W CTA pairs walks `rounds` rounds; in round j pair w multiplies
//    the tile entry[j * W + w] (0 = nothing). The host cuts every 256-row band of C into pieces of
//    different widths (multiples of 32 columns) so that the pairs finish together: with 128 tiles of
//    256 x 256 on 74 pairs a uniform walk costs two full rounds for 1.73 rounds of work, the cut costs
//    1.75. Tile width changes nothing in the arithmetic of an output element (same k order).
//    rounds == 0: tiles come from the raster formula of gemm_x3_kernel (large problems, where the
//    last round hardly matters).
//  * Split of A. Eight more warps per CTA turn FP32 rows of A into the hi / lo planes while the
//    products run: work items of one band (256 rows) x 128 columns of k are claimed from a counter in
//    the workspace, converted, and published through one flag per item (release store); the thread
//    that issues the TMA loads reads the flag (acquire) before it loads the first k-block of an item,
//    then orders that against the TMA unit's reads (fence.proxy.async). Items are numbered in the
//    order the tiles need them: the bands of the first round k-chunk by k-chunk, then the later bands.
//    Whoever claims an item completes it without waiting for anything, so the flags never deadlock;
//    the wait on a flag is bounded like every other wait here. B's planes are written by the
//    transposing split kernel before this kernel (which also clears counter and flags).
// ---------------------------------------------------------------------------------------
constexpr int kStreamThreads = 192 + 256;     // roles of gemm_x3_kernel + 8 split warps
constexpr int kSchedMaxEntries = 640;
constexpr int kSplitItemK = 128;              // k-extent of one split item

struct TileSchedule {
  uint32_t rounds;                            // 0: raster formula
  uint32_t workers;                           // CTA pairs = entries per round
  uint32_t entry[kSchedMaxEntries];           // band | (col0 / 32) << 12 | (width / 32) << 24
};

struct SplitWork {
  const float* A;
  const float* B;
  int64_t lda, ldb;
  void* a_hi;
  void* a_lo;
  void* b_hi;
  void* b_lo;
  int* ctrl;          // [0] claim counter, [1] finished items, then one flag per item: A's (band, chunk) flags at
                      // 2 + band * chunks + chunk, B's (block, chunk) flags `b_flags` words further on; all zero at launch
  int M, N, K, Kp;
  int chunks;         // kSplitItemK-wide chunks of k
  int a_bands;        // 256-row bands of A split in this kernel (0: A's planes are already there)
  int b_blocks;       // 256-column blocks of B split in this kernel (0: B's planes are already there)
  int b_flags;        // offset of B's flags behind A's
  int ga, gb;         // bands of A / blocks of B the first round needs: their items come first, chunk by chunk
  int items;          // (a_bands + b_blocks) * chunks
  int a_vec_ok;       // A 16-byte aligned and lda % 4 == 0
  int b_vec_ok;       // the same for B
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acquire_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta_shared(uint32_t addr) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(uint32_t addr, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bar_sync_named(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// `count` units numbered in groups of `group`, chunk-major inside a group: j -> (unit, chunk).
__device__ __forceinline__ void grouped_coords(int j, int count, int group, int chunks, int& unit, int& chunk) {
  const int per_group = group * chunks;
  const int groups = (count + group - 1) / group;
  int g = j / per_group;
  if (g >= groups) g = groups - 1;
  const int first = g * group;
  const int gsize = min(group, count - first);
  const int r = j - g * per_group;
  chunk = r / gsize;
  unit = first + r % gsize;
}

// Item number -> (operand, unit, chunk), in the order the tiles need them: first, chunk by chunk, the `ga` bands of A
// and the `gb` blocks of B the first round touches; then the other blocks of B (the walk crosses all columns before
// it leaves its first bands); then the other bands of A.
__device__ __forceinline__ void split_item_coords(const SplitWork& w, int item, bool& is_b, int& unit, int& chunk) {
  const int first = (w.ga + w.gb) * w.chunks;
  if (item < first) {
    chunk = item / (w.ga + w.gb);
    const int r = item % (w.ga + w.gb);
    is_b = r >= w.ga;
    unit = is_b ? r - w.ga : r;
    return;
  }
  item -= first;
  const int rest_b = (w.b_blocks - w.gb) * w.chunks;
  if (item < rest_b) {
    is_b = true;
    grouped_coords(item, w.b_blocks - w.gb, max(w.gb, 1), w.chunks, unit, chunk);
    unit += w.gb;
    return;
  }
  item -= rest_b;
  is_b = false;
  grouped_coords(item, w.a_bands - w.ga, max(w.ga, 1), w.chunks, unit, chunk);
  unit += w.ga;
}

// One item: rows [band * 256, +256) x k [chunk * 128, +128) of A -> both planes. Warp `sw` of the eight takes rows
// sw, sw + 8, ...; a lane converts four consecutive k of a row per step, eight rows in flight.
template <class KIND>
__device__ __forceinline__ void split_item(const SplitWork& w, int band, int chunk, int sw, int lane) {
  using E = typename KIND::elem;
  E* __restrict__ hi = static_cast<E*>(w.a_hi);
  E* __restrict__ lo = static_cast<E*>(w.a_lo);
  const int k = chunk * kSplitItemK + lane * 4;
  if (k >= w.Kp) return;
  const int row0 = band * 256 + sw;
  const bool full_k = k + 3 < w.K;
#pragma unroll 1
  for (int batch = 0; batch < 4; ++batch) {
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int row = row0 + (batch * 8 + j) * 8;
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < w.M) {
        const float* src = w.A + (int64_t)row * w.lda + k;
        if (full_k && w.a_vec_ok) {
          v[j] = ld_stream_f4(reinterpret_cast<const float4*>(src));
        } else {
          if (k < w.K) v[j].x = src[0];
          if (k + 1 < w.K) v[j].y = src[1];
          if (k + 2 < w.K) v[j].z = src[2];
          if (k + 3 < w.K) v[j].w = src[3];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int row = row0 + (batch * 8 + j) * 8;
      if (row >= w.M) continue;
      __align__(16) E h[4];
      __align__(16) E l[4];
      KIND::split(v[j].x, h[0], l[0]);
      KIND::split(v[j].y, h[1], l[1]);
      KIND::split(v[j].z, h[2], l[2]);
      KIND::split(v[j].w, h[3], l[3]);
      const int64_t o = (int64_t)row * w.Kp + k;
      if constexpr (KIND::kElemBytes == 2) {
        *reinterpret_cast<uint2*>(hi + o) = *reinterpret_cast<uint2*>(h);
        *reinterpret_cast<uint2*>(lo + o) = *reinterpret_cast<uint2*>(l);
      } else {
        *reinterpret_cast<uint4*>(hi + o) = *reinterpret_cast<uint4*>(h);
        *reinterpret_cast<uint4*>(lo + o) = *reinterpret_cast<uint4*>(l);
      }
    }
  }
}

// One item of B: columns [block * 256, +256) x k [chunk * 128, +128) -> both transposed planes, as 64-column x
// kBlockK tiles through the shared-memory scratch. All 256 split threads take part; `sync` is their barrier.
template <class KIND, class SYNC>
__device__ __forceinline__ void split_item_b(const SplitWork& w, int block, int chunk, uint8_t* scratch, int tid, SYNC sync) {
  using E = typename KIND::elem;
  constexpr int kTilesK = kSplitItemK / KIND::kBlockK;
  for (int ny = 0; ny < 4; ++ny) {
    const int block_y = block * 4 + ny;
    if (block_y * 64 >= w.N) break;
    for (int kx = 0; kx < kTilesK; ++kx) {
      const int block_x = chunk * kTilesK + kx;
      if (block_x * KIND::kBlockK >= w.Kp) break;
      split_transpose_tile<KIND>(w.B, w.ldb, w.K, w.N, w.Kp, static_cast<E*>(w.b_hi), static_cast<E*>(w.b_lo), block_x, block_y,
                                 w.b_vec_ok, scratch, tid, sync);
      sync();   // the scratch is free again
    }
  }
}

template <int KIND /*0 = bf16, 1 = tf32*/>
__global__ void __launch_bounds__(kStreamThreads, 1)
gemm_x3_stream_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                      const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                      const __grid_constant__ CUtensorMap tm_b16_hi, const __grid_constant__ CUtensorMap tm_b16_lo,
                      float* __restrict__ C, int64_t ldc, int M, int N, int num_kb, int tiles_m, int tiles_n,
                      int group_m, int c_vec_ok, int* __restrict__ status, const __grid_constant__ SplitWork sw,
                      const __grid_constant__ TileSchedule sched) {
  using Cfg = GemmCfg<2, 256>;
  using SplitKind = typename std::conditional<KIND == 0, Bf16Kind, Tf32Kind>::type;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBlockKElems = (KIND == 0) ? 64 : 32;
  constexpr int kKbPerItem = kSplitItemK / kBlockKElems;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  uint8_t* bar_ptr = tiles_ptr + kStages * Cfg::kStageBytes;
  const uint32_t bar_addr = tiles_addr + kStages * Cfg::kStageBytes;
  auto full_bar = [&](int s) { return bar_addr + 8u * s; };
  auto empty_bar = [&](int s) { return bar_addr + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_addr + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_addr + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * kStages + 4) + 8);
  volatile int* claimed = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * kStages + 4) + 16);   // two slots
  uint8_t* transpose_scratch = bar_ptr + Cfg::kBarrierBytes;   // kTransposeScratchBytes, 16-byte aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int unit = blockIdx.x >> 1;
  const int num_units = gridDim.x >> 1;
  const int num_tiles = tiles_m * tiles_n;
  const int steps = sched.rounds ? (int)sched.rounds : (num_tiles + num_units - 1) / num_units;

  // Tile of this pair in step j: band (256 rows), first column, width; false when the pair has nothing in that step.
  auto tile_of = [&](int j, int& band, int& col0, int& width) -> bool {
    if (sched.rounds) {
      const uint32_t e = sched.entry[j * (int)sched.workers + unit];
      if (e == 0) return false;
      band = (int)(e & 0xfffu);
      col0 = (int)((e >> 12) & 0xfffu) * 32;
      width = (int)(e >> 24) * 32;
      return true;
    }
    const int t = unit + j * num_units;
    if (t >= num_tiles) return false;
    int tn;
    tile_coords(t, tiles_m, tiles_n, group_m, band, tn);
    col0 = tn * 256;
    width = 256;
    return true;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
    ptx::tma_prefetch_desc(&tm_a_hi);
    ptx::tma_prefetch_desc(&tm_a_lo);
    ptx::tma_prefetch_desc(&tm_b_hi);
    ptx::tma_prefetch_desc(&tm_b_lo);
    ptx::tma_prefetch_desc(&tm_b16_hi);
    ptx::tma_prefetch_desc(&tm_b16_lo);
  }
  if (warp == 1) {
    ptx::tmem_alloc<2>(smem_u32(tmem_holder), Cfg::kTmemCols);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // The kernel before this one in the stream writes B's planes and clears counter and flags.
  ptx::grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------- TMA producer --------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool all_split = sw.items == 0;   // once every item is finished no flag needs looking at any more
      int boundary = 0;
      const uint32_t leader_full0 = ptx::map_to_cta(full_bar(0), 0);
      for (int j = 0; j < steps && ok; ++j) {
        int band, col0, width;
        if (!tile_of(j, band, col0, width)) continue;
        const int half = width >> 1;
        const int row_a = band * 256 + (int)rank * 128;
        const int row_b = col0 + (int)rank * half;
        const uint32_t stage_bytes = 2u * (uint32_t)Cfg::kABytes + 2u * (uint32_t)half * kTileRowBytes;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!all_split && (kb % kKbPerItem) == 0) {
            // this k-block reads rows of the planes that are converted inside this kernel: wait for their items.
            // Once every item of the kernel is finished (looked at every fourth time) no flag matters any more.
            if ((boundary++ & 3) == 0 && ld_acquire_gpu(sw.ctrl + 1) == sw.items) {
              all_split = true;
            } else {
              const int chunk = kb / kKbPerItem;
              const int* flags[3];
              int n_flags = 0;
              if (sw.a_bands) flags[n_flags++] = sw.ctrl + 2 + band * sw.chunks + chunk;
              if (sw.b_blocks && row_b < N) {
                const int first = row_b >> 8, last = min(row_b + half - 1, N - 1) >> 8;   // this CTA's rows of B's planes
                flags[n_flags++] = sw.ctrl + 2 + sw.b_flags + first * sw.chunks + chunk;
                if (last != first) flags[n_flags++] = sw.ctrl + 2 + sw.b_flags + last * sw.chunks + chunk;
              }
              for (int f = 0; f < n_flags && ok; ++f) {
                if (ld_acquire_gpu(flags[f]) != 0) continue;
                const long long start = clock64();
                while (ld_acquire_gpu(flags[f]) == 0) {
                  if (*abort_flag || clock64() - start > ptx::kWaitBudgetCycles) {
                    *abort_flag = 1;
                    atomicExch(status, 0x500 | (int)(blockIdx.x & 0xff));
                    ok = false;
                    break;
                  }
                  __nanosleep(64);
                }
              }
              if (!ok) break;
            }
            fence_proxy_async_all();   // what the split warps wrote is ordered before this thread's TMA reads
          }
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            atomicExch(status, 0x100 | (int)(blockIdx.x & 0xff));
            ok = false;
            break;
          }
          const uint32_t sa_hi = tiles_addr + stage * Cfg::kStageBytes;
          const uint32_t sa_lo = sa_hi + Cfg::kABytes;
          const uint32_t sb_hi = sa_lo + Cfg::kABytes;
          const uint32_t sb_lo = sb_hi + Cfg::kBBytes;
          const int kx = kb * kBlockKElems;
          const uint32_t fb = leader_full0 + 8u * stage;
          if (rank == 0) ptx::mbar_expect_tx(full_bar(stage), 2u * stage_bytes);
          ptx::tma_load_2d_pair(sa_hi, &tm_a_hi, kx, row_a, fb);
          ptx::tma_load_2d_pair(sa_lo, &tm_a_lo, kx, row_a, fb);
          if (half == 128) {
            ptx::tma_load_2d_pair(sb_hi, &tm_b_hi, kx, row_b, fb);
            ptx::tma_load_2d_pair(sb_lo, &tm_b_lo, kx, row_b, fb);
          } else {
            for (int r = 0; r < half; r += 16) {
              ptx::tma_load_2d_pair(sb_hi + (uint32_t)r * kTileRowBytes, &tm_b16_hi, kx, row_b + r, fb);
              ptx::tma_load_2d_pair(sb_lo + (uint32_t)r * kTileRowBytes, &tm_b16_lo, kx, row_b + r, fb);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------
    // All 32 lanes of the leader CTA's warp walk the loop and wait on the barriers; an elected lane issues. With
    // uniform control flow and operands the descriptors stay in uniform registers, and the twelve products of a
    // k-block cost the warp a few dozen instructions on a scheduler it shares with split and epilogue warps.
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int j = 0; j < steps && ok; ++j) {
        int band, col0, width;
        if (!tile_of(j, band, col0, width)) continue;
        const uint32_t idesc = ptx::umma_idesc(KIND == 0 ? 1 : 2, 256, width);
        const int acc = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        ++iter;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag))) {
          if (lane == 0) atomicExch(status, 0x200 | (int)(blockIdx.x & 0xff));
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(full_bar(stage), phase, abort_flag))) {
            if (lane == 0) atomicExch(status, 0x300 | (int)(blockIdx.x & 0xff));
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa_hi = tiles_addr + stage * Cfg::kStageBytes;
          const uint32_t sa_lo = sa_hi + Cfg::kABytes;
          const uint32_t sb_hi = sa_lo + Cfg::kABytes;
          const uint32_t sb_lo = sb_hi + Cfg::kBBytes;
          ptx::umma_x3_kblock<KIND, 2>(d_tmem, ptx::desc_lo_sw128(sa_hi), ptx::desc_lo_sw128(sa_lo), ptx::desc_lo_sw128(sb_hi),
                                         ptx::desc_lo_sw128(sb_lo), idesc, kb != 0 ? 1u : 0u);
          ptx::umma_commit_elected<2>(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit_elected<2>(tfull_bar(acc));
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------- epilogue ------------------------------------------
    const int quarter = warp & 3;
    const uint32_t leader_tempty0 = ptx::map_to_cta(tempty_bar(0), 0);
    int iter = 0;
    for (int j = 0; j < steps; ++j) {
      int band, col0, width;
      if (!tile_of(j, band, col0, width)) continue;
      const int acc = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      ++iter;
      const bool ready = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) atomicExch(status, 0x400 | (int)(blockIdx.x & 0xff));
        break;
      }
      ptx::tc_fence_after();
      const int row = band * 256 + (int)rank * 128 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
      float* crow = C + (int64_t)row * ldc + col0;
#pragma unroll 1
      for (int c = 0; c < width / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(t_row + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
        if (row < M) {
          if (c_vec_ok && col0 + c * 32 + 32 <= N) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(crow + c * 32 + 4 * q) =
                  make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (col0 + c * 32 + q < N) crow[c * 32 + q] = __uint_as_float(r[q]);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(leader_tempty0 + 8u * acc);
    }
  } else {
    // ------------------------------- split of A and B -----------------------------------
    const int st = (int)threadIdx.x - 192;      // 0..255
    const int swarp = st >> 5;
    int parity = 0;
    while (sw.items) {
      if (st == 0) claimed[parity] = atomicAdd(sw.ctrl, 1);
      bar_sync_named(1, 256);
      const int item = claimed[parity];
      parity ^= 1;
      if (item >= sw.items) break;
      bool is_b;
      int unit, chunk;
      split_item_coords(sw, item, is_b, unit, chunk);
      auto sync = [] { bar_sync_named(1, 256); };
      if (is_b)
        split_item_b<SplitKind>(sw, unit, chunk, transpose_scratch, st, sync);
      else
        split_item<SplitKind>(sw, unit, chunk, swarp, lane);
      __threadfence();            // this thread's plane stores are visible device-wide ...
      fence_proxy_async_all();    // ... also to reads made by the TMA unit
      bar_sync_named(1, 256);
      if (st == 0) {
        st_release_gpu(sw.ctrl + 2 + (is_b ? sw.b_flags : 0) + unit * sw.chunks + chunk, 1);
        red_release_gpu_add(sw.ctrl + 1, 1);
      }
    }
  }

  // ------------------------------- teardown --------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<2>(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map of a K-major plane [rows, Kp] of `elem_bytes` elements; box = 128 bytes x box_rows.
static int make_plane_map(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t K,
                          int64_t Kp, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  DTN_REQUIRE(enc != nullptr, DTN_ERR_CUDA, "gemm: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)Kp * (cuuint64_t)elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(kTileRowBytes / elem_bytes), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DTN_OK;
}

// Tile-variant selection of dtn_gemm_set_variant: one value per host thread (a thread that pins a
// variant for a measurement does not change what other threads' calls run).
static thread_local int g_gemm_variant = 0;

// Tile width forced on the fused-split variant (DTN_GEMM_FUSED_BN), read once.
static int fused_bn_override() {
  static const int value = [] {
    const char* text = getenv("DTN_GEMM_FUSED_BN");
    return text ? atoi(text) : 0;
  }();
  return value;
}

// m-tiles per raster group. DTN_GEMM_GROUP_M overrides the default for experiments.
static int raster_group_m() {
  static int value = [] {
    const char* text = getenv("DTN_GEMM_GROUP_M");
    const int parsed = text ? atoi(text) : 0;
    return parsed > 0 && parsed <= 64 ? parsed : kDefaultGroupM;
  }();
  return value;
}

// Workspace layout: Bt_hi, Bt_lo, A_hi, A_lo. The B planes come first so that their place depends on
// (mode, N, K) only: a caller that walks row blocks of A of any heights against one B splits B once.
// Tuning aids of the stream kernel, read once: DTN_GEMM_STREAM_SPLIT = mask of the operands it may split itself
// (1 = A, 2 = B; default: decided per shape), DTN_GEMM_TABLE = 0 keeps the plain walk whatever the shape.
static int stream_split_override() {
  static const int value = [] {
    const char* text = getenv("DTN_GEMM_STREAM_SPLIT");
    return text ? atoi(text) : -1;
  }();
  return value;
}
static bool table_allowed() {
  static const bool value = [] {
    const char* text = getenv("DTN_GEMM_TABLE");
    return !(text && text[0] == '0');
  }();
  return value;
}

struct PlaneLayout {
  int64_t Kp;
  size_t a_plane, b_plane;  // bytes of one plane, rounded to 1024
  size_t ctrl_bytes;        // claim counter and item flags of the in-kernel split of A, after the planes
  int bands, blocks, chunks; // 256-row bands of A, 256-column blocks of B, kSplitItemK-wide chunks of k: one flag per
                             // (band, chunk) and per (block, chunk)
  size_t total;
  size_t planes() const { return 2 * a_plane + 2 * b_plane; }
  size_t ctrl() const { return planes(); }
  size_t b_hi() const { return 0; }
  size_t b_lo() const { return b_plane; }
  size_t a_hi() const { return 2 * b_plane; }
  size_t a_lo() const { return 2 * b_plane + a_plane; }
};
static PlaneLayout plane_layout(int mode, int64_t M, int64_t N, int64_t K) {
  PlaneLayout L;
  const int eb = (mode == DTN_GEMM_BF16X3) ? 2 : 4;
  const int bk = kTileRowBytes / eb;
  L.Kp = (K + bk - 1) / bk * bk;
  auto round1k = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
  L.a_plane = round1k((size_t)M * L.Kp * eb);
  L.b_plane = round1k((size_t)N * L.Kp * eb);
  L.bands = (int)((M + 255) / 256);
  L.blocks = (int)((N + 255) / 256);
  L.chunks = (int)((L.Kp + kSplitItemK - 1) / kSplitItemK);
  L.ctrl_bytes = round1k(sizeof(int) * (2 + ((size_t)L.bands + L.blocks) * L.chunks));
  L.total = L.planes() + L.ctrl_bytes;
  return L;
}

template <int KIND, int CTAS, int BN>
static int launch_tc(const void* a_hi, const void* a_lo, const void* b_hi, const void* b_lo, float* C,
                     int64_t M, int64_t N, int64_t K, int64_t Kp, int64_t ldc, cudaStream_t s,
                     int* status_word = nullptr) {
  using Cfg = GemmCfg<CTAS, BN>;
  constexpr int eb = (KIND == 0) ? 2 : 4;
  CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
  int rc;
  if ((rc = make_plane_map(&ma_hi, a_hi, eb, M, K, Kp, 128))) return rc;
  if ((rc = make_plane_map(&ma_lo, a_lo, eb, M, K, Kp, 128))) return rc;
  if ((rc = make_plane_map(&mb_hi, b_hi, eb, N, K, Kp, Cfg::kBnLoad))) return rc;
  if ((rc = make_plane_map(&mb_lo, b_lo, eb, N, K, Kp, Cfg::kBnLoad))) return rc;

  auto kernel = gemm_x3_kernel<KIND, CTAS, BN>;
  // The attribute is per device; set it on every device the first time it is seen.
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_dev = dev;
  }

  int* status = status_word ? status_word : device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gemm: could not allocate the device status word");
  const int bm = 128 * CTAS;
  const int tiles_m = (int)((M + bm - 1) / bm), tiles_n = (int)((N + BN - 1) / BN);
  const int num_kb = (int)(Kp / (kTileRowBytes / eb));
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
  const int sms = sm_count();
  int units = CTAS == 2 ? sms / 2 : sms;
  if (num_tiles < units) units = (int)num_tiles;
  const int c_vec_ok = aligned_to(C, 16) && (ldc % 4 == 0);

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * CTAS));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // overlap this kernel's set-up with the split kernel
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  DTN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ma_hi, ma_lo, mb_hi, mb_lo, C, ldc, (int)M, (int)N, num_kb,
                                    tiles_m, tiles_n, raster_group_m(), c_vec_ok, status));
  return DTN_OK;
}

template <class KIND>
static int run_split(const float* A, const float* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                     const PlaneLayout& L, uint8_t* ws, cudaStream_t s, bool do_a = true, bool do_b = true,
                     bool zero_ctrl = false) {
  using E = typename KIND::elem;
  E* a_hi = reinterpret_cast<E*>(ws + L.a_hi());
  E* a_lo = reinterpret_cast<E*>(ws + L.a_lo());
  E* b_hi = reinterpret_cast<E*>(ws + L.b_hi());
  E* b_lo = reinterpret_cast<E*>(ws + L.b_lo());
  {
    const int64_t ax = (L.Kp / kSplitRowElems<KIND> + 255) / 256, a_blocks = ax * M;
    const int b_vec_ok = aligned_to(B, 16) && (ldb % 4 == 0);
    const int64_t bx = L.Kp / KIND::kBlockK, b_blocks = bx * ((N + 63) / 64);
    // One launch for both operands saves a launch on small and medium problems; from about 4096^2 elements per operand
    // two launches are faster (8192^3: 84 + 102 us against 207 us in one: the row split then runs at the occupancy of
    // its own registers, not at that of the transposing split's shared-memory tile).
    const bool one_launch = (double)M * (double)K + (double)K * (double)N < 2.0 * 4096.0 * 4096.0;
    if (do_a && do_b && !zero_ctrl && one_launch && a_blocks + b_blocks < (int64_t)2000000000) {
      const int vec_ok = aligned_to(A, 16) && (lda % 4 == 0);
      split_both_kernel<KIND><<<(unsigned)(a_blocks + b_blocks), 256, 0, s>>>(A, lda, (int)K, (int)L.Kp, a_hi, a_lo, vec_ok,
                                                                             (int)ax, (int)a_blocks, B, ldb, (int)N, b_hi,
                                                                             b_lo, (int)bx, b_vec_ok);
      DTN_LAUNCH_CHECK("split_both_kernel");
      return DTN_OK;
    }
  }
  if (do_a) {
    const int vec_ok = aligned_to(A, 16) && (lda % 4 == 0);
    dim3 grid((unsigned)((L.Kp / kSplitRowElems<KIND> + 255) / 256), (unsigned)M);
    DTN_REQUIRE(M <= 65535 * 1024LL, DTN_ERR_UNSUPPORTED, "gemm: M too large");
    // grid.y is limited to 65535 rows per launch
    for (int64_t r0 = 0; r0 < M; r0 += 65535) {
      const int rows = (int)((M - r0) < 65535 ? (M - r0) : 65535);
      grid.y = (unsigned)rows;
      split_rows_kernel<KIND><<<grid, 256, 0, s>>>(A + r0 * lda, lda, rows, (int)K, (int)L.Kp, a_hi + r0 * L.Kp,
                                                   a_lo + r0 * L.Kp, vec_ok);
      DTN_LAUNCH_CHECK("split_rows_kernel");
    }
  }
  if (do_b) {
    const int64_t ny = (N + 63) / 64;
    for (int64_t y0 = 0; y0 < ny; y0 += 65535) {
      const int cnt = (int)((ny - y0) < 65535 ? (ny - y0) : 65535);
      dim3 grid((unsigned)(L.Kp / KIND::kBlockK), (unsigned)cnt);
      const int64_t n_off = y0 * 64;
      const bool zero_here = zero_ctrl && y0 == 0;
      split_transpose_kernel<KIND><<<grid, 256, 0, s>>>(B + n_off, ldb, (int)K, (int)(N - n_off), (int)L.Kp,
                                                        b_hi + n_off * L.Kp, b_lo + n_off * L.Kp,
                                                        aligned_to(B + n_off, 16) && (ldb % 4 == 0),
                                                        zero_here ? reinterpret_cast<int*>(ws + L.ctrl()) : nullptr,
                                                        zero_here ? 2 + (L.bands + L.blocks) * L.chunks : 0);
      DTN_LAUNCH_CHECK("split_transpose_kernel");
    }
  }
  return DTN_OK;
}

// ---------------------------------------------------------------------------------------
// Tile schedule of the stream kernel
// ---------------------------------------------------------------------------------------
constexpr int kTileFixedCost = 12;   // what a tile costs beyond its products, in columns (barrier hand-offs, first loads)

struct ScheduleChoice {
  bool table = false;        // false: raster formula
  int first_round_bands = 0; // bands of A the first round touches (table mode)
  int first_round_blocks = 0; // 256-column blocks of B the first round touches (table mode)
  double makespan = 0, uniform = 0;
  TileSchedule sched;
};

// What a tile of `units` 32-column units costs a CTA pair, in columns of a 256-wide tile. Measured on B200 (148 tiles
// of one width on 74 pairs, K = 4096, bf16x3; tf32x3 has the same shape): 256, 224 and 192 columns all take the time
// of 256, 160 takes 0.775 of it, 128 takes 0.56, 96 and 64 hardly less (0.545, 0.51): the products of a tile between
// 129 and 256 columns cost the same, and below 128 columns the shared-memory reads of the A tile, which do not shrink
// with the width, set the pace. So only 256-, 128- and 64-wide pieces are worth cutting.
static double tile_cost(int units) {
  static const double relative[9] = {0.0, 0.50, 0.51, 0.545, 0.56, 0.775, 0.97, 1.0, 1.0};
  return 256.0 * relative[std::max(0, std::min(units, 8))] + kTileFixedCost;
}

// Cuts each of `bands` bands of `units` 32-column units into pieces of `piece` units (the last piece of a band takes
// what is left); of the full pieces, `halved` (spread evenly over all of them, in band order) become two halves.
// Appends band | first unit << 12 | width in units << 24.
static bool cut_bands(int bands, int units, int piece, int halved, std::vector<uint32_t>* tiles) {
  tiles->clear();
  const int full_per_band = units / piece;
  const int64_t full_total = (int64_t)bands * full_per_band;
  if (halved > full_total || (halved && piece % 2)) return false;
  int64_t seen = 0;
  for (int b = 0; b < bands; ++b) {
    int at = 0;
    for (int i = 0; i < full_per_band; ++i, ++seen) {
      const bool cut = full_total && ((seen + 1) * halved / full_total) != (seen * halved / full_total);
      if (cut) {
        tiles->push_back((uint32_t)b | ((uint32_t)at << 12) | ((uint32_t)(piece / 2) << 24));
        tiles->push_back((uint32_t)b | ((uint32_t)(at + piece / 2) << 12) | ((uint32_t)(piece / 2) << 24));
      } else {
        tiles->push_back((uint32_t)b | ((uint32_t)at << 12) | ((uint32_t)piece << 24));
      }
      at += piece;
    }
    if (at < units) tiles->push_back((uint32_t)b | ((uint32_t)at << 12) | ((uint32_t)(units - at) << 24));
  }
  return true;
}

// Deals the tiles (in band order) out in rounds of `workers`; within a round the costliest tile goes to the pair with
// the least work so far. Returns the largest total of any pair; fills `out` (entry[round * workers + pair]) if given.
static double deal_rounds(const std::vector<uint32_t>& tiles, int workers, TileSchedule* out, int* first_round_bands,
                          int* first_round_blocks = nullptr) {
  std::vector<double> load(workers, 0.0);
  std::vector<int> order(workers);
  std::vector<uint32_t> round;
  const int rounds = (int)((tiles.size() + workers - 1) / workers);
  if (out) {
    if ((size_t)rounds * workers > (size_t)kSchedMaxEntries) return -1.0;
    out->rounds = (uint32_t)rounds;
    out->workers = (uint32_t)workers;
    for (int i = 0; i < rounds * workers; ++i) out->entry[i] = 0;
  }
  for (int j = 0; j < rounds; ++j) {
    const size_t begin = (size_t)j * workers, end = std::min(tiles.size(), begin + workers);
    round.assign(tiles.begin() + begin, tiles.begin() + end);
    if (j == 0 && first_round_bands) *first_round_bands = (int)(round.back() & 0xfffu) + 1;
    if (j == 0 && first_round_blocks) {
      int reach = 0;   // 256-column blocks of B up to the rightmost column a tile of this round reads
      for (uint32_t e : round) reach = std::max(reach, (int)((((e >> 12) & 0xfffu) + (e >> 24)) * 32 + 255) / 256);
      *first_round_blocks = reach;
    }
    std::stable_sort(round.begin(), round.end(), [](uint32_t a, uint32_t b) { return (a >> 24) > (b >> 24); });
    for (int w = 0; w < workers; ++w) order[w] = w;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return load[a] < load[b]; });
    for (size_t i = 0; i < round.size(); ++i) {
      const int w = order[i];
      load[w] += tile_cost((int)(round[i] >> 24));
      if (out) out->entry[j * workers + w] = round[i];
    }
  }
  return *std::max_element(load.begin(), load.end());
}

// The cut with the smallest largest total among: 256-wide pieces with any number of them halved (the plain walk is the
// one with none), 128-wide pieces, 64-wide pieces. The table is used when it saves at least 3 % over the plain walk.
static void choose_schedule(int bands, int64_t N, int workers, ScheduleChoice* choice) {
  choice->table = false;
  const int units = (int)((N + 31) / 32);
  std::vector<uint32_t> tiles;
  cut_bands(bands, units, 8, 0, &tiles);
  choice->uniform = deal_rounds(tiles, workers, nullptr, nullptr);
  choice->makespan = choice->uniform;
  if (bands >= 4096 || units >= 4096 || workers < 1 || !table_allowed()) return;
  int best_piece = 0, best_halved = 0;
  double best = choice->uniform;
  auto consider = [&](int piece, int halved) {
    if (!cut_bands(bands, units, piece, halved, &tiles)) return;
    const int rounds = (int)((tiles.size() + workers - 1) / workers);
    if ((int64_t)rounds * workers > kSchedMaxEntries) return;
    const double span = deal_rounds(tiles, workers, nullptr, nullptr);
    if (span > 0 && span < best) { best = span; best_piece = piece; best_halved = halved; }
  };
  const int64_t full = (int64_t)bands * (units / 8);
  if (full <= kSchedMaxEntries)
    for (int64_t halved = 1, step = std::max<int64_t>(1, full / 96); halved <= full; halved += step) consider(8, (int)halved);
  consider(4, 0);
  consider(2, 0);
  if (best_piece == 0 || best > 0.97 * choice->uniform) return;
  cut_bands(bands, units, best_piece, best_halved, &tiles);
  if (deal_rounds(tiles, workers, &choice->sched, &choice->first_round_bands, &choice->first_round_blocks) < 0) return;
  choice->makespan = best;
  choice->table = true;
}

// Schedules are a pure function of (bands, N, pairs); the last few are kept per host thread.
static const ScheduleChoice& schedule_for(int bands, int64_t N, int workers) {
  struct Slot { int bands = -1; int64_t n = -1; int workers = -1; ScheduleChoice choice; };
  static thread_local Slot slots[4];
  static thread_local int next = 0;
  for (const Slot& slot : slots)
    if (slot.bands == bands && slot.n == N && slot.workers == workers) return slot.choice;
  Slot& slot = slots[next];
  next = (next + 1) % 4;
  slot.bands = bands; slot.n = N; slot.workers = workers;
  choose_schedule(bands, N, workers, &slot.choice);
  return slot.choice;
}

// Tensor map of a K-major plane with a given box height.
template <int KIND>
static int launch_stream(uint8_t* ws, const PlaneLayout& L, const float* A, int64_t lda, bool split_a_here, const float* B,
                         int64_t ldb, bool split_b_here, float* C, int64_t M, int64_t N, int64_t K, int64_t ldc, cudaStream_t s,
                         int* status_word = nullptr) {
  constexpr int kStreamSmemBytes = GemmCfg<2, 256>::kSmemBytes + kTransposeScratchBytes;
  using Cfg = GemmCfg<2, 256>;
  constexpr int eb = (KIND == 0) ? 2 : 4;
  const void* a_hi = ws + L.a_hi();
  const void* a_lo = ws + L.a_lo();
  const void* b_hi = ws + L.b_hi();
  const void* b_lo = ws + L.b_lo();
  CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo, mb16_hi, mb16_lo;
  int rc;
  if ((rc = make_plane_map(&ma_hi, a_hi, eb, M, K, L.Kp, 128))) return rc;
  if ((rc = make_plane_map(&ma_lo, a_lo, eb, M, K, L.Kp, 128))) return rc;
  if ((rc = make_plane_map(&mb_hi, b_hi, eb, N, K, L.Kp, 128))) return rc;
  if ((rc = make_plane_map(&mb_lo, b_lo, eb, N, K, L.Kp, 128))) return rc;
  if ((rc = make_plane_map(&mb16_hi, b_hi, eb, N, K, L.Kp, 16))) return rc;
  if ((rc = make_plane_map(&mb16_lo, b_lo, eb, N, K, L.Kp, 16))) return rc;

  auto kernel = gemm_x3_stream_kernel<KIND>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemBytes));
    attr_dev = dev;
  }
  int* status = status_word ? status_word : device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gemm: could not allocate the device status word");

  const int tiles_m = (int)((M + 255) / 256), tiles_n = (int)((N + 255) / 256);
  const int num_kb = (int)(L.Kp / (kTileRowBytes / eb));
  const int pairs = sm_count() / 2;
  const ScheduleChoice& choice = schedule_for(tiles_m, N, pairs);
  int units = pairs;
  if (!choice.table && (int64_t)tiles_m * tiles_n < units) units = (int)((int64_t)tiles_m * tiles_n);
  const int group_m = raster_group_m();

  SplitWork work = {};
  work.A = A;
  work.B = B;
  work.lda = lda;
  work.ldb = ldb;
  work.a_hi = ws + L.a_hi();
  work.a_lo = ws + L.a_lo();
  work.b_hi = ws + L.b_hi();
  work.b_lo = ws + L.b_lo();
  work.ctrl = reinterpret_cast<int*>(ws + L.ctrl());
  work.M = (int)M;
  work.N = (int)N;
  work.K = (int)K;
  work.Kp = (int)L.Kp;
  work.chunks = L.chunks;
  work.a_bands = split_a_here ? L.bands : 0;
  work.b_blocks = split_b_here ? L.blocks : 0;
  work.b_flags = L.bands * L.chunks;
  work.items = (work.a_bands + work.b_blocks) * L.chunks;
  work.a_vec_ok = aligned_to(A, 16) && (lda % 4 == 0);
  work.b_vec_ok = aligned_to(B, 16) && (ldb % 4 == 0);
  if (choice.table) {
    work.ga = choice.first_round_bands;
    work.gb = choice.first_round_blocks;
  } else {
    // the raster walks groups of group_m bands, all columns of a group before the next group
    const int gsize = std::min(group_m, tiles_m);
    const int64_t first_group = (int64_t)gsize * tiles_n;
    if (units <= first_group) {
      work.ga = gsize;
      work.gb = (units - 1) / gsize + 1;
    } else {
      work.ga = (int)std::min<int64_t>(tiles_m, (units + first_group - 1) / first_group * gsize);
      work.gb = tiles_n;
    }
  }
  work.ga = std::max(0, std::min(work.ga, work.a_bands));
  work.gb = std::max(0, std::min(work.gb, work.b_blocks));
  if (work.items && work.ga + work.gb == 0) {   // cannot happen with a sane schedule; keep the numbering well-defined
    work.ga = work.a_bands ? 1 : 0;
    work.gb = work.a_bands ? 0 : 1;
  }

  static thread_local TileSchedule raster = {};   // rounds = 0: tiles from the raster formula
  const TileSchedule& sched = choice.table ? choice.sched : raster;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * 2));
  cfg.blockDim = dim3(kStreamThreads);
  cfg.dynamicSmemBytes = kStreamSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const int c_vec_ok = aligned_to(C, 16) && (ldc % 4 == 0);
  DTN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ma_hi, ma_lo, mb_hi, mb_lo, mb16_hi, mb16_lo, C, ldc, (int)M, (int)N,
                                    num_kb, tiles_m, tiles_n, group_m, c_vec_ok, status, work, sched));
  return DTN_OK;
}

// True when the automatic choice takes CTA-pair tiles: from three quarters of a round of pair tiles.
static bool pairs_preferred(int64_t M, int64_t N) {
  const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  return pair_tiles * 8 >= (int64_t)(sm_count() / 2) * 6;
}

template <int KIND>
static int run_tc(int variant, const uint8_t* ws, const PlaneLayout& L, float* C, int64_t M, int64_t N, int64_t K,
                  int64_t ldc, cudaStream_t s, int* status_word = nullptr) {
  const void* a_hi = ws + L.a_hi();
  const void* a_lo = ws + L.a_lo();
  const void* b_hi = ws + L.b_hi();
  const void* b_lo = ws + L.b_lo();
  if (variant == 0) {
    // Large problems: a CTA pair per 256x256 tile (least shared-memory traffic per flop); smaller
    // ones: more, smaller tiles keep more SMs busy.
    // Measured (bf16x3, us, variants 1 / 2 / 3): 1536^3 (36 pair tiles) 27.9 / 40.7 / 39.8; 2048^3 (64) 54.1 / 49.8 / 49.1;
    // 3072^3 (144) 157 / 149 / 136; 8192^3 2723 / 2594 / 2341. Pairs win from about three quarters of a wave of pairs.
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t wide_tiles = ((M + 127) / 128) * ((N + 255) / 256);
    const int64_t square_tiles = ((M + 127) / 128) * ((N + 127) / 128);
    variant = (pair_tiles * 8 >= (int64_t)(sm_count() / 2) * 6) ? 3 : (wide_tiles >= sm_count()) ? 2 : 1;
    // fewer 128x128 tiles than half the SMs: 128x64 tiles put twice as many CTAs to work (768^3 14.3 vs 16.7 us,
    // 1024^3 16.8 vs 18.2 us)
    if (variant == 1 && square_tiles * 2 <= sm_count()) variant = 5;
  }
  if (variant >= 7) variant = 3;
  switch (variant) {
    case 1: return launch_tc<KIND, 1, 128>(a_hi, a_lo, b_hi, b_lo, C, M, N, K, L.Kp, ldc, s, status_word);
    case 2: return launch_tc<KIND, 1, 256>(a_hi, a_lo, b_hi, b_lo, C, M, N, K, L.Kp, ldc, s, status_word);
    case 3: return launch_tc<KIND, 2, 256>(a_hi, a_lo, b_hi, b_lo, C, M, N, K, L.Kp, ldc, s, status_word);
    case 5: return launch_tc<KIND, 1, 64>(a_hi, a_lo, b_hi, b_lo, C, M, N, K, L.Kp, ldc, s, status_word);
    default:
      set_error("gemm: unknown variant %d", variant);
      return DTN_ERR_INVALID;
  }
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant: the operand planes live in a fixed array inside the library image.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = (size_t)32 << 20;   // largest set of operand planes the array can hold
// The planes must start on a 1024-byte boundary; the array is 256-byte aligned, so it carries
// 1024 bytes of slack and the usable part starts at the first 1024-byte boundary inside it.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes + 1024];
static __device__ int g_static_status;   // where this variant's kernels report a wait that ran out

struct StaticScratch {
  uint8_t* planes = nullptr;   // device address of the usable, 1024-byte aligned part
  int* status = nullptr;
};
static std::mutex g_static_mutex;
static StaticScratch g_static_by_device[64];

// Device addresses of the two symbols on the current device, resolved once per device. In host code
// the symbols' names are host-side stand-ins, never device addresses: only cudaGetSymbolAddress,
// called with the device current, yields a pointer a kernel may use.
static int static_scratch_for_current_device(StaticScratch* out) {
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  DTN_REQUIRE(dev >= 0 && dev < 64, DTN_ERR_UNSUPPORTED, "gemm: device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticScratch& entry = g_static_by_device[dev];
  if (entry.planes == nullptr) {
    void* scratch = nullptr;
    void* status = nullptr;
    DTN_CUDA_CHECK(cudaGetSymbolAddress(&scratch, g_static_scratch));
    DTN_CUDA_CHECK(cudaGetSymbolAddress(&status, g_static_status));
    const uintptr_t aligned = (reinterpret_cast<uintptr_t>(scratch) + 1023) & ~(uintptr_t)1023;
    entry.status = static_cast<int*>(status);
    entry.planes = reinterpret_cast<uint8_t*>(aligned);
  }
  *out = entry;
  return DTN_OK;
}

}  // namespace dtn

extern "C" {

int dtn_gemm_x3_static(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldc, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(mode == DTN_GEMM_TF32X3 || mode == DTN_GEMM_BF16X3, DTN_ERR_INVALID,
              "gemm (static scratch): mode must be DTN_GEMM_BF16X3 or DTN_GEMM_TF32X3, got %d", mode);
  DTN_REQUIRE(M >= 0 && N >= 0 && K >= 0, DTN_ERR_INVALID, "gemm (static scratch): negative extent");
  if (M == 0 || N == 0) return DTN_OK;
  DTN_REQUIRE(C != nullptr, DTN_ERR_INVALID, "gemm (static scratch): C is null");
  DTN_REQUIRE(lda >= K && ldb >= N && ldc >= N, DTN_ERR_INVALID,
              "gemm (static scratch): leading dimension smaller than the row");
  DTN_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), DTN_ERR_UNSUPPORTED,
              "gemm (static scratch): extents must fit 31 bits");
  cudaStream_t s = as_stream(stream);
  if (K == 0) {   // an empty sum: C = 0, as dtn_gemm_x3 gives
    DTN_CUDA_CHECK(cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, s));
    return DTN_OK;
  }
  DTN_REQUIRE(A != nullptr && B != nullptr, DTN_ERR_INVALID, "gemm (static scratch): operand pointer is null");
  DTN_REQUIRE(aligned_to(A, 4) && aligned_to(B, 4) && aligned_to(C, 4), DTN_ERR_INVALID,
              "gemm (static scratch): pointers must be 4-byte aligned");
  // This entry point always runs the split kernels and the tensor-memory product kernel. The selections of
  // dtn_gemm_set_variant that name a tile of that kernel (1, 2, 3, 5) are honoured; 4 and 6 name other kernels
  // (which use no scratch at all) and fall back to the automatic tile choice here.
  const int variant = (g_gemm_variant == 4 || g_gemm_variant == 6) ? 0 : (g_gemm_variant >= 7 ? 3 : g_gemm_variant);
  const PlaneLayout L = plane_layout(mode, M, N, K);
  DTN_REQUIRE(L.planes() <= kStaticScratchBytes, DTN_ERR_WORKSPACE,
              "gemm (static scratch): %lld x %lld x %lld needs %zu bytes of operand planes, the built-in array holds %zu; "
              "use dtn_gemm_x3 with a caller-owned workspace",
              (long long)M, (long long)N, (long long)K, L.planes(), kStaticScratchBytes);
  StaticScratch scratch;
  int rc;
  if ((rc = static_scratch_for_current_device(&scratch))) return rc;
  // Nothing in the array has to start at zero: the split kernels overwrite every byte of the planes the
  // product kernel reads, padding included. The status word is only ever set by a kernel that gave up.
  if (mode == DTN_GEMM_BF16X3) {
    if ((rc = run_split<Bf16Kind>(A, B, M, N, K, lda, ldb, L, scratch.planes, s))) return rc;
    return run_tc<0>(variant, scratch.planes, L, C, M, N, K, ldc, s, scratch.status);
  }
  if ((rc = run_split<Tf32Kind>(A, B, M, N, K, lda, ldb, L, scratch.planes, s))) return rc;
  return run_tc<1>(variant, scratch.planes, L, C, M, N, K, ldc, s, scratch.status);
}

int dtn_gemm_x3_static_status(int* status_out, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(status_out != nullptr, DTN_ERR_INVALID, "dtn_gemm_x3_static_status: status_out is null");
  StaticScratch scratch;
  int rc;
  if ((rc = static_scratch_for_current_device(&scratch))) return rc;
  cudaStream_t s = as_stream(stream);
  int host = 0;
  DTN_CUDA_CHECK(cudaMemcpyAsync(&host, scratch.status, sizeof(int), cudaMemcpyDeviceToHost, s));
  DTN_CUDA_CHECK(cudaStreamSynchronize(s));
  if (host != 0) DTN_CUDA_CHECK(cudaMemsetAsync(scratch.status, 0, sizeof(int), s));
  *status_out = host;
  return DTN_OK;
}

int dtn_gemm_tile_schedule(int64_t M, int64_t N, int pairs, uint32_t* entries_out, int capacity, int* rounds_out,
                           double* longest_out, double* longest_uniform_out) {
  using namespace dtn;
  DTN_REQUIRE(M > 0 && N > 0 && pairs > 0 && pairs <= 1024, DTN_ERR_INVALID, "tile schedule: M, N and pairs must be positive");
  DTN_REQUIRE(rounds_out != nullptr, DTN_ERR_INVALID, "tile schedule: rounds_out is null");
  DTN_REQUIRE(M < (1LL << 31) && N < (1LL << 31), DTN_ERR_UNSUPPORTED, "tile schedule: extents must fit 31 bits");
  ScheduleChoice choice;
  choose_schedule((int)((M + 255) / 256), N, pairs, &choice);
  *rounds_out = choice.table ? (int)choice.sched.rounds : 0;
  if (longest_out) *longest_out = choice.makespan;
  if (longest_uniform_out) *longest_uniform_out = choice.uniform;
  if (choice.table && entries_out != nullptr) {
    const int count = (int)choice.sched.rounds * pairs;
    DTN_REQUIRE(capacity >= count, DTN_ERR_INVALID, "tile schedule: %d entries needed, room for %d", count, capacity);
    for (int i = 0; i < count; ++i) entries_out[i] = choice.sched.entry[i];
  }
  return DTN_OK;
}

int dtn_gemm_set_variant(int variant) {
  DTN_REQUIRE(variant >= 0 && variant <= 10, DTN_ERR_INVALID, "gemm: variant must be 0..10");
  dtn::g_gemm_variant = variant;
  return DTN_OK;
}

int dtn_gemm_skinny_plan(int64_t N, int64_t K, int workers, int64_t* unit_begin_out, int* first_out, int* last_out) {
  return dtn::gemm_skinny_plan(N, K, workers, unit_begin_out, first_out, last_out);
}

int dtn_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, size_t* bytes_out) {
  using namespace dtn;
  DTN_REQUIRE(bytes_out != nullptr, DTN_ERR_INVALID, "gemm: bytes_out is null");
  DTN_REQUIRE(M >= 0 && N >= 0 && K >= 0, DTN_ERR_INVALID, "gemm: negative extent");
  DTN_REQUIRE(mode == DTN_GEMM_F32 || mode == DTN_GEMM_TF32X3 || mode == DTN_GEMM_BF16X3 || mode == DTN_GEMM_F32_SPLITK,
              DTN_ERR_INVALID, "gemm: unknown mode %d", mode);
  *bytes_out = (mode == DTN_GEMM_F32 || mode == DTN_GEMM_F32_SPLITK || M == 0 || N == 0 || K == 0) ? 0 : plane_layout(mode, M, N, K).total;
  return DTN_OK;
}

int dtn_gemm_x3_phase(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, void* workspace, size_t workspace_bytes, int phase,
                      void* stream) {
  using namespace dtn;
  DTN_REQUIRE(phase >= 1 && phase <= 15 && (phase & 3) != 0, DTN_ERR_INVALID,
              "gemm: phase is a mask of 1 (split), 2 (products), 4 (keep A planes), 8 (keep B planes)");
  const bool split_a = (phase & 1) && !(phase & 4), split_b = (phase & 1) && !(phase & 8);
  DTN_REQUIRE(mode == DTN_GEMM_F32 || mode == DTN_GEMM_TF32X3 || mode == DTN_GEMM_BF16X3 || mode == DTN_GEMM_F32_SPLITK,
              DTN_ERR_INVALID, "gemm: unknown mode %d", mode);
  DTN_REQUIRE(M >= 0 && N >= 0 && K >= 0, DTN_ERR_INVALID, "gemm: negative extent");
  if (M == 0 || N == 0) return DTN_OK;
  DTN_REQUIRE(C != nullptr, DTN_ERR_INVALID, "gemm: C is null");
  DTN_REQUIRE(lda >= K && ldb >= N && ldc >= N, DTN_ERR_INVALID, "gemm: leading dimension smaller than the row");
  DTN_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), DTN_ERR_UNSUPPORTED,
              "gemm: extents must fit 31 bits");
  cudaStream_t s = as_stream(stream);
  if (K == 0) {
    DTN_CUDA_CHECK(cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, s));
    return DTN_OK;
  }
  DTN_REQUIRE(A != nullptr && B != nullptr, DTN_ERR_INVALID, "gemm: operand pointer is null");
  DTN_REQUIRE(aligned_to(A, 4) && aligned_to(B, 4) && aligned_to(C, 4), DTN_ERR_INVALID,
              "gemm: pointers must be 4-byte aligned");
  if (mode == DTN_GEMM_F32 || mode == DTN_GEMM_F32_SPLITK)
    return (phase & 2) ? gemm_f32_launch(A, B, C, M, N, K, lda, ldb, ldc, s, mode == DTN_GEMM_F32_SPLITK) : DTN_OK;

  // At most 16 rows: the TMA-fed single-pass kernel when B is worth streaming (measured: 16 x 4736 x 8192 33.7 against
  // 59.5 us, 16 x 2048 x 4096 16.5 against 15.5 us for the cp.async kernel; variant 10 takes it wherever it applies).
  // Its partial sums live in the workspace, which is sized for B's planes and therefore large enough whenever B is.
  // DTN_GEMM_SKINNY_TMA=0 keeps the cp.async kernel.
  static const bool skinny_tma = [] {
    const char* text = getenv("DTN_GEMM_SKINNY_TMA");
    return !(text && text[0] == '0');
  }();
  const bool skinny_wanted = g_gemm_variant == 10 || (g_gemm_variant == 0 && skinny_tma && (double)N * (double)K >= 12.0 * 1024 * 1024);
  if (phase == 3 && skinny_wanted && gemm_skinny_supported(A, B, M, N, K, lda, ldb) && workspace != nullptr && aligned_to(workspace, 16) &&
      workspace_bytes >= gemm_skinny_workspace_bytes(N, K))
    return gemm_skinny_launch(mode, A, B, C, M, N, K, lda, ldb, ldc, workspace, s);
  DTN_REQUIRE(g_gemm_variant != 10, DTN_ERR_UNSUPPORTED,
              "gemm: the streamed skinny kernel needs at most 16 rows, 16-byte aligned A and B with leading dimensions that are "
              "multiples of 4, both phases in one call and a workspace");
  if (phase == 3 && (g_gemm_variant == 4 || (g_gemm_variant == 0 && prefers_small_kernel(M, N, K))))
    return gemm_small_launch(mode, A, B, C, M, N, K, lda, ldb, ldc, s);
  DTN_REQUIRE(g_gemm_variant != 4, DTN_ERR_INVALID, "gemm: the single-kernel variant has no separate phases");
  if (phase == 3 && g_gemm_variant == 6) {
    return gemm_fused_launch(mode, A, B, C, M, N, K, lda, ldb, ldc, s, fused_bn_override());
  }
  DTN_REQUIRE(g_gemm_variant != 6, DTN_ERR_INVALID, "gemm: the fused-split variant has no separate phases");

  const PlaneLayout L = plane_layout(mode, M, N, K);
  DTN_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, DTN_ERR_WORKSPACE,
              "gemm: workspace of %zu bytes needed, %zu given", L.total, workspace_bytes);
  DTN_REQUIRE(aligned_to(workspace, 1024), DTN_ERR_WORKSPACE, "gemm: workspace must be 1024-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int rc;
  // CTA-pair tiles (automatic for large products): the stream kernel. It splits both operands itself, beside its
  // products: one kernel, preceded by a memset of its counters.
  if ((phase & 2) && (g_gemm_variant >= 7 || (g_gemm_variant == 0 && pairs_preferred(M, N)))) {
    // which operands the kernel splits itself, beside its products, and which a split kernel handles before it
    // (variants 8 and 9 pin the choice: neither / both)
    const int inside = g_gemm_variant == 8 ? 0 : g_gemm_variant == 9 ? 3 : stream_split_override() >= 0 ? stream_split_override() : 1;
    // Measured (8192 x N x 8192 back to back, split outside against inside): the split of A inside the kernel pays
    // when the plain walk has at least two rounds (N = 1024: 359 -> 329 us, 4096: 1229 -> 1192, 8192: 2485 -> 2441).
    // With a single round every tile needs its operands at once and the split sits on the critical path (2048^3: 60
    // against 53 us); with a tile table the narrow tiles of the first round ask for more bands at once than the split
    // warps deliver (N = 2048: 653 outside, 675 inside). B's transposing split is always slower inside (one tile in
    // flight per SM instead of a dozen).
    const bool several_rounds = ((M + 255) / 256) * ((N + 255) / 256) > (int64_t)(sm_count() / 2);
    const bool pinned = g_gemm_variant >= 8 || stream_split_override() >= 0;
    const bool table = schedule_for((int)((M + 255) / 256), N, sm_count() / 2).table;
    const bool a_inside = split_a && (inside & 1) && ((several_rounds && !table) || pinned), b_inside = split_b && (inside & 2);
    const bool a_before = split_a && !a_inside, b_before = split_b && !b_inside;
    const bool counters = a_inside || b_inside;
    if (a_before || b_before) {
      const bool zero = counters && b_before;   // the transposing split kernel can clear the counters on its way
      rc = (mode == DTN_GEMM_BF16X3) ? run_split<Bf16Kind>(A, B, M, N, K, lda, ldb, L, ws, s, a_before, b_before, zero)
                                     : run_split<Tf32Kind>(A, B, M, N, K, lda, ldb, L, ws, s, a_before, b_before, zero);
      if (rc) return rc;
      if (counters && !zero)
        DTN_CUDA_CHECK(cudaMemsetAsync(ws + L.ctrl(), 0, sizeof(int) * (2 + ((size_t)L.bands + L.blocks) * L.chunks), s));
    } else if (counters) {
      DTN_CUDA_CHECK(cudaMemsetAsync(ws + L.ctrl(), 0, sizeof(int) * (2 + ((size_t)L.bands + L.blocks) * L.chunks), s));
    }
    return (mode == DTN_GEMM_BF16X3) ? launch_stream<0>(ws, L, A, lda, a_inside, B, ldb, b_inside, C, M, N, K, ldc, s)
                                     : launch_stream<1>(ws, L, A, lda, a_inside, B, ldb, b_inside, C, M, N, K, ldc, s);
  }
  if (mode == DTN_GEMM_BF16X3) {
    if ((phase & 1) && (rc = run_split<Bf16Kind>(A, B, M, N, K, lda, ldb, L, ws, s, split_a, split_b))) return rc;
    return (phase & 2) ? run_tc<0>(g_gemm_variant, ws, L, C, M, N, K, ldc, s) : DTN_OK;
  }
  if ((phase & 1) && (rc = run_split<Tf32Kind>(A, B, M, N, K, lda, ldb, L, ws, s, split_a, split_b))) return rc;
  return (phase & 2) ? run_tc<1>(g_gemm_variant, ws, L, C, M, N, K, ldc, s) : DTN_OK;
}

int dtn_gemm_x3(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                int64_t ldb, int64_t ldc, void* workspace, size_t workspace_bytes, void* stream) {
  return dtn_gemm_x3_phase(mode, A, B, C, M, N, K, lda, ldb, ldc, workspace, workspace_bytes, 3, stream);
}

}  // extern "C"
