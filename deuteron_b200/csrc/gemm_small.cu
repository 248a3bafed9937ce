// Compensated FP32 GEMM for small and skinny problems: one kernel, operand split inside it.
//
// A tcgen05 GEMM needs a split pass over the operands, tensor-memory allocation and 128-row
// tiles; for a 128^3 or 512^3 product, or for 16 rows, that set-up is most of the run time.
// This kernel keeps the structure of the reference's emitted code instead: FP32 B tiles go to
// shared memory through a 4-slot cp.async ring and every warp converts the B fragments it needs to a
// rounded high part and a rounded residual in registers; the A tile, whose fragments every warp of a
// k group shares, is split once per CTA into two planes. Each warp issues the three warp-level
// products per k-step in the reference's order (lo*hi, hi*lo, hi*hi; mma.sync m16n8k16 for
// bf16, m16n8k8 for tf32) into FP32 accumulators. Two configurations: a 64x64 CTA tile with 4 warps
// of 32x32 and a 32-deep k-tile (small square problems; the reference's accumulation order, so its
// published outputs are reproduced bit for bit), and a 16x64 tile with a 64-deep k-tile and two
// groups of four warps that each take half of the k-tile (at most 16 rows).
// Any M, N, K and leading dimensions: out-of-range elements are zero-filled by the copies.
#include <stdlib.h>

#include "dtn_common.cuh"

namespace dtn {

constexpr int S_BN = 64, S_THREADS = 128;   // 4 warps; the tile height, k-tile and ring depth are template parameters

// BM = 64: 2 x 2 warps of 32 x 32 (general small problems). BM = 16: 1 x 4 warps of 16 x 16 for skinny
// products (at most 16 rows), which are bound by streaming B once from HBM: a 64-deep k-tile and four
// slots keep ~50 KB of loads in flight per CTA.
template <int MODE, int BM, int BK, int STAGES>
struct SmallCfg {
  // leading dimensions chosen so that the fragment reads below are bank-conflict free
  static constexpr int kLda = (MODE == 0) ? BK + 8 : BK + 4;   // A tile [BM][kLda]
  static constexpr int kLdb = (MODE == 0) ? 68 : 72;           // B tile [BK][kLdb]
  static constexpr int kAFloats = (MODE == 0 ? 1 : 2) * BM * kLda;   // high and residual plane of the A tile (bf16 pairs / tf32 words)
  static constexpr int kStageFloats = kAFloats + BK * kLdb;
  static constexpr int kSmemBytes = STAGES * kStageFloats * 4;
  static constexpr int kMI = BM == 64 ? 2 : 1;                 // m16 tiles per warp
  static constexpr int kNI = BM == 16 ? 2 : 4;                 // n8 tiles per warp
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int valid_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int valid_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(valid_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
  __nv_bfloat162 v = __floats2bfloat162_rn(low, high);   // .x (low half) = first k index
  return *reinterpret_cast<uint32_t*>(&v);
}
// hi = bf16_rn(v) pairs, lo = bf16_rn(v - hi) pairs. One conversion rounds both values; the residuals come from the
// mixed-precision fma of sm_100, which takes the bf16 halves as they are: v - hi = hi * (-1) + v, exact, without
// the shift and the mask that bring hi back to FP32 (four instructions per pair instead of six; these kernels are
// bound by exactly this arithmetic).
__device__ __forceinline__ void split_bf16_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(a, b);
  float ra, rb;
  asm("{\n\t.reg .b16 h0, h1, m;\n\tmov.b32 {h0, h1}, %2;\n\tmov.b16 m, 0xBF80;\n\t"   // m = -1.0
      "fma.rn.f32.bf16 %0, h0, m, %3;\n\tfma.rn.f32.bf16 %1, h1, m, %4;\n\t}"
      : "=f"(ra), "=f"(rb)
      : "r"(hi), "f"(a), "f"(b));
  lo = pack_bf16(ra, rb);
}
// The high part is rounded with integer arithmetic (half a tf32 unit added to the bit pattern, thirteen low bits
// cleared: equal to cvt.rna.tf32.f32 on all 2^32 inputs but NaNs, and not on the slow conversion pipe); the residual,
// which is NaN whenever v is NaN or infinite, keeps the conversion instruction, so a NaN still reaches every product.
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u;
  const float rest = v - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// KSPLIT = 2: eight warps, the second group of four takes the upper half of every k-tile and the two partial
// accumulators are added through shared memory at the end (twice the warps to hide conversion and MMA latency).
template <int MODE /*0 = bf16x3, 1 = tf32x3*/, int ALIGNED /*0: any addresses, 1: 128-bit accesses, 2: and only full tiles*/, int BM, int BK, int STAGES, int KSPLIT>
__global__ void __launch_bounds__(S_THREADS * KSPLIT)
gemm_x3_small_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                     int64_t lda, int64_t ldb, int64_t ldc) {
  using Cfg = SmallCfg<MODE, BM, BK, STAGES>;
  constexpr int MI = Cfg::kMI, NI = Cfg::kNI;
  extern __shared__ __align__(16) float small_smem[];
  constexpr int kThreads = S_THREADS * KSPLIT;
  const int tid = threadIdx.x, warp = (tid >> 5) & 3, kgroup = tid >> 7, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * S_BN;
  const int wm = BM == 64 ? (warp >> 1) * 32 : (BM == 32 ? (warp >> 1) * 16 : 0), wn = BM == 16 ? warp * 16 : (warp & 1) * 32;
  const uint32_t smem_base = smem_u32(small_smem);

  // EXACT: every tile of the launch is full (M, N and K are multiples of the tile), so no access needs a bounds check
  // (512^3: 8.85 -> about 8.2 us; a tenth of the instructions were comparisons and selects on the extents)
  constexpr bool EXACT = ALIGNED == 2;
  const int b_piece_n = (tid & 15) * 4;
  const int b_col_bytes = EXACT ? 16 : min(max((N - (n0 + b_piece_n)) * 4, 0), 16);
  const float* b_col = B + n0 + b_piece_n;
  const uint32_t b_piece_smem = (uint32_t)b_piece_n * 4u;
  static_assert((BK * 16) % (S_THREADS * KSPLIT) == 0, "B tile must divide among the threads");
  auto load_tile = [&](int kt, int slot) {
    const int k0 = kt * BK;
    const uint32_t a_s = smem_base + (uint32_t)(slot * Cfg::kStageFloats) * 4u;
    const uint32_t b_s = a_s + (uint32_t)Cfg::kAFloats * 4u;
    if constexpr (ALIGNED) {
      // B: BK rows x 16 pieces; a thread always copies the same piece of a row (column offset, byte count and
      // the shared-memory column are fixed), only the row moves
#pragma unroll
      for (int i = 0; i < BK * 16 / kThreads; ++i) {
        const int br = (tid >> 4) + i * (kThreads >> 4);
        const int bbytes = (EXACT || k0 + br < K) ? b_col_bytes : 0;
        cp_async_16(b_s + b_piece_smem + (uint32_t)(br * Cfg::kLdb) * 4u,
                    (EXACT || bbytes) ? (const void*)(b_col + (int64_t)(k0 + br) * ldb) : (const void*)B, bbytes);
      }
    } else {
#pragma unroll 4
      for (int v = tid; v < BK * 64; v += kThreads) {
        const int br = v >> 6, bn = v & 63;
        const bool bin = (k0 + br < K) && (n0 + bn < N);
        cp_async_4(b_s + (uint32_t)(br * Cfg::kLdb + bn) * 4u, bin ? (const void*)(B + (int64_t)(k0 + br) * ldb + n0 + bn) : (const void*)B, bin ? 4 : 0);
      }
    }
  };

  // The A tile does not go through the copy ring. Every warp of a k group needs the same A fragments, so splitting
  // them after the fragment read would repeat the conversion once per warp; instead each thread reads its share of
  // the tile one k-tile ahead, splits it once and writes the high and the residual plane ([BM][kLda] each: packed
  // bf16 pairs, or tf32 words) at the head of the stage. Same arithmetic, same operands.
  constexpr int kAVecs = (BM * BK / 4) / kThreads;   // float4 of the A tile per thread
  static_assert((BM * BK / 4) % kThreads == 0, "A tile must divide among the threads");
  auto load_a = [&](int kt, float4 (&r)[kAVecs > 0 ? kAVecs : 1]) {
    const int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < kAVecs; ++i) {
      const int v = i * kThreads + tid, ar = v / (BK / 4), ak = (v % (BK / 4)) * 4;
      const int gr = m0 + ar, gk = k0 + ak;
      const float* p = A + (int64_t)gr * lda + gk;
      if (EXACT || (ALIGNED && gr < M && gk + 3 < K)) {
        r[i] = __ldg(reinterpret_cast<const float4*>(p));
      } else {
        const bool row_in = gr < M;
        r[i].x = (row_in && gk < K) ? __ldg(p) : 0.f;
        r[i].y = (row_in && gk + 1 < K) ? __ldg(p + 1) : 0.f;
        r[i].z = (row_in && gk + 2 < K) ? __ldg(p + 2) : 0.f;
        r[i].w = (row_in && gk + 3 < K) ? __ldg(p + 3) : 0.f;
      }
    }
  };
  auto store_a = [&](int slot, const float4 (&r)[kAVecs > 0 ? kAVecs : 1]) {
    uint32_t* hi_plane = reinterpret_cast<uint32_t*>(small_smem + slot * Cfg::kStageFloats);
    uint32_t* lo_plane = hi_plane + Cfg::kAFloats / 2;
#pragma unroll
    for (int i = 0; i < kAVecs; ++i) {
      const int v = i * kThreads + tid, ar = v / (BK / 4), ak = (v % (BK / 4)) * 4;
      if constexpr (MODE == 0) {
        uint2 hi, lo;
        split_bf16_pair(r[i].x, r[i].y, hi.x, lo.x);
        split_bf16_pair(r[i].z, r[i].w, hi.y, lo.y);
        *reinterpret_cast<uint2*>(hi_plane + (ar * Cfg::kLda + ak) / 2) = hi;
        *reinterpret_cast<uint2*>(lo_plane + (ar * Cfg::kLda + ak) / 2) = lo;
      } else {
        uint4 hi, lo;
        split_tf32(r[i].x, hi.x, lo.x);
        split_tf32(r[i].y, hi.y, lo.y);
        split_tf32(r[i].z, hi.z, lo.z);
        split_tf32(r[i].w, hi.w, lo.w);
        *reinterpret_cast<uint4*>(hi_plane + ar * Cfg::kLda + ak) = hi;
        *reinterpret_cast<uint4*>(lo_plane + ar * Cfg::kLda + ak) = lo;
      }
    }
  };

  float acc[MI][NI][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  // With gridDim.z > 1 the launch is a cluster of gridDim.z CTAs along z that share one output tile: each takes a
  // contiguous share of the k-tiles and the partial sums meet in the first CTA's shared memory at the end.
  const int k_parts = (int)gridDim.z, k_part = (int)blockIdx.z;
  const int all_ktiles = (K + BK - 1) / BK;
  const int kt_first = (int)((int64_t)all_ktiles * k_part / k_parts);
  const int ktiles = (int)((int64_t)all_ktiles * (k_part + 1) / k_parts) - kt_first;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < ktiles) load_tile(kt_first + s, s);
    cp_async_commit();
  }
  float4 a_next[kAVecs > 0 ? kAVecs : 1];   // A of k-tile kt + 1, read during k-tile kt
  if (ktiles > 0) {
    load_a(kt_first, a_next);
    store_a(0, a_next);
  }
  if (ktiles > 1) load_a(kt_first + 1, a_next);
  for (int kt = 0; kt < ktiles; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt + STAGES - 1 < ktiles) load_tile(kt_first + kt + STAGES - 1, (kt + STAGES - 1) % STAGES);
    cp_async_commit();
    // The slot of k-tile kt + 1 was last read STAGES - 1 k-tiles ago; its A planes are written here, before the
    // barrier that opens k-tile kt + 1, and the tile after that is requested.
    if (kt + 1 < ktiles) store_a((kt + 1) % STAGES, a_next);
    if (kt + 2 < ktiles) load_a(kt_first + kt + 2, a_next);
    const float* As = small_smem + (kt % STAGES) * Cfg::kStageFloats;
    const float* Bs = As + Cfg::kAFloats;
    if constexpr (MODE == 0) {
#pragma unroll
      for (int kk = kgroup * (BK / KSPLIT); kk < (kgroup + 1) * (BK / KSPLIT); kk += 16) {
        uint32_t a_hi[MI][4], a_lo[MI][4];
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          const uint32_t* hp = reinterpret_cast<const uint32_t*>(As) + ((wm + i * 16 + g) * Cfg::kLda + kk + 2 * t) / 2;
          const uint32_t* lp = hp + Cfg::kAFloats / 2;
          a_hi[i][0] = hp[0];                      // row g,   k 2t, 2t+1
          a_hi[i][1] = hp[4 * Cfg::kLda];          // row g+8
          a_hi[i][2] = hp[4];                      // row g,   k 2t+8, 2t+9
          a_hi[i][3] = hp[4 * Cfg::kLda + 4];      // row g+8
          a_lo[i][0] = lp[0];
          a_lo[i][1] = lp[4 * Cfg::kLda];
          a_lo[i][2] = lp[4];
          a_lo[i][3] = lp[4 * Cfg::kLda + 4];
        }
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const float* bp = Bs + (kk + 2 * t) * Cfg::kLdb + wn + j * 8 + g;
          uint32_t b_hi[2], b_lo[2];
          split_bf16_pair(bp[0], bp[Cfg::kLdb], b_hi[0], b_lo[0]);
          split_bf16_pair(bp[8 * Cfg::kLdb], bp[9 * Cfg::kLdb], b_hi[1], b_lo[1]);
#pragma unroll
          for (int i = 0; i < MI; ++i) {
            mma_bf16(acc[i][j], a_lo[i], b_hi);
            mma_bf16(acc[i][j], a_hi[i], b_lo);
            mma_bf16(acc[i][j], a_hi[i], b_hi);
          }
        }
      }
    } else {
#pragma unroll
      for (int kk = kgroup * (BK / KSPLIT); kk < (kgroup + 1) * (BK / KSPLIT); kk += 8) {
        uint32_t a_hi[MI][4], a_lo[MI][4];
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          const uint32_t* hp = reinterpret_cast<const uint32_t*>(As) + (wm + i * 16 + g) * Cfg::kLda + kk + t;
          const uint32_t* lp = hp + Cfg::kAFloats / 2;
          a_hi[i][0] = hp[0];                      // row g,   k t
          a_hi[i][1] = hp[8 * Cfg::kLda];          // row g+8
          a_hi[i][2] = hp[4];                      // row g,   k t+4
          a_hi[i][3] = hp[8 * Cfg::kLda + 4];      // row g+8
          a_lo[i][0] = lp[0];
          a_lo[i][1] = lp[8 * Cfg::kLda];
          a_lo[i][2] = lp[4];
          a_lo[i][3] = lp[8 * Cfg::kLda + 4];
        }
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const float* bp = Bs + (kk + t) * Cfg::kLdb + wn + j * 8 + g;
          uint32_t b_hi[2], b_lo[2];
          split_tf32(bp[0], b_hi[0], b_lo[0]);
          split_tf32(bp[4 * Cfg::kLdb], b_hi[1], b_lo[1]);
#pragma unroll
          for (int i = 0; i < MI; ++i) {
            mma_tf32(acc[i][j], a_lo[i], b_hi);
            mma_tf32(acc[i][j], a_hi[i], b_lo);
            mma_tf32(acc[i][j], a_hi[i], b_hi);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  if constexpr (KSPLIT == 2) {
    // the upper k-half hands its partial sums to the lower half through the (now idle) ring memory
    __syncthreads();
    float* exchange = small_smem + (warp * 32 + lane) * (MI * NI * 4);
    if (kgroup == 1) {
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) exchange[(i * NI + j) * 4 + e] = acc[i][j][e];
    }
    __syncthreads();
    if (kgroup == 0) {
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[i][j][e] += exchange[(i * NI + j) * 4 + e];
    }
  }
  if (k_parts > 1) {
    // Partial sums of the other CTAs of the cluster go to the first CTA's shared memory (distributed shared memory
    // stores), in a fixed slot per CTA and thread, and are added there in rank order: no atomics, one result.
    constexpr int kPerThread = MI * NI * 4;
    float* slots = small_smem + 2048;   // past the intra-CTA exchange block above
    cluster_barrier();                  // every CTA of the cluster is done with its ring and its exchange block
    if (k_part != 0 && kgroup == 0) {
      const uint32_t local = smem_u32(slots + ((k_part - 1) * S_THREADS + (warp * 32 + lane)) * kPerThread);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(local));
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * ((i * NI + j) * 4 + e)), "f"(acc[i][j][e]) : "memory");
    }
    cluster_barrier();
    if (k_part != 0) return;
    if (kgroup == 0) {
      for (int part = 1; part < k_parts; ++part) {
        const float* theirs = slots + ((part - 1) * S_THREADS + (warp * 32 + lane)) * kPerThread;
#pragma unroll
        for (int i = 0; i < MI; ++i)
#pragma unroll
          for (int j = 0; j < NI; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] += theirs[(i * NI + j) * 4 + e];
      }
    }
  }
  if (kgroup != 0) return;

#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j) {
      const int col = n0 + wn + j * 8 + 2 * t;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = m0 + wm + i * 16 + g + h * 8;
        if (!EXACT && row >= M) continue;
        float* p = C + (int64_t)row * ldc + col;
        if (EXACT || (ALIGNED && col + 1 < N)) {
          *reinterpret_cast<float2*>(p) = make_float2(acc[i][j][2 * h], acc[i][j][2 * h + 1]);
        } else {
          if (col < N) p[0] = acc[i][j][2 * h];
          if (col + 1 < N) p[1] = acc[i][j][2 * h + 1];
        }
      }
    }
}

template <int MODE, int ALIGNED, int BM, int BK, int STAGES, int KSPLIT>
static int gemm_small_launch_cfg(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                 int64_t ldb, int64_t ldc, cudaStream_t s, int k_parts = 1) {
  using Cfg = SmallCfg<MODE, BM, BK, STAGES>;
  dim3 grid((unsigned)((N + S_BN - 1) / S_BN), (unsigned)((M + BM - 1) / BM));
  DTN_REQUIRE(grid.y <= 65535, DTN_ERR_UNSUPPORTED, "gemm: M too large for the small-problem kernel");
  auto kernel = gemm_x3_small_kernel<MODE, ALIGNED, BM, BK, STAGES, KSPLIT>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_dev = dev;
  }
  if (k_parts > 1) {
    grid.z = (unsigned)k_parts;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(S_THREADS * KSPLIT);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)k_parts;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DTN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc));
    return DTN_OK;
  }
  kernel<<<grid, S_THREADS * KSPLIT, Cfg::kSmemBytes, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
  DTN_LAUNCH_CHECK("gemm_x3_small_kernel");
  return DTN_OK;
}

template <int MODE>
static int gemm_small_launch_mode(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                  int64_t ldb, int64_t ldc, cudaStream_t s) {
  const bool aligned = aligned_to(A, 16) && aligned_to(B, 16) && aligned_to(C, 8) && lda % 4 == 0 && ldb % 4 == 0 && ldc % 2 == 0;
  static const int forced = [] {
    const char* text = getenv("DTN_GEMM_SMALL_CFG");   // tuning aid: 1..8 pick a configuration, anything else = automatic
    return text ? atoi(text) : 0;
  }();
#define DTN_SMALL_CFG_ST(BM, BK, KS, ST)                                                                              \
  return !aligned ? gemm_small_launch_cfg<MODE, 0, BM, BK, ST, KS>(A, B, C, M, N, K, lda, ldb, ldc, s, k_parts)         \
         : (M % BM == 0 && N % S_BN == 0 && K % BK == 0)                                                               \
             ? gemm_small_launch_cfg<MODE, 2, BM, BK, ST, KS>(A, B, C, M, N, K, lda, ldb, ldc, s, k_parts)              \
             : gemm_small_launch_cfg<MODE, 1, BM, BK, ST, KS>(A, B, C, M, N, K, lda, ldb, ldc, s, k_parts)
#define DTN_SMALL_CFG(BM, BK, KS) DTN_SMALL_CFG_ST(BM, BK, KS, 4)
  // Skinny products have too few output tiles to fill the device (128 for N = 8192): clusters of CTAs along k share a
  // tile. DTN_GEMM_SKINNY_KPARTS overrides the count (1, 2 or 4).
  static const int forced_parts = [] {
    const char* text = getenv("DTN_GEMM_SKINNY_KPARTS");
    return text ? atoi(text) : 0;
  }();
  int k_parts = 1;
  if (M <= 16 && K >= 2048) {
    const int64_t tiles = (N + S_BN - 1) / S_BN;
    k_parts = tiles * 2 <= (int64_t)sm_count() * 2 ? 2 : 1;
    if (tiles * 4 <= (int64_t)sm_count() * 2) k_parts = 4;
    if (forced_parts >= 1 && forced_parts <= 4) k_parts = forced_parts;
  }
  int choice = forced;
  if (choice < 1 || choice > 8) {
    // Measured on B200 (us, bf16x3): 128^3 3.1 with 16-row tiles against 5.2 with 64-row tiles, 128x64x256 4.8 / 8.5,
    // 256^3 5.2 / 8.8, 512^3 10.4 (32-row tiles, two k groups) / 15.5, 16x8192x8192 95 (two k groups) / 215.
    // The 16-row single-group configuration keeps the sequential-k accumulation order, so small products stay
    // bit-identical to the reference's emitted kernel.
    const double volume = (double)M * (double)N * (double)K;
    if (M <= 16 && K >= 256) choice = 2;
    else if (volume <= 320.0 * 320.0 * 320.0) choice = 3;
    else if (volume <= 520.0 * 520.0 * 520.0 && M >= 32) {
      // two k groups either way (the same bits); 16-row tiles while they are one wave of CTAs (384^3: 144 CTAs, 5.4 us
      // against 7.1 us for 72 CTAs of 32 rows), 32-row tiles beyond (512^3: 8.8 us against 9.6 us for 256 CTAs of 16 rows)
      const int64_t short_tiles = ((M + 15) / 16) * ((N + S_BN - 1) / S_BN);
      choice = short_tiles <= (int64_t)sm_count() ? 2 : 6;
    }
    else choice = 1;
  }
  switch (choice) {
    case 2: DTN_SMALL_CFG(16, 64, 2);
    case 3: DTN_SMALL_CFG(16, 64, 1);
    case 4: DTN_SMALL_CFG(32, 32, 1);
    case 5: DTN_SMALL_CFG(32, 64, 1);
    case 6: DTN_SMALL_CFG(32, 64, 2);
    case 7: DTN_SMALL_CFG(16, 32, 1);
    case 8: DTN_SMALL_CFG_ST(16, 64, 2, 3);
    default: DTN_SMALL_CFG(64, 32, 1);
  }
#undef DTN_SMALL_CFG
#undef DTN_SMALL_CFG_ST
}

// mode: DTN_GEMM_BF16X3 or DTN_GEMM_TF32X3
int gemm_small_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, cudaStream_t s) {
  return mode == DTN_GEMM_BF16X3 ? gemm_small_launch_mode<0>(A, B, C, M, N, K, lda, ldb, ldc, s)
                                 : gemm_small_launch_mode<1>(A, B, C, M, N, K, lda, ldb, ldc, s);
}

}  // namespace dtn
