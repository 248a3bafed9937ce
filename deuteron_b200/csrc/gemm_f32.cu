// Plain FP32 GEMM (contraction_precision = "f32"): C = A*B with FP32 FMA on the CUDA cores.
// 128x128 CTA tile, 8x8 register micro-tile per thread, K advanced 16 at a time through
// double-buffered shared memory. A is stored transposed in shared memory so that both
// operand reads in the inner loop are conflict-free 128-bit loads. Any M, N, K and any
// leading dimensions; the vector global loads are used when pointers and strides allow.
#include <stdlib.h>

#include "dtn_common.cuh"

namespace dtn {

constexpr int F_BM = 128, F_BN = 128, F_BK = 16, F_THREADS = 256;

template <bool ALIGNED>
__global__ void __launch_bounds__(F_THREADS)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc) {
  __shared__ __align__(16) float As[2][F_BK][F_BM + 4];
  __shared__ __align__(16) float Bs[2][F_BK][F_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * F_BM, n0 = blockIdx.x * F_BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 8 x 8 outputs

  // Global -> register staging assignment.
  // A tile: 128 rows x 16 k  = 512 float4 (along k); thread loads 2.
  // B tile: 16 k x 128 cols = 512 float4 (along n); thread loads 2.
  float4 ra[2], rb[2];
  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int v = tid + i * F_THREADS;   // 0..511
      const int ar = v >> 2, ak = (v & 3) * 4;
      const int gr = m0 + ar, gk = k0 + ak;
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gr < M) {
        const float* p = A + (int64_t)gr * lda + gk;
        if (ALIGNED && gk + 3 < K) {
          t = *reinterpret_cast<const float4*>(p);
        } else {
          if (gk + 0 < K) t.x = p[0];
          if (gk + 1 < K) t.y = p[1];
          if (gk + 2 < K) t.z = p[2];
          if (gk + 3 < K) t.w = p[3];
        }
      }
      ra[i] = t;
      const int bk = v >> 5, bn = (v & 31) * 4;
      const int gkb = k0 + bk, gn = n0 + bn;
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gkb < K) {
        const float* p = B + (int64_t)gkb * ldb + gn;
        if (ALIGNED && gn + 3 < N) {
          u = *reinterpret_cast<const float4*>(p);
        } else {
          if (gn + 0 < N) u.x = p[0];
          if (gn + 1 < N) u.y = p[1];
          if (gn + 2 < N) u.z = p[2];
          if (gn + 3 < N) u.w = p[3];
        }
      }
      rb[i] = u;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int v = tid + i * F_THREADS;
      const int ar = v >> 2, ak = (v & 3) * 4;
      As[buf][ak + 0][ar] = ra[i].x;
      As[buf][ak + 1][ar] = ra[i].y;
      As[buf][ak + 2][ar] = ra[i].z;
      As[buf][ak + 3][ar] = ra[i].w;
      const int bk = v >> 5, bn = (v & 31) * 4;
      *reinterpret_cast<float4*>(&Bs[buf][bk][bn]) = rb[i];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int ktiles = (K + F_BK - 1) / F_BK;
  if (ktiles > 0) {
    load_tiles(0);
    store_tiles(0);
  }
  __syncthreads();
  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ktiles) load_tiles((kt + 1) * F_BK);
#pragma unroll
    for (int k = 0; k < F_BK; ++k) {
      float a[8], b[8];
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
      a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
      b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) store_tiles(buf ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (r >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = n0 + h * 64 + tx * 4;
      float* p = C + (int64_t)r * ldc + c;
      if (ALIGNED && c + 3 < N) {
        *reinterpret_cast<float4*>(p) =
            make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c + j < N) p[j] = acc[i][h * 4 + j];
      }
    }
  }
}

// Small products: 32x32 CTA tiles (2x2 outputs per thread, 256 threads), so that a 128^3 product runs on 16 SMs
// instead of one. The k order per output element is the same sequential FMA chain as in the large-tile kernel, so the
// results are bit-identical to it (and to the reference's f32 kernel).
constexpr int FS_B = 32, FS_BK = 16;

__device__ __forceinline__ void f32_copy_4(uint32_t dst, const void* src, int valid_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(valid_bytes) : "memory");
}

// Few output tiles and a short launch: the time is one CTA's chain of k-tiles. The k-tiles go through a ring of
// FS_STAGES slots filled by cp.async (4-byte copies, so any alignment and any edge: out-of-range elements are
// zero-filled), all slots requested before the first product. One k-tile is a few hundred cycles of arithmetic against
// a global-memory latency of about a thousand: with the next tile alone in flight (registers, as the large-tile kernels
// do) every k-tile cost a full latency, 0.48 us per 16 k.
__global__ void __launch_bounds__(F_THREADS)
gemm_f32_small_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                      int64_t lda, int64_t ldb, int64_t ldc) {
  constexpr int FS_STAGES = 8;
  __shared__ float As[FS_STAGES][FS_BK][FS_B + 1];
  __shared__ float Bs[FS_STAGES][FS_BK][FS_B + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * FS_B, n0 = blockIdx.x * FS_B;
  const int tx = tid & 15, ty = tid >> 4;   // 16 x 16 threads, each 2 x 2 outputs
  auto request_tile = [&](int k0, int slot) {   // 512 elements per operand tile, two per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int v = tid + i * F_THREADS;          // 0..511
      const int ar = v >> 4, ak = v & 15;         // A: 32 rows x 16 k, k fastest in memory, stored [k][row]
      const bool a_in = m0 + ar < M && k0 + ak < K;
      f32_copy_4(smem_u32(&As[slot][ak][ar]), a_in ? (const void*)(A + (int64_t)(m0 + ar) * lda + k0 + ak) : (const void*)A, a_in ? 4 : 0);
      const int bk = v >> 5, bn = v & 31;         // B: 16 k x 32 columns, column fastest
      const bool b_in = k0 + bk < K && n0 + bn < N;
      f32_copy_4(smem_u32(&Bs[slot][bk][bn]), b_in ? (const void*)(B + (int64_t)(k0 + bk) * ldb + n0 + bn) : (const void*)B, b_in ? 4 : 0);
    }
  };
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int ktiles = (K + FS_BK - 1) / FS_BK;
#pragma unroll
  for (int s = 0; s < FS_STAGES - 1; ++s) {
    if (s < ktiles) request_tile(s * FS_BK, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(FS_STAGES - 2) : "memory");
    __syncthreads();   // tile kt has landed for every thread, and everybody is done with the slot requested next
    if (kt + FS_STAGES - 1 < ktiles) request_tile((kt + FS_STAGES - 1) * FS_BK, (kt + FS_STAGES - 1) % FS_STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int buf = kt % FS_STAGES;
#pragma unroll
    for (int k = 0; k < FS_BK; ++k) {
      const float a0 = As[buf][k][ty * 2], a1 = As[buf][k][ty * 2 + 1];
      const float b0 = Bs[buf][k][tx * 2], b1 = Bs[buf][k][tx * 2 + 1];
      acc[0][0] = fmaf(a0, b0, acc[0][0]);
      acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]);
      acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = m0 + ty * 2 + i, c = n0 + tx * 2 + j;
      if (r < M && c < N) C[(int64_t)r * ldc + c] = acc[i][j];
    }
}

// Split k: a cluster of KPARTS CTAs along z shares one 32 x 32 output tile, each CTA takes a contiguous slice of k,
// and the partial sums meet in the first CTA's shared memory (distributed-shared-memory stores into a fixed slot per
// CTA and thread) where they are added in rank order: no atomics, the same bits on every run. Used for contractions
// too small to give the SMs work otherwise (the reference's split-K workload: 128 x 64 outputs, k = 256). Inside a
// CTA the two halves of the threads take the first and the last eight k of every k-tile, 4 x 2 outputs per thread
// from one 128-bit and one 64-bit shared load per k (the 2 x 2 form above needs four loads for four products and is
// bound by them: 850 cycles per k-tile against 150), and the second half's sums are added to the first's before the
// cluster's. The k order of an output element therefore differs from the one-CTA form, which is why the product of
// the reference's 128^3 example never takes this kernel.
constexpr int FK_PITCH = FS_B + 4;   // rows of a k-tile start 16-byte aligned

template <int KPARTS>
__global__ void __launch_bounds__(F_THREADS)
gemm_f32_splitk_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                       int64_t lda, int64_t ldb, int64_t ldc) {
  constexpr int FK_STAGES = KPARTS > 4 ? 3 : 4;   // eight slots of partial sums leave room for three
  __shared__ __align__(16) float As[FK_STAGES][FS_BK][FK_PITCH];
  __shared__ __align__(16) float Bs[FK_STAGES][FS_BK][FK_PITCH];
  __shared__ __align__(16) float partials[KPARTS * (F_THREADS / 2) * 8];   // slot 0: this CTA's second half
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * FS_B, n0 = blockIdx.x * FS_B;
  // this CTA's slice of k: whole k-tiles, the last CTA takes what is left
  const int all_tiles = (K + FS_BK - 1) / FS_BK;
  const int per_part = (all_tiles + KPARTS - 1) / KPARTS;
  const int k_begin = (int)blockIdx.z * per_part * FS_BK;
  const int k_end = min(K, k_begin + per_part * FS_BK);
  const int half = tid >> 7, t = tid & 127;
  const int tx = t & 15, ty = t >> 4;   // 8 x 16 threads, each 4 rows x 2 columns
  auto request_tile = [&](int k0, int slot) {   // 512 elements per operand tile, two per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int v = tid + i * F_THREADS;          // 0..511
      const int ar = v >> 4, ak = v & 15;         // A: 32 rows x 16 k, k fastest in memory, stored [k][row]
      const bool a_in = m0 + ar < M && k0 + ak < k_end;
      f32_copy_4(smem_u32(&As[slot][ak][ar]), a_in ? (const void*)(A + (int64_t)(m0 + ar) * lda + k0 + ak) : (const void*)A, a_in ? 4 : 0);
      const int bk = v >> 5, bn = v & 31;         // B: 16 k x 32 columns, column fastest
      const bool b_in = k0 + bk < k_end && n0 + bn < N;
      f32_copy_4(smem_u32(&Bs[slot][bk][bn]), b_in ? (const void*)(B + (int64_t)(k0 + bk) * ldb + n0 + bn) : (const void*)B, b_in ? 4 : 0);
    }
  };
  float acc[4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = 0.f;
  const int ktiles = k_end > k_begin ? (k_end - k_begin + FS_BK - 1) / FS_BK : 0;
#pragma unroll
  for (int s = 0; s < FK_STAGES - 1; ++s) {
    if (s < ktiles) request_tile(k_begin + s * FS_BK, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(FK_STAGES - 2) : "memory");
    __syncthreads();   // tile kt has landed for every thread, and everybody is done with the slot requested next
    if (kt + FK_STAGES - 1 < ktiles) request_tile(k_begin + (kt + FK_STAGES - 1) * FS_BK, (kt + FK_STAGES - 1) % FK_STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int buf = kt % FK_STAGES;
#pragma unroll
    for (int kk = 0; kk < FS_BK / 2; ++kk) {
      const int k = half * (FS_BK / 2) + kk;
      const float4 a4 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float2 b2 = *reinterpret_cast<const float2*>(&Bs[buf][k][tx * 2]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i][0] = fmaf(a[i], b2.x, acc[i][0]);
        acc[i][1] = fmaf(a[i], b2.y, acc[i][1]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // second half -> first half of this CTA
  if (half == 1) {
    float4* mine = reinterpret_cast<float4*>(partials + t * 8);
    mine[0] = make_float4(acc[0][0], acc[0][1], acc[1][0], acc[1][1]);
    mine[1] = make_float4(acc[2][0], acc[2][1], acc[3][0], acc[3][1]);
  }
  __syncthreads();
  const int part = (int)blockIdx.z;
  if (half == 0) {
    const float* theirs = partials + t * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e >> 1][e & 1] += theirs[e];
    if (part != 0) {   // this CTA's sums -> slot `part` of the first CTA
      const uint32_t local = smem_u32(partials + (part * (F_THREADS / 2) + t) * 8);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(local));
#pragma unroll
      for (int e = 0; e < 8; e += 4)
        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + 4u * e), "f"(acc[e >> 1][0]),
                     "f"(acc[e >> 1][1]), "f"(acc[(e >> 1) + 1][0]), "f"(acc[(e >> 1) + 1][1])
                     : "memory");
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (part != 0 || half != 0) return;
  for (int other = 1; other < KPARTS; ++other) {
    const float4* theirs = reinterpret_cast<const float4*>(partials + (other * (F_THREADS / 2) + t) * 8);
    const float4 lo = theirs[0], hi = theirs[1];
    acc[0][0] += lo.x; acc[0][1] += lo.y; acc[1][0] += lo.z; acc[1][1] += lo.w;
    acc[2][0] += hi.x; acc[2][1] += hi.y; acc[3][0] += hi.z; acc[3][1] += hi.w;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 2 + j;
      if (r < M && c < N) C[(int64_t)r * ldc + c] = acc[i][j];
    }
}

template <int KPARTS>
static int launch_small_split(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                              int64_t ldc, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((N + FS_B - 1) / FS_B), (unsigned)((M + FS_B - 1) / FS_B), KPARTS);
  cfg.blockDim = dim3(F_THREADS);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = KPARTS;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DTN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_f32_splitk_kernel<KPARTS>, A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc));
  return DTN_OK;
}

// Mid-size products: 64x64 CTA tiles, 4x4 outputs per thread, several CTAs per SM. A 1024^3 product is 64 tiles of
// 128x128 (under half of the SMs) but 256 of these. Same sequential FMA chain per output element.
constexpr int FM_B = 64, FM_BK = 16;

template <bool ALIGNED>
__global__ void __launch_bounds__(F_THREADS)
gemm_f32_mid_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                    int64_t lda, int64_t ldb, int64_t ldc) {
  __shared__ __align__(16) float As[2][FM_BK][FM_B + 4];   // transposed: [k][row]
  __shared__ __align__(16) float Bs[2][FM_BK][FM_B + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * FM_B, n0 = blockIdx.x * FM_B;
  const int tx = tid & 15, ty = tid >> 4;   // 16 x 16 threads, each 4 x 4 outputs
  // staging: each operand tile is 256 float4, one per thread (A along k, B along n)
  const int ar = tid >> 2, ak = (tid & 3) * 4;
  const int bk = tid >> 4, bn = (tid & 15) * 4;
  float4 ra, rb;
  auto load_tiles = [&](int k0) {
    ra = make_float4(0.f, 0.f, 0.f, 0.f);
    rb = ra;
    const int gr = m0 + ar, gk = k0 + ak;
    if (gr < M) {
      const float* p = A + (int64_t)gr * lda + gk;
      if (ALIGNED && gk + 3 < K) {
        ra = *reinterpret_cast<const float4*>(p);
      } else {
        if (gk + 0 < K) ra.x = p[0];
        if (gk + 1 < K) ra.y = p[1];
        if (gk + 2 < K) ra.z = p[2];
        if (gk + 3 < K) ra.w = p[3];
      }
    }
    const int gkb = k0 + bk, gn = n0 + bn;
    if (gkb < K) {
      const float* p = B + (int64_t)gkb * ldb + gn;
      if (ALIGNED && gn + 3 < N) {
        rb = *reinterpret_cast<const float4*>(p);
      } else {
        if (gn + 0 < N) rb.x = p[0];
        if (gn + 1 < N) rb.y = p[1];
        if (gn + 2 < N) rb.z = p[2];
        if (gn + 3 < N) rb.w = p[3];
      }
    }
  };
  auto store_tiles = [&](int buf) {
    As[buf][ak + 0][ar] = ra.x;
    As[buf][ak + 1][ar] = ra.y;
    As[buf][ak + 2][ar] = ra.z;
    As[buf][ak + 3][ar] = ra.w;
    *reinterpret_cast<float4*>(&Bs[buf][bk][bn]) = rb;
  };
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int ktiles = (K + FM_BK - 1) / FM_BK;
  if (ktiles > 0) {
    load_tiles(0);
    store_tiles(0);
  }
  __syncthreads();
  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ktiles) load_tiles((kt + 1) * FM_BK);
#pragma unroll
    for (int k = 0; k < FM_BK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) store_tiles(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i, c = n0 + tx * 4;
    if (r >= M) continue;
    float* p = C + (int64_t)r * ldc + c;
    if (ALIGNED && c + 3 < N) {
      *reinterpret_cast<float4*>(p) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < N) p[j] = acc[i][j];
    }
  }
}

int gemm_f32_launch(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t s, bool split_k_allowed) {
  static const int forced_tile = [] {
    const char* text = getenv("DTN_GEMM_F32_TILE");   // tuning aid: 32, 64 or 128 forces that tile
    return text ? atoi(text) : 0;
  }();
  const int64_t tiles64 = ((M + FM_B - 1) / FM_B) * ((N + FM_B - 1) / FM_B);
  const int64_t tiles128 = ((M + F_BM - 1) / F_BM) * ((N + F_BN - 1) / F_BN);
  // The tile is the largest that still gives every SM work: 32x32 while 64x64 tiles would cover at most half of the
  // SMs, 64x64 while 128x128 tiles would cover under three quarters of them, 128x128 beyond.
  int tile = forced_tile == 32 || forced_tile == 64 || forced_tile == 128 ? forced_tile
             : tiles64 * 2 <= (int64_t)sm_count()                        ? 32
             : tiles128 * 4 < (int64_t)sm_count() * 3                    ? 64
                                                                         : 128;
  if (tile == 32 && (M + FS_B - 1) / FS_B > 65535) tile = 64;
  if (tile == 64 && (M + FM_B - 1) / FM_B > 65535) tile = 128;
  if (tile == 32) {
    dim3 small_grid((unsigned)((N + FS_B - 1) / FS_B), (unsigned)((M + FS_B - 1) / FS_B));
    // A handful of tiles with a long k (the reference's split-K workload is 8 tiles of k = 256): clusters of 4 or 8
    // CTAs along k put 32 or 64 SMs to work instead of 8. Only when the caller allows another k order
    // (`split_k_allowed`: contractions the reference itself computes with atomic partial sums).
    const int64_t tiles32 = (int64_t)small_grid.x * small_grid.y;
    static const int parts_limit = [] {
      const char* text = getenv("DTN_GEMM_F32_KPARTS");   // tuning aid: 1 or 4 caps the k-split
      return text ? atoi(text) : 8;
    }();
    if (split_k_allowed && parts_limit >= 8 && tiles32 * 8 <= (int64_t)sm_count() && K >= 8 * FS_BK * 2 && small_grid.y <= 65535)
      return launch_small_split<8>(A, B, C, M, N, K, lda, ldb, ldc, s);
    if (split_k_allowed && parts_limit >= 4 && tiles32 * 4 <= (int64_t)sm_count() && K >= 4 * FS_BK * 2 && small_grid.y <= 65535)
      return launch_small_split<4>(A, B, C, M, N, K, lda, ldb, ldc, s);
    gemm_f32_small_kernel<<<small_grid, F_THREADS, 0, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
    DTN_LAUNCH_CHECK("gemm_f32_small_kernel");
    return DTN_OK;
  }
  dim3 grid((unsigned)((N + F_BN - 1) / F_BN), (unsigned)((M + F_BM - 1) / F_BM));
  DTN_REQUIRE(grid.y <= 65535, DTN_ERR_UNSUPPORTED, "gemm f32: M too large");
  const bool aligned = aligned_to(A, 16) && aligned_to(B, 16) && aligned_to(C, 16) && lda % 4 == 0 &&
                       ldb % 4 == 0 && ldc % 4 == 0;
  if (tile == 64) {
    dim3 mid_grid((unsigned)((N + FM_B - 1) / FM_B), (unsigned)((M + FM_B - 1) / FM_B));
    if (aligned)
      gemm_f32_mid_kernel<true><<<mid_grid, F_THREADS, 0, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
    else
      gemm_f32_mid_kernel<false><<<mid_grid, F_THREADS, 0, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
    DTN_LAUNCH_CHECK("gemm_f32_mid_kernel");
    return DTN_OK;
  }
  if (aligned)
    gemm_f32_kernel<true><<<grid, F_THREADS, 0, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
  else
    gemm_f32_kernel<false><<<grid, F_THREADS, 0, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc);
  DTN_LAUNCH_CHECK("gemm_f32_kernel");
  return DTN_OK;
}

}  // namespace dtn
