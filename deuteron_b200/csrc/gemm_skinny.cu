// Compensated FP32 GEMM with at most 16 rows: one pass over B at memory speed.
//
// C[M <= 16][N] = A[M][K] * B[K][N] is bound by reading B once, and every element of B has to be rounded to a high part
// and a residual on the way (hi = rn(v), lo = rn(v - hi); bf16 pairs or tf32 words), so the kernel is built around
// keeping a deep queue of B in flight per SM and spending as few instructions per element as the fragment layout of
// the warp-level product allows:
//
//   * Work unit: 64 k-rows x 128 columns of B (32 KiB of FP32). The units of the whole product, numbered column block
//     by column block with k fastest, are cut into one contiguous range per CTA (one CTA per SM), whatever N and K
//     are: every SM reads the same number of bytes.
//   * One thread brings each unit in as four TMA boxes of 32 columns (128-byte swizzle), plus the matching 16 x 64
//     tile of A, into a ring of five stages with full/empty mbarriers: 160 KiB of loads in flight per SM, and nothing
//     the issuing thread has to wait for but a free stage. A second warp splits each A tile once, from shared memory
//     into two planes beside it, and reports them on a barrier of their own.
//   * Sixteen compute warps: eight column groups of 16 columns x the lower and the upper 32 k-rows of every unit (a
//     warp's chain of conversions and products is latency-bound, so the SM wants many of them). A thread reads the two columns 2g, 2g+1 of its four k-rows with one
//     8-byte shared-memory load per row (conflict-free under the swizzle), splits them (one packed conversion, two
//     mixed-precision fma, one packed conversion per pair) and issues lo*hi, hi*lo, hi*hi (mma.sync m16n8k16 for bf16,
//     m16n8k8 for tf32) into FP32 accumulators: column 2g feeds one n8 tile, column 2g+1 the other, so that after the
//     products a thread owns four consecutive output columns of rows g and g+8.
//   * A CTA's range ends inside a column block more often than not, and its two k-halves hold separate sums. Each
//     warp writes its 16 x 16 partial sums to the workspace and marks its slot's arrival flag with the launch's token;
//     the warp that then finds every contributor's flag set adds the partial sums of all contributors in (CTA, k-half)
//     order (a fixed order: the result does not depend on who was last) and writes C. Nobody waits for anybody, and
//     nothing in the workspace has to be cleared before a launch.
//
// Every wait on a barrier is bounded (sm100_ptx.cuh); a wait that gives up records where in the device status word.
#include <cuda.h>
#include <stdlib.h>

#include <atomic>
#include <chrono>
#include <mutex>

#include "dtn_common.cuh"
#include "sm100_ptx.cuh"

namespace dtn {

constexpr int K_BN = 128, K_BK = 64;
constexpr int K_STAGES = 5;
constexpr int K_COLUMN_GROUPS = 8;                  // 16 columns each
constexpr int K_WARPS = 16;                         // compute warps: a column group x the lower or upper 32 k-rows of a unit
constexpr int K_THREADS = (K_WARPS + 2) * 32;       // + the warp that issues the loads + the warp that splits A
constexpr int K_B_BYTES = K_BK * K_BN * 4;          // four boxes of [64 rows][32 columns]
constexpr int K_BOX_BYTES = K_BK * 32 * 4;
constexpr int K_A_BYTES = 16 * K_BK * 4;            // the unit's [16 rows][64 k] tile of A as it is in memory

template <int MODE>
struct SkinnyCfg {
  // A planes [16][72]: bf16 elements or tf32 words; with this pitch the fragment reads (4-byte loads of bf16 pairs,
  // 8-byte loads of tf32 word pairs) are free of bank conflicts
  static constexpr int kPitch = 72;
  static constexpr int kPlaneBytes = 16 * kPitch * (MODE == 0 ? 2 : 4);
  static constexpr int kStageBytes = ((K_B_BYTES + K_A_BYTES + 2 * kPlaneBytes + 1023) / 1024) * 1024;   // B | A | A's two planes
  static constexpr int kSmemBytes = K_STAGES * kStageBytes + 256 + 1024;   // + barriers + alignment slack
};

__device__ __forceinline__ void skinny_split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);   // .x (low half) = first value
  hi = *reinterpret_cast<uint32_t*>(&h);
  float ra, rb;
  asm("{\n\t.reg .b16 h0, h1, m;\n\tmov.b32 {h0, h1}, %2;\n\tmov.b16 m, 0xBF80;\n\t"   // m = -1.0: v - hi = hi * m + v, exact
      "fma.rn.f32.bf16 %0, h0, m, %3;\n\tfma.rn.f32.bf16 %1, h1, m, %4;\n\t}"
      : "=f"(ra), "=f"(rb)
      : "r"(hi), "f"(a), "f"(b));
  __nv_bfloat162 l = __floats2bfloat162_rn(ra, rb);
  lo = *reinterpret_cast<uint32_t*>(&l);
}
// hi = rna_tf32(v), lo = rna_tf32(v - hi). The high part is rounded with integer arithmetic: adding half a tf32 unit
// to the bit pattern and clearing the thirteen low bits is round-to-nearest, ties away from zero, and equals
// cvt.rna.tf32.f32 on every one of the 2^32 inputs except NaNs (checked exhaustively on the GPU) -- and the
// conversion instruction runs on a slow pipe, which is what bounds the tf32 form of this kernel. A NaN may come out
// of the integer form as a zero, so the residual, which is NaN whenever v is NaN or infinite, keeps the conversion
// instruction: its NaN reaches every product of the element, as it does with both parts converted.
__device__ __forceinline__ void skinny_split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  hi = (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u;
  const float rest = v - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}
__device__ __forceinline__ void skinny_mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void skinny_mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Range of units of CTA w: [floor(w U / W), floor((w + 1) U / W)); the CTA that holds unit x.
__host__ __device__ __forceinline__ long long skinny_first_unit(long long w, long long units, long long workers) {
  return w * units / workers;
}
__host__ __device__ __forceinline__ int skinny_owner(long long x, long long units, long long workers) {
  return (int)(((x + 1) * workers - 1) / units);
}

template <int MODE /*0 = bf16x3, 1 = tf32x3*/>
__global__ void __launch_bounds__(K_THREADS, 1)
gemm_x3_skinny_kernel(const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_a, float* __restrict__ C, int M, int N,
                      int K, int64_t ldc, float* __restrict__ partials, unsigned long long* __restrict__ flags, unsigned long long token, int c_vec_ok,
                      int* __restrict__ status) {
  using Cfg = SkinnyCfg<MODE>;
  extern __shared__ uint8_t skinny_smem[];
  const uint32_t raw = smem_u32(skinny_smem);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = skinny_smem + (base - raw);
  const uint32_t bar_addr = base + K_STAGES * Cfg::kStageBytes;
  auto full_bar = [&](int s) { return bar_addr + 8u * s; };
  auto empty_bar = [&](int s) { return bar_addr + 8u * (K_STAGES + s); };
  auto planes_bar = [&](int s) { return bar_addr + 8u * (2 * K_STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + K_STAGES * Cfg::kStageBytes + 8 * 3 * K_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + K_BK - 1) / K_BK, n_tiles = (N + K_BN - 1) / K_BN;
  const long long units = (long long)k_tiles * n_tiles, workers = gridDim.x;
  const long long u_begin = skinny_first_unit(blockIdx.x, units, workers), u_end = skinny_first_unit(blockIdx.x + 1, units, workers);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < K_STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);              // the TMA bytes of B and A (the expect_tx arrival)
      ptx::mbar_init(empty_bar(s), K_WARPS + 1);   // one arrival per compute warp + the warp that splits A
      ptx::mbar_init(planes_bar(s), 1);            // A's planes are written
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
    ptx::tma_prefetch_desc(&tm_b);
    ptx::tma_prefetch_desc(&tm_a);
  }
  __syncthreads();

  if (warp == K_WARPS) {
    // ------------------------------------ loads ------------------------------------------------
    if (lane == 0) {
      int i = 0;
      for (long long u = u_begin; u < u_end; ++u, ++i) {
        const int s = i % K_STAGES;
        const uint32_t parity = (uint32_t)(i / K_STAGES) & 1u;
        if (!ptx::mbar_wait(empty_bar(s), parity ^ 1u, abort_flag)) {
          atomicExch(status, 0x5100 | (int)(blockIdx.x & 0xff));
          for (int n = 0; n < 64; ++n) __nanosleep(1000);   // copies already in flight land before this CTA's shared memory goes away
          break;
        }
        const uint32_t stage = base + (uint32_t)s * Cfg::kStageBytes;
        const int nt = (int)(u / k_tiles), kt = (int)(u % k_tiles);
        ptx::mbar_expect_tx(full_bar(s), K_B_BYTES + K_A_BYTES);
#pragma unroll
        for (int b = 0; b < 4; ++b) ptx::tma_load_2d(stage + b * K_BOX_BYTES, &tm_b, nt * K_BN + b * 32, kt * K_BK, full_bar(s));
        ptx::tma_load_2d(stage + K_B_BYTES, &tm_a, kt * K_BK, 0, full_bar(s));
      }
    }
    return;
  }
  if (warp == K_WARPS + 1) {
    // ------------------------------------ split of A -------------------------------------------
    // the unit's tile of A ([16 rows][64 k], rows past M filled with zeros by the load) -> two planes, once per unit
    int i = 0;
    for (long long u = u_begin; u < u_end; ++u, ++i) {
      const int s = i % K_STAGES;
      const uint32_t parity = (uint32_t)(i / K_STAGES) & 1u;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(full_bar(s), parity, abort_flag))) {
        if (lane == 0) atomicExch(status, 0x5300 | (int)(blockIdx.x & 0xff));
        for (int n = 0; n < 64; ++n) __nanosleep(1000);
        return;
      }
      const uint8_t* raw_a = base_ptr + (size_t)s * Cfg::kStageBytes + K_B_BYTES;
      uint8_t* planes = base_ptr + (size_t)s * Cfg::kStageBytes + K_B_BYTES + K_A_BYTES;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = q * 32 + lane, row = v >> 4, kq = (v & 15) * 4;
        const float4 x = *reinterpret_cast<const float4*>(raw_a + (row * K_BK + kq) * 4);
        if constexpr (MODE == 0) {
          uint2 hi, lo;
          skinny_split_bf16(x.x, x.y, hi.x, lo.x);
          skinny_split_bf16(x.z, x.w, hi.y, lo.y);
          *reinterpret_cast<uint2*>(planes + (row * Cfg::kPitch + kq) * 2) = hi;
          *reinterpret_cast<uint2*>(planes + Cfg::kPlaneBytes + (row * Cfg::kPitch + kq) * 2) = lo;
        } else {
          uint4 hi, lo;
          skinny_split_tf32(x.x, hi.x, lo.x);
          skinny_split_tf32(x.y, hi.y, lo.y);
          skinny_split_tf32(x.z, hi.z, lo.z);
          skinny_split_tf32(x.w, hi.w, lo.w);
          *reinterpret_cast<uint4*>(planes + (row * Cfg::kPitch + kq) * 4) = hi;
          *reinterpret_cast<uint4*>(planes + Cfg::kPlaneBytes + (row * Cfg::kPitch + kq) * 4) = lo;
        }
      }
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(planes_bar(s));
        ptx::mbar_arrive(empty_bar(s));   // this warp is done with the stage's copy of A
      }
    }
    return;
  }

  // -------------------------------------- compute ------------------------------------------------
  const int g = lane >> 2, t = lane & 3;
  const int group = warp & (K_COLUMN_GROUPS - 1), k_half = warp / K_COLUMN_GROUPS;
  // this warp's columns inside the unit: 16 * group .. + 15 = box (group >> 1), columns (group & 1) * 16 .. inside the
  // box; the thread reads columns 2g, 2g + 1 of those: 16-byte piece ((group & 1) * 16 + 2g) / 4, byte (2g & 3) * 4 in it
  const uint32_t box_offset = (uint32_t)(group >> 1) * K_BOX_BYTES;
  const uint32_t piece = (uint32_t)(((group & 1) * 16 + 2 * g) >> 2), inside = (uint32_t)((2 * g) & 3) * 4u;
  float acc[2][4];
  auto clear = [&]() {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  };
  clear();

  // Hands the warp's 16 x 16 partial sums of column block nt over: through the workspace, counted in; the last of the
  // contributing CTAs adds them up in CTA order and writes C.
  auto finish_block = [&](int nt) {
    const int first = skinny_owner((long long)nt * k_tiles, units, workers);
    const int last = skinny_owner((long long)(nt + 1) * k_tiles - 1, units, workers);
    const int col = nt * K_BN + group * 16 + 4 * t;
    auto store_c = [&](const float (&v0)[4], const float (&v1)[4]) {   // rows g and g + 8, columns col .. col + 3
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = g + 8 * h;
        if (row >= M) continue;
        const float(&v)[4] = h ? v1 : v0;
        float* p = C + (int64_t)row * ldc + col;
        if (c_vec_ok && col + 3 < N) {
          *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col + e < N) p[e] = v[e];
        }
      }
    };
    // thread's values: rows g / g + 8, columns 4t + {0, 2} from n8 tile 0 and 4t + {1, 3} from tile 1
    float lower[4] = {acc[0][0], acc[1][0], acc[0][1], acc[1][1]};
    float upper[4] = {acc[0][2], acc[1][2], acc[0][3], acc[1][3]};
    // slot of (CTA, k-half, column block): (CTA index + column block index, k-half) is unique, and there are at most
    // workers + n_tiles such sums
    auto slot_of = [&](int w, int h) { return partials + (((size_t)(w + nt) * 2 + h) * K_COLUMN_GROUPS + group) * 256; };   // [16 rows][16 columns]
    float* mine = slot_of((int)blockIdx.x, k_half);
    *reinterpret_cast<float4*>(mine + g * 16 + 4 * t) = make_float4(lower[0], lower[1], lower[2], lower[3]);
    *reinterpret_cast<float4*>(mine + (g + 8) * 16 + 4 * t) = make_float4(upper[0], upper[1], upper[2], upper[3]);
    // Arrival without a counter, so that nothing has to be cleared before the launch: a contributor writes the launch's
    // token into the flag of its slot and then looks at the flags of all the block's contributors. A sequentially
    // consistent fence between the two makes sure that at least one contributor sees every flag set; when two do,
    // both add the same sums in the same order and write the same bits. Whoever adds clears the flags afterwards
    // (a graph replay repeats the token); a flag left over from other use of the workspace is not the token.
    auto flag_of = [&](int w, int h) { return flags + ((size_t)(w + nt) * 2 + h) * K_COLUMN_GROUPS + group; };
    __threadfence();
    __syncwarp();
    if (lane == 0) asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(flag_of((int)blockIdx.x, k_half)), "l"(token) : "memory");
    __syncwarp();
    asm volatile("fence.sc.gpu;" ::: "memory");
    bool all_in = true;
    for (int c = 2 * first + lane; c <= 2 * last + 1; c += 32) {
      unsigned long long seen;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag_of(c >> 1, c & 1)) : "memory");
      all_in = all_in && seen == token;
    }
    if (!__all_sync(0xffffffffu, all_in)) return;   // somebody else will finish this block
    float sum0[4] = {0.f, 0.f, 0.f, 0.f}, sum1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 2 * first; c <= 2 * last + 1; ++c) {
      const float* theirs = slot_of(c >> 1, c & 1);
      const float4 a = __ldcg(reinterpret_cast<const float4*>(theirs + g * 16 + 4 * t));
      const float4 b = __ldcg(reinterpret_cast<const float4*>(theirs + (g + 8) * 16 + 4 * t));
      if (c == 2 * first) {
        sum0[0] = a.x; sum0[1] = a.y; sum0[2] = a.z; sum0[3] = a.w;
        sum1[0] = b.x; sum1[1] = b.y; sum1[2] = b.z; sum1[3] = b.w;
      } else {
        sum0[0] += a.x; sum0[1] += a.y; sum0[2] += a.z; sum0[3] += a.w;
        sum1[0] += b.x; sum1[1] += b.y; sum1[2] += b.z; sum1[3] += b.w;
      }
    }
    store_c(sum0, sum1);
    for (int c = 2 * first + lane; c <= 2 * last + 1; c += 32) *flag_of(c >> 1, c & 1) = 0ull;   // ready for the next launch
  };

  int i = 0;
  for (long long u = u_begin; u < u_end; ++u, ++i) {
    const int s = i % K_STAGES;
    const uint32_t parity = (uint32_t)(i / K_STAGES) & 1u;
    if (!__all_sync(0xffffffffu, ptx::mbar_wait(full_bar(s), parity, abort_flag) && ptx::mbar_wait(planes_bar(s), parity, abort_flag))) {
      if (lane == 0) atomicExch(status, 0x5200 | (int)(blockIdx.x & 0xff));
      for (int n = 0; n < 64; ++n) __nanosleep(1000);
      return;
    }
    const uint32_t b_box = base + (uint32_t)s * Cfg::kStageBytes + box_offset;
    const uint8_t* planes = base_ptr + (size_t)s * Cfg::kStageBytes + K_B_BYTES + K_A_BYTES;
    // 16-byte piece p of row r of a box lies at position p ^ (r & 7) of the row (128-byte swizzle)
    auto b_pair = [&](int row) {
      float2 v;
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                   : "=f"(v.x), "=f"(v.y)
                   : "r"(b_box + (uint32_t)row * 128u + ((piece ^ (uint32_t)(row & 7)) << 4) + inside));
      return v;
    };
    if constexpr (MODE == 0) {
#pragma unroll
      for (int kk = k_half * (K_BK / 2); kk < (k_half + 1) * (K_BK / 2); kk += 16) {
        uint32_t a_hi[4], a_lo[4];
        const uint32_t* hp = reinterpret_cast<const uint32_t*>(planes) + (g * Cfg::kPitch + kk + 2 * t) / 2;
        const uint32_t* lp = hp + Cfg::kPlaneBytes / 4;
        a_hi[0] = hp[0];                        // row g,     k 2t, 2t+1
        a_hi[1] = hp[4 * Cfg::kPitch];          // row g + 8
        a_hi[2] = hp[4];                        // row g,     k 2t+8, 2t+9
        a_hi[3] = hp[4 * Cfg::kPitch + 4];      // row g + 8
        a_lo[0] = lp[0];
        a_lo[1] = lp[4 * Cfg::kPitch];
        a_lo[2] = lp[4];
        a_lo[3] = lp[4 * Cfg::kPitch + 4];
        const float2 r0 = b_pair(kk + 2 * t), r1 = b_pair(kk + 2 * t + 1), r2 = b_pair(kk + 2 * t + 8), r3 = b_pair(kk + 2 * t + 9);
        uint32_t b_hi[2], b_lo[2];
        skinny_split_bf16(r0.x, r1.x, b_hi[0], b_lo[0]);
        skinny_split_bf16(r2.x, r3.x, b_hi[1], b_lo[1]);
        skinny_mma_bf16(acc[0], a_lo, b_hi);
        skinny_mma_bf16(acc[0], a_hi, b_lo);
        skinny_mma_bf16(acc[0], a_hi, b_hi);
        skinny_split_bf16(r0.y, r1.y, b_hi[0], b_lo[0]);
        skinny_split_bf16(r2.y, r3.y, b_hi[1], b_lo[1]);
        skinny_mma_bf16(acc[1], a_lo, b_hi);
        skinny_mma_bf16(acc[1], a_hi, b_lo);
        skinny_mma_bf16(acc[1], a_hi, b_hi);
      }
    } else {
      // m16n8k8: the step's eight k values are rows kk .. kk + 7; slot t of the instruction takes row kk + 2t and slot
      // t + 4 row kk + 2t + 1, for A and B alike, so that B's rows are the conflict-free pattern of the bf16 form
#pragma unroll
      for (int kk = k_half * (K_BK / 2); kk < (k_half + 1) * (K_BK / 2); kk += 8) {
        uint32_t a_hi[4], a_lo[4];
        const uint32_t* hp = reinterpret_cast<const uint32_t*>(planes) + g * Cfg::kPitch + kk + 2 * t;
        const uint32_t* lp = hp + Cfg::kPlaneBytes / 4;
        const uint2 h0 = *reinterpret_cast<const uint2*>(hp), h1 = *reinterpret_cast<const uint2*>(hp + 8 * Cfg::kPitch);
        const uint2 l0 = *reinterpret_cast<const uint2*>(lp), l1 = *reinterpret_cast<const uint2*>(lp + 8 * Cfg::kPitch);
        a_hi[0] = h0.x;   // row g,     slot t
        a_hi[1] = h1.x;   // row g + 8
        a_hi[2] = h0.y;   // row g,     slot t + 4
        a_hi[3] = h1.y;   // row g + 8
        a_lo[0] = l0.x;
        a_lo[1] = l1.x;
        a_lo[2] = l0.y;
        a_lo[3] = l1.y;
        const float2 r0 = b_pair(kk + 2 * t), r1 = b_pair(kk + 2 * t + 1);
        uint32_t b_hi[2], b_lo[2];
        skinny_split_tf32(r0.x, b_hi[0], b_lo[0]);
        skinny_split_tf32(r1.x, b_hi[1], b_lo[1]);
        skinny_mma_tf32(acc[0], a_lo, b_hi);
        skinny_mma_tf32(acc[0], a_hi, b_lo);
        skinny_mma_tf32(acc[0], a_hi, b_hi);
        skinny_split_tf32(r0.y, b_hi[0], b_lo[0]);
        skinny_split_tf32(r1.y, b_hi[1], b_lo[1]);
        skinny_mma_tf32(acc[1], a_lo, b_hi);
        skinny_mma_tf32(acc[1], a_hi, b_lo);
        skinny_mma_tf32(acc[1], a_hi, b_hi);
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(empty_bar(s));
    const int kt = (int)(u % k_tiles);
    if (kt == k_tiles - 1 || u + 1 == u_end) {   // the column block, or this CTA's share of it, is complete
      finish_block((int)(u / k_tiles));
      clear();
    }
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*SkinnyEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static SkinnyEncodeFn skinny_encode_fn() {
  static SkinnyEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<SkinnyEncodeFn>(p);
  });
  return fn;
}

static int skinny_workers(int64_t units) {
  const int64_t sms = sm_count();
  return (int)(units < sms ? units : sms);
}

// Bytes of workspace the kernel needs: two [16][128] blocks of partial sums (one per k-half) per (CTA, column block)
// pair that can occur, then one 8-byte arrival flag per (block of partial sums, column group).
size_t gemm_skinny_workspace_bytes(int64_t N, int64_t K) {
  const int64_t k_tiles = (K + K_BK - 1) / K_BK, n_tiles = (N + K_BN - 1) / K_BN;
  const int64_t slots = skinny_workers(k_tiles * n_tiles) + n_tiles;
  return (size_t)slots * 2 * 16 * K_BN * 4 + (size_t)slots * 2 * K_COLUMN_GROUPS * 8;
}

// A value no earlier launch of this process has used and that is never zero.
static unsigned long long skinny_next_token() {
  static std::atomic<unsigned long long> next{
      (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9E3779B97F4A7C15ull};
  unsigned long long token = next.fetch_add(1) + 1;
  return token ? token : next.fetch_add(1) + 1;
}

// True when the kernel can take the product: at most 16 rows, A and B addressable by tensor maps.
bool gemm_skinny_supported(const float* A, const float* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb) {
  return M >= 1 && M <= 16 && N >= 1 && K >= 1 && aligned_to(A, 16) && lda % 4 == 0 && aligned_to(B, 16) && ldb % 4 == 0 &&
         skinny_encode_fn() != nullptr;
}

template <int MODE>
static int gemm_skinny_launch_mode(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                   int64_t ldc, void* workspace, cudaStream_t s) {
  using Cfg = SkinnyCfg<MODE>;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
  const cuuint64_t strides[1] = {(cuuint64_t)ldb * 4};
  const cuuint32_t box[2] = {32, (cuuint32_t)K_BK};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = skinny_encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(B), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gemm: cuTensorMapEncodeTiled (skinny B) failed with CUresult %d", (int)r);
  const int64_t k_tiles = (K + K_BK - 1) / K_BK, n_tiles = (N + K_BN - 1) / K_BN;
  const int workers = skinny_workers(k_tiles * n_tiles);
  float* partials = static_cast<float*>(workspace);
  unsigned long long* flags = reinterpret_cast<unsigned long long*>(partials + (size_t)(workers + n_tiles) * 2 * 16 * K_BN);
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gemm: could not allocate the device status word");
  CUtensorMap map_a;   // A as [M rows][K]: boxes of 64 k x 16 rows, rows past M read as zeros
  {
    const cuuint64_t a_dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t a_strides[1] = {(cuuint64_t)lda * 4};
    const cuuint32_t a_box[2] = {(cuuint32_t)K_BK, 16};
    r = skinny_encode_fn()(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(A), a_dims, a_strides, a_box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gemm: cuTensorMapEncodeTiled (skinny A) failed with CUresult %d", (int)r);
  }
  const int c_vec = aligned_to(C, 16) && ldc % 4 == 0;
  auto kernel = gemm_x3_skinny_kernel<MODE>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_dev = dev;
  }
  kernel<<<(unsigned)workers, K_THREADS, Cfg::kSmemBytes, s>>>(map, map_a, C, (int)M, (int)N, (int)K, ldc, partials, flags, skinny_next_token(), c_vec, status);
  DTN_LAUNCH_CHECK("gemm_x3_skinny_kernel");
  return DTN_OK;
}

// Host-side copy of the kernel's partition, for inspection and tests (pure arithmetic, no device needed).
int gemm_skinny_plan(int64_t N, int64_t K, int workers, int64_t* unit_begin_out, int* first_out, int* last_out) {
  const int64_t k_tiles = (K + K_BK - 1) / K_BK, n_tiles = (N + K_BN - 1) / K_BN, units = k_tiles * n_tiles;
  DTN_REQUIRE(N >= 1 && K >= 1 && workers >= 1 && workers <= units, DTN_ERR_INVALID,
              "gemm: the skinny plan needs positive extents and between 1 and %lld workers", (long long)units);
  if (unit_begin_out)
    for (int w = 0; w <= workers; ++w) unit_begin_out[w] = skinny_first_unit(w, units, workers);
  for (int64_t nt = 0; nt < n_tiles; ++nt) {
    if (first_out) first_out[nt] = skinny_owner(nt * k_tiles, units, workers);
    if (last_out) last_out[nt] = skinny_owner((nt + 1) * k_tiles - 1, units, workers);
  }
  return DTN_OK;
}

int gemm_skinny_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                       int64_t ldc, void* workspace, cudaStream_t s) {
  return mode == DTN_GEMM_BF16X3 ? gemm_skinny_launch_mode<0>(A, B, C, M, N, K, lda, ldb, ldc, workspace, s)
                                 : gemm_skinny_launch_mode<1>(A, B, C, M, N, K, lda, ldb, ldc, workspace, s);
}

}  // namespace dtn
