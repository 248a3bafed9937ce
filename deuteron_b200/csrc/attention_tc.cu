// Grouped-query attention forward on the sm_100a tensor cores (f16 storage, head_dim 128).
//
// A work item is 256 query rows of one query head (two 128-row tiles); its keys are walked 128 at a
// time. Every product is a tcgen05.mma with FP32 accumulation in tensor memory:
//   S_t = Q_t * K_j^T          f16 x f16 products are exact; 128x128 FP32 scores per tile
//   O_t += P_t * V_j           the FP32 probabilities are split into an f16 high part and an f16
//                              residual (two products), which keeps ~22 bits of each weight
// The online-softmax recurrence runs in FP32 on the CUDA cores: one thread owns one query row
// (one tensor-memory lane), so the row max and row sum need no shuffles; exp is ex2 of the
// scaled difference. The probabilities are written back over the scores in tensor memory and
// read from there as the A operand of the second product. The output accumulator is rescaled
// lazily: only when a row's maximum has grown by more than 2^8 since the last rescale.
//
// Per tile one or two softmax warpgroups (softmax + output); one warp issues the TMA loads (the
// queries of each work item, and a two-slot ring of K and V tiles); one warp issues the MMAs.
// While one tile's softmax runs, the tensor core works on the other tile. The kernel is
// persistent: one CTA per SM walks the work items (256 query rows of one head each) as a single
// stream of key steps, so the output of one item is normalised and stored while the products of
// the next are already running.
//
// Tensor-memory columns: [0,128) scores/probabilities of tile 0, [128,256) of tile 1,
// [256,384) output of tile 0, [384,512) output of tile 1.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>

#include <mutex>

#include "dtn_common.cuh"
#include "sm100_ptx.cuh"

namespace dtn {

constexpr int attn_threads(int split) { return (8 * split + 2) * 32; }   // softmax warps + TMA warp + MMA warp
constexpr int A_BM = 128;          // query rows per tile (two tiles per CTA)
constexpr int A_BN = 128;          // keys per step
constexpr int A_D = 128;           // head dimension
constexpr int A_HALF_BYTES = 128 * 128;           // one [128 rows][64 f16] swizzled block
constexpr int A_TILE_BYTES = 2 * A_HALF_BYTES;    // one [128][128] f16 tile
constexpr int A_KV_STAGES = 2;
constexpr int A_SMEM_TILES = 2 /*Q*/ + 2 * A_KV_STAGES /*K,V*/;
constexpr int A_XCHG_BYTES = 2 * 2 * 128 * 8;   // [tile][column share][row] (value, sequence) slots
constexpr int A_STAGE_BYTES = 16 * 1024;        // 1 KiB of output staging per softmax warp (at most 16 of them)
constexpr int A_SMEM_BYTES = A_SMEM_TILES * A_TILE_BYTES + 256 + A_XCHG_BYTES + A_STAGE_BYTES + 1024;
constexpr float A_RESCALE_THRESHOLD = 8.0f;   // in log2 units
constexpr float A_BIAS = 4.0f;                // probabilities are kept scaled by 2^4 (f16 residuals stay normal)

// Shared-memory descriptor of an MN-major operand (V tile: rows = keys, 128-byte rows of 64
// head-dimension elements, 128-byte swizzle). The 64-element blocks along the head dimension are
// A_HALF_BYTES apart (leading offset); groups of 8 keys are 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)(A_HALF_BYTES >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// max(a, b, c) in one instruction (sm_100 has a three-input FP32 max).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// idesc: f16 operands, FP32 accumulate, M = 128, N = 128; b_mn = 1 when B is MN-major.
__host__ __device__ constexpr uint32_t attn_idesc(int b_mn) {
  return ptx::umma_idesc(0, 128, 128) | ((uint32_t)b_mn << 16);
}

// Hands `value` to the thread that owns the other column share of the same row and returns that
// thread's value in `other`. A slot holds (value, sequence number); the 8-byte store makes both
// visible together. The wait is bounded like every other wait in this file.
__device__ __forceinline__ bool exchange_with_peer(volatile float2* mine, volatile float2* theirs, float value, int seq,
                                                   volatile int* abort_flag, float& other) {
  float2 packed = make_float2(value, __int_as_float(seq));
  asm volatile("st.volatile.shared.v2.f32 [%0], {%1, %2};" ::"r"(smem_u32((const void*)mine)), "f"(packed.x), "f"(packed.y)
               : "memory");
  const uint32_t addr = smem_u32((const void*)theirs);
  const long long start = clock64();
  while (true) {
    float a, b;
    asm volatile("ld.volatile.shared.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "r"(addr) : "memory");
    if (__float_as_int(b) == seq) {
      other = a;
      return true;
    }
    if (*abort_flag) return false;
    if (clock64() - start > ptx::kWaitBudgetCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Work items: one item = 256 query rows of one query head. A CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...
// and runs them as ONE stream of key steps: barrier phases, the K/V ring and the exchange sequence numbers keep
// counting across items, so the next item's first products are issued while the previous item's output is still being
// written (the per-item prologue, pipeline fill and output no longer leave the tensor core idle). With as many CTAs
// as items the kernel degenerates to one item per CTA.
struct AttnItem {
  int q_row0;     // first query row in the [B*Hq*S, D] view
  int kv_row0;    // first key row in the [B*Hkv*S, D] view
};
__device__ __forceinline__ AttnItem attn_item(int item, int qblocks, int Hq, int Hkv, int S, int group_begin) {
  const int heads_per_group = Hq / Hkv;
  const int head_local = item / qblocks, qb = item % qblocks;
  const int group = group_begin + head_local / heads_per_group;
  const int b = group / Hkv, hkv = group % Hkv;
  const int hq = hkv * heads_per_group + head_local % heads_per_group;
  AttnItem it;
  it.q_row0 = (b * Hq + hq) * S + qb * (2 * A_BM);
  it.kv_row0 = (b * Hkv + hkv) * S;
  return it;
}

template <int SPLIT /*warpgroups per 128-row tile: 1 or 2*/>
__global__ void __launch_bounds__(attn_threads(SPLIT), 1)
gqa_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, float* __restrict__ out, int Hq, int Hkv, int S,
              float scale_log2e, int group_begin, int total_items, int early_pv, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t q_addr = base;                                   // 2 tiles
  const uint32_t k_addr = base + 2 * A_TILE_BYTES;                // A_KV_STAGES tiles
  const uint32_t v_addr = k_addr + A_KV_STAGES * A_TILE_BYTES;    // A_KV_STAGES tiles
  const uint32_t bar_addr = base + A_SMEM_TILES * A_TILE_BYTES;
  uint8_t* bar_ptr = base_ptr + A_SMEM_TILES * A_TILE_BYTES;
  // barrier slots
  auto q_full = [&](int t) { return bar_addr + 8u * (0 + t); };
  auto k_full = [&](int s) { return bar_addr + 8u * (2 + s); };
  auto v_full = [&](int s) { return bar_addr + 8u * (4 + s); };
  auto k_empty = [&](int s) { return bar_addr + 8u * (6 + s); };
  auto v_empty = [&](int s) { return bar_addr + 8u * (8 + s); };
  auto s_full = [&](int t) { return bar_addr + 8u * (10 + t); };
  auto p_half = [&](int t, int h) { return bar_addr + 8u * (12 + 2 * t + h); };   // half of a tile's probabilities is in tensor memory
  auto o_done = [&](int t) { return bar_addr + 8u * (16 + t); };
  auto q_empty = [&](int t) { return bar_addr + 8u * (18 + t); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * 20 + 8);
  volatile float2* xchg = reinterpret_cast<volatile float2*>(bar_ptr + 256);
  float* stage_base = reinterpret_cast<float*>(bar_ptr + 256 + A_XCHG_BYTES);   // 1 KiB per softmax warp
  constexpr int kTmaWarp = 8 * SPLIT, kMmaWarp = 8 * SPLIT + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblocks = S / (2 * A_BM);
  const int num_kv = S / A_BN;
  const int my_items = ((int)blockIdx.x < total_items) ? (total_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total_steps = my_items * num_kv;

  for (int i = threadIdx.x; i < 2 * 2 * 128; i += blockDim.x) {   // sequence 0 = empty
    xchg[i].x = 0.f;
    xchg[i].y = 0.f;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < A_KV_STAGES; ++s) {
      ptx::mbar_init(k_full(s), 1);
      ptx::mbar_init(v_full(s), 1);
      ptx::mbar_init(k_empty(s), 1);
      ptx::mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(q_full(t), 1);
      ptx::mbar_init(q_empty(t), 1);
      ptx::mbar_init(s_full(t), 1);
      ptx::mbar_init(p_half(t, 0), 4 * SPLIT);   // one arrival per softmax warp
      ptx::mbar_init(p_half(t, 1), 4 * SPLIT);
      ptx::mbar_init(o_done(t), 1);
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
    ptx::tma_prefetch_desc(&tm_q);
    ptx::tma_prefetch_desc(&tm_k);
    ptx::tma_prefetch_desc(&tm_v);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc<1>(smem_u32(tmem_holder), 512);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == kTmaWarp) {
    // ------------------------------------ TMA producer ---------------------------------------
    if (lane == 0) {
      int g = 0;
      bool ok = true;
      for (int it = 0; it < my_items && ok; ++it) {
        const AttnItem item = attn_item((int)blockIdx.x + it * (int)gridDim.x, qblocks, Hq, Hkv, S, group_begin);
        for (int j = 0; j < num_kv; ++j, ++g) {
          const int s = g % A_KV_STAGES;
          const uint32_t ph = (uint32_t)(g / A_KV_STAGES) & 1u;
          if (!ptx::mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1100); ok = false; break; }
          ptx::mbar_expect_tx(k_full(s), A_TILE_BYTES);
          for (int h = 0; h < 2; ++h)
            ptx::tma_load_2d(k_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_k, h * 64, item.kv_row0 + j * A_BN, k_full(s));
          if (!ptx::mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1200); ok = false; break; }
          ptx::mbar_expect_tx(v_full(s), A_TILE_BYTES);
          for (int h = 0; h < 2; ++h)
            ptx::tma_load_2d(v_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_v, h * 64, item.kv_row0 + j * A_BN, v_full(s));
          if (j == 0) {
            // this item's queries, after its first keys so that the K/V stream never waits for a query buffer;
            // a buffer is free once the previous item's last score product has read it
            for (int t = 0; t < 2 && ok; ++t) {
              if (it > 0 && !ptx::mbar_wait(q_empty(t), (uint32_t)(it - 1) & 1u, abort_flag)) { atomicExch(status, 0x1300); ok = false; break; }
              ptx::mbar_expect_tx(q_full(t), A_TILE_BYTES);
              for (int h = 0; h < 2; ++h)
                ptx::tma_load_2d(q_addr + t * A_TILE_BYTES + h * A_HALF_BYTES, &tm_q, h * 64, item.q_row0 + t * A_BM, q_full(t));
            }
            if (!ok) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------ MMA issuer -----------------------------------------
    if (lane == 0 && total_steps > 0) {
      constexpr uint32_t kIdescQK = attn_idesc(0);
      constexpr uint32_t kIdescPV = attn_idesc(1);
      bool ok = true;
      // S_t = Q_t K^T : 8 k-steps of 16 along the head dimension (two 64-element swizzled halves)
      auto issue_qk = [&](int t, int s) {
        const uint32_t qa = q_addr + t * A_TILE_BYTES, ka = k_addr + s * A_TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * A_HALF_BYTES + (uint32_t)(kk & 3) * 32u;
          ptx::umma_ss<0, 1>(tmem_base + (uint32_t)(t * 128), ptx::umma_desc_sw128(qa + off),
                             ptx::umma_desc_sw128(ka + off), kIdescQK, kk ? 1u : 0u);
        }
      };
      // O_t += P_t V : 8 k-steps of 16 keys; per step the high and the residual plane of P. The probabilities arrive
      // in two halves (the 32-key chunks every softmax warpgroup finishes first, then the rest), so the products of
      // the first half run while the second is still being computed: half h covers k-steps kk with
      // ((kk >> 1) / chunks-per-warpgroup-half) matching the order the warpgroups write their chunks.
      auto issue_pv = [&](int t, int s, bool first, int half) {
        const uint32_t va = v_addr + s * A_TILE_BYTES;
        const uint32_t o_tmem = tmem_base + (uint32_t)(256 + t * 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // SPLIT == 2: warpgroup 0 writes chunks 0, 1 and warpgroup 1 chunks 2, 3 -> halves {0, 2} and {1, 3};
          // SPLIT == 1: one warpgroup writes chunks 0..3 in order -> halves {0, 1} and {2, 3}
          const int chunk = SPLIT == 2 ? 2 * (i >> 1) + half : 2 * half + (i >> 1);
          const int kk = 2 * chunk + (i & 1);
          const uint32_t p_col = tmem_base + (uint32_t)(t * 128 + 32 * (kk >> 1) + 8 * (kk & 1));
          const uint64_t vd = umma_desc_mn_sw128(va + (uint32_t)kk * 2048u);
          ptx::umma_ts_f16(o_tmem, p_col + 16u, vd, kIdescPV, (first && half == 0 && i == 0) ? 0u : 1u);  // residual first
          ptx::umma_ts_f16(o_tmem, p_col, vd, kIdescPV, 1u);
        }
      };
      // scores of tile t for global step g + 1 (the next step of this item, or the first of the next item)
      auto next_scores = [&](int t, int g) -> bool {
        const int gn = g + 1, jn = gn % num_kv, sn = gn % A_KV_STAGES;
        if (jn == 0 && !ptx::mbar_wait(q_full(t), (uint32_t)(gn / num_kv) & 1u, abort_flag)) { atomicExch(status, 0x2100 | t); return false; }
        if (t == 0 && !ptx::mbar_wait(k_full(sn), (uint32_t)(gn / A_KV_STAGES) & 1u, abort_flag)) { atomicExch(status, 0x2500); return false; }
        ptx::tc_fence_after();
        issue_qk(t, sn);
        ptx::umma_commit<1>(s_full(t));
        if (t == 1) ptx::umma_commit<1>(k_empty(sn));
        if (jn == num_kv - 1) ptx::umma_commit<1>(q_empty(t));   // the item's last read of this query tile
        return true;
      };
      ok = next_scores(0, -1) && next_scores(1, -1);
      for (int g = 0; g < total_steps && ok; ++g) {
        const int s = g % A_KV_STAGES, j = g % num_kv;
        const uint32_t ph = (uint32_t)(g / A_KV_STAGES) & 1u;
        const bool more = g + 1 < total_steps, first = j == 0, last = j == num_kv - 1;
        if (!ptx::mbar_wait(v_full(s), ph, abort_flag)) { atomicExch(status, 0x2300); break; }
        if (!ptx::mbar_wait(p_half(0, 0), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2400); break; }
        ptx::tc_fence_after();
        if (early_pv) issue_pv(0, s, first, 0);
        if (!ptx::mbar_wait(p_half(0, 1), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2400); break; }
        ptx::tc_fence_after();
        if (!early_pv) issue_pv(0, s, first, 0);
        issue_pv(0, s, first, 1);
        if (last) ptx::umma_commit<1>(o_done(0));
        if (more && !next_scores(0, g)) break;
        if (!ptx::mbar_wait(p_half(1, 0), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2600); break; }
        ptx::tc_fence_after();
        if (early_pv) issue_pv(1, s, first, 0);
        if (!ptx::mbar_wait(p_half(1, 1), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2600); break; }
        ptx::tc_fence_after();
        if (!early_pv) issue_pv(1, s, first, 0);
        issue_pv(1, s, first, 1);
        ptx::umma_commit<1>(v_empty(s));
        if (last) ptx::umma_commit<1>(o_done(1));
        if (more && !next_scores(1, g)) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax + output -----------------------------------
    // SPLIT warpgroups share one tile: each owns 128 / SPLIT score columns (and the same share of
    // the output columns) of all 128 rows. Partner threads of a row agree on the row maximum
    // through a shared-memory slot (bounded spin, no block-wide barrier).
    constexpr int kChunks = 4 / SPLIT;             // 32-column chunks per thread
    const int t = warp / (4 * SPLIT);              // tile
    const int part = (warp >> 2) % SPLIT;          // column share of this warpgroup
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int c0 = part * kChunks;
    const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_field + (uint32_t)(t * 128);
    const uint32_t o_tmem = tmem_base + lane_field + (uint32_t)(256 + t * 128);
    volatile float2* my_slot = xchg + ((t * 2 + part) * 128 + row_in_tile);
    volatile float2* peer_slot = xchg + ((t * 2 + (part ^ 1)) * 128 + row_in_tile);
    float* stage = stage_base + warp * 256;   // [32 rows][8 floats], 16-byte pieces swapped on every other group of 4 rows
    float m_used = -INFINITY;   // log2-domain maximum the current probabilities are scaled by
    float mass = 0.f;
    for (int g = 0; g < total_steps; ++g) {
      const int j = g % num_kv;
      if (j == 0) {   // a new item starts
        m_used = -INFINITY;
        mass = 0.f;
      }
      const bool ready = ptx::mbar_wait(s_full(t), (uint32_t)g & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) atomicExch(status, 0x3100 | t);
        break;
      }
      ptx::tc_fence_after();
      // pass 1: row maximum of the raw scores (three-input max: two scores per instruction)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(s_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      }
      if constexpr (SPLIT == 2) {
        float other;
        const bool got = exchange_with_peer(my_slot, peer_slot, mx, 2 * g + 1, abort_flag, other);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) atomicExch(status, 0x3300 | t);
          break;
        }
        mx = fmaxf(mx, other);
      }
      const float mx2 = mx * scale_log2e;
      const bool grow = (j == 0) || (mx2 > m_used + A_RESCALE_THRESHOLD);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx2 : m_used;
        const float alpha = (j == 0) ? 0.f : ex2_approx_ftz(m_used - m_new);   // 1 when this row does not grow
        if (j > 0) {
          // All earlier products into O_t are complete: s_full(t) of this step was committed after them.
#pragma unroll 1
          for (int c = c0; c < c0 + kChunks; ++c) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(o_tmem + (uint32_t)(c * 32), r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            ptx::tmem_st_32x32(o_tmem + (uint32_t)(c * 32), r);
          }
          ptx::tmem_st_wait();
        }
        mass *= alpha;
        m_used = m_new;
      }
      // pass 2: probabilities, row sum, f16 high/residual split written over the scores
      const float shift = A_BIAS - m_used;
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32], w[32];
        ptx::tmem_ld_32x32(s_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2_approx_ftz(fmaf(__uint_as_float(r[2 * i]), scale_log2e, shift));
          const float p1 = ex2_approx_ftz(fmaf(__uint_as_float(r[2 * i + 1]), scale_log2e, shift));
          mass += p0 + p1;
          const __half2 hi = __floats2half2_rn(p0, p1);
          const float2 back = __half22float2(hi);
          const __half2 lo = __floats2half2_rn(p0 - back.x, p1 - back.y);
          w[i] = *reinterpret_cast<const uint32_t*>(&hi);
          w[16 + i] = *reinterpret_cast<const uint32_t*>(&lo);
        }
        ptx::tmem_st_32x32(s_tmem + (uint32_t)(c * 32), w);
        if (((c - c0 + 1) % (kChunks / 2)) == 0) {   // this warp's share of one half is in tensor memory
          ptx::tmem_st_wait();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(p_half(t, (c - c0) / (kChunks / 2)));
        }
      }
      if (j != num_kv - 1) continue;

      // ---- the item's last step: normalise and store its output while the tensor core already works on the other
      // tile and on the next item's scores (the next item's first product into O_t waits for this warp's next arrival
      // on p_half, which comes after the reads below) ----
      const int it = g / num_kv;
      bool done = ptx::mbar_wait(o_done(t), (uint32_t)it & 1u, abort_flag);
      if constexpr (SPLIT == 2) {
        float other = 0.f;
        done = done && exchange_with_peer(my_slot, peer_slot, mass, 2 * g + 2, abort_flag, other);
        mass += other;
      }
      if (!__all_sync(0xffffffffu, done)) {
        if (lane == 0) atomicExch(status, 0x3200 | t);
        break;
      }
      ptx::tc_fence_after();
      const float inv = 1.0f / mass;
      const AttnItem item = attn_item((int)blockIdx.x + it * (int)gridDim.x, qblocks, Hq, Hkv, S, group_begin);
      float* obase = out + ((int64_t)item.q_row0 + t * A_BM + quarter * 32) * A_D;
      // Each thread owns one row in tensor memory, but a warp-wide store should cover whole 32-byte sectors of
      // several rows: 8 columns of the warp's 32 rows go through a 1 KiB staging block (16-byte pieces swapped on
      // every other group of four rows, so neither side has bank conflicts) and come back 16 rows per instruction.
      const int wr_swap = (lane >> 2) & 1;
      const int rd_row = lane >> 1, rd_piece = lane & 1;
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(o_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
            *reinterpret_cast<float4*>(stage + lane * 8 + 4 * (i ^ wr_swap)) =
                make_float4(__uint_as_float(r[8 * sub + 4 * i]) * inv, __uint_as_float(r[8 * sub + 4 * i + 1]) * inv,
                            __uint_as_float(r[8 * sub + 4 * i + 2]) * inv, __uint_as_float(r[8 * sub + 4 * i + 3]) * inv);
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int rloc = rd_row + 16 * h;
            const float4 val = *reinterpret_cast<const float4*>(stage + rloc * 8 + 4 * (rd_piece ^ ((rloc >> 2) & 1)));
            *reinterpret_cast<float4*>(obase + (int64_t)rloc * A_D + c * 32 + sub * 8 + 4 * rd_piece) = val;
          }
          __syncwarp();
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn attn_encode_fn() {
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

// [rows, 128] f16 matrix, box = 64 columns (128 bytes) x 128 rows, 128-byte swizzle.
static int make_rows_map(CUtensorMap* map, const void* base, int64_t rows) {
  EncodeTiledFn enc = attn_encode_fn();
  DTN_REQUIRE(enc != nullptr, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)A_D, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)A_D * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DTN_OK;
}

bool gqa_tc_supported(int64_t S, int64_t D, int storage) {
  return storage == DTN_STORAGE_F16 && D == A_D && S >= 2 * A_BM && S % (2 * A_BM) == 0;
}

template <int SPLIT>
static int gqa_tc_launch_t(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                           int64_t S, float scale, int64_t gb, int64_t ge, cudaStream_t s) {
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_rows_map(&mq, q, B * Hq * S))) return rc;
  if ((rc = make_rows_map(&mk, k, B * Hkv * S))) return rc;
  if ((rc = make_rows_map(&mv, v, B * Hkv * S))) return rc;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(gqa_tc_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, A_SMEM_BYTES));
    attr_dev = dev;
  }
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gqa: could not allocate the device status word");
  const int64_t items = (ge - gb) * (Hq / Hkv) * (S / (2 * A_BM));
  DTN_REQUIRE(items < (1LL << 31) && B * Hq * S < (1LL << 31), DTN_ERR_UNSUPPORTED, "gqa: too many query rows for one launch");
  // One CTA per SM walks the items round-robin; DTN_GQA_PERSISTENT=0 launches one CTA per item instead.
  static const bool persistent = [] {
    const char* text = getenv("DTN_GQA_PERSISTENT");
    return !(text && text[0] == '0');
  }();
  static const int early_pv = [] {
    const char* text = getenv("DTN_GQA_EARLY_PV");   // 0: issue a tile's value products only when all its probabilities are ready
    return (text && text[0] == '0') ? 0 : 1;
  }();
  const int64_t ctas = persistent && items > sm_count() ? sm_count() : items;
  const float scale_log2e = scale * 1.4426950408889634f;
  gqa_tc_kernel<SPLIT><<<(unsigned)ctas, attn_threads(SPLIT), A_SMEM_BYTES, s>>>(mq, mk, mv, out, (int)Hq, (int)Hkv, (int)S, scale_log2e,
                                                                                 (int)gb, (int)items, early_pv, status);
  DTN_LAUNCH_CHECK("gqa_tc_kernel");
  return DTN_OK;
}

int gqa_tc_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                  int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s) {
  return split == 2 ? gqa_tc_launch_t<2>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s)
                    : gqa_tc_launch_t<1>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);
}

}  // namespace dtn
