// Pieces shared by the tensor-core attention kernels (one CTA per work item stream, and CTA pairs).
#pragma once
#include <cuda.h>
#include <math.h>

#include "dtn_common.cuh"
#include "sm100_ptx.cuh"

namespace dtn {

#ifdef DTN_ATTN_TRACE
__device__ long long g_attn_trace[32 * 32 * 8];
#define ATRACE(role, g, point)                                                                              \
  do {                                                                                                      \
    if (blockIdx.x == 0 && (g) >= DTN_ATTN_TRACE && (g) < DTN_ATTN_TRACE + 32 && lane == 0) g_attn_trace[(((g)-DTN_ATTN_TRACE) * 32 + (role)) * 8 + (point)] = clock64(); \
  } while (0)
#define ATRACE2(g, point)                                                                                   \
  do {                                                                                                      \
    if (blockIdx.x == 0 && warp == 0 && (g) >= DTN_ATTN_TRACE && (g) < DTN_ATTN_TRACE + 32 && lane == 0) g_attn_trace[(((g)-DTN_ATTN_TRACE) * 32 + 20) * 8 + (point)] = clock64(); \
  } while (0)
#else
#define ATRACE(role, g, point)
#define ATRACE2(g, point)
#endif

// split: softmax warpgroups per 128-row tile (1 or 2), or 4 = all sixteen softmax warps on one tile at a time
constexpr int attn_softmax_warps(int split) { return split == 4 ? 16 : 8 * split; }
constexpr int attn_threads(int split) { return (attn_softmax_warps(split) + 2) * 32; }   // softmax warps + TMA warp + MMA warp
constexpr int attn_p_half_arrivals(int split) { return split == 4 ? 8 : 4 * split; }     // warps arriving per half tile of probabilities
constexpr int A_BM = 128;          // query rows per tile (two tiles per CTA)
constexpr int A_BN = 128;          // keys per step
constexpr int A_D = 128;           // head dimension
constexpr int A_HALF_BYTES = 128 * 128;           // one [128 rows][64 f16] swizzled block
constexpr int A_TILE_BYTES = 2 * A_HALF_BYTES;    // one [128][128] f16 tile
constexpr int A_KV_STAGES = 2;
constexpr int A_SMEM_TILES = 2 /*Q*/ + 2 * A_KV_STAGES /*K,V*/;
constexpr int A_XCHG_BYTES = 2 * 4 * 128 * 8;   // [tile][column share (up to 4)][row] (value, sequence) slots
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

// ---- products issued a block at a time ------------------------------------------------------------------------
// All 32 lanes of the issuing warp reach these blocks; `elect.sync` picks the lane that issues. One election covers
// the block's eight products, and the descriptors of the k-steps are formed inside it from a 32-bit low word plus an
// immediate (the high word is the same for every operand here), so the issuing warp spends about three instructions
// per product: it shares its scheduler with four softmax warps, and every instruction it needs is one they wait for.
constexpr uint32_t A_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride offset 1024 B, version 1, 128-byte swizzle
__device__ __forceinline__ uint32_t desc_lo_k_major(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_mn_major(uint32_t smem_addr) {
  return ((smem_addr >> 4) & 0x3FFFu) | ((uint32_t)(A_HALF_BYTES >> 4) << 16);
}

// S = Q K^T of one tile: 8 k-steps of 16 along the head dimension. A k-step moves both start addresses by 32 bytes
// inside a swizzled row (+2 in the address field); the second 64-element half lies A_HALF_BYTES further (+1024).
__device__ __forceinline__ void issue_score_products(uint32_t s_tmem, uint32_t q_lo, uint32_t k_lo, uint32_t idesc) {
#define DTN_QK_STEP(OFF)                                                                          \
  "add.u32 qa, %1, " #OFF ";\n\tadd.u32 ka, %2, " #OFF ";\n\tmov.b64 da, {qa, %3};\n\tmov.b64 db, {ka, %3};\n\t" \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, acc;\n\t"
  asm volatile(
      "{\n\t.reg .pred q, acc;\n\t.reg .b32 qa, ka;\n\t.reg .b64 da, db;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 acc, 0, 0;\n\t"
      DTN_QK_STEP(0)
      "setp.eq.b32 acc, 0, 0;\n\t"
      DTN_QK_STEP(2) DTN_QK_STEP(4) DTN_QK_STEP(6) DTN_QK_STEP(1024) DTN_QK_STEP(1026) DTN_QK_STEP(1028) DTN_QK_STEP(1030)
      "}" ::"r"(s_tmem), "r"(q_lo), "r"(k_lo), "r"(A_DESC_HI), "r"(idesc)
      : "memory");
#undef DTN_QK_STEP
}

// O += P V for four k-steps of 16 keys: per step the residual plane of P (16 columns after the high plane), then the
// high plane, both against the same 16 key rows of V (+128 in the address field per step). COL / KEY: tensor-memory
// column of the step's high plane relative to p_tmem, and the step's address-field offset relative to v_lo.
template <int COL1, int KEY1, int COL2, int KEY2, int COL3, int KEY3>
__device__ __forceinline__ void issue_value_products(uint32_t o_tmem, uint32_t p_tmem, uint32_t v_lo, uint32_t idesc,
                                                     uint32_t accumulate_first) {
#define DTN_PV_STEP(COL, KEY, FIRST)                                                                                     \
  "add.u32 ph, %1, " COL ";\n\tadd.u32 pl, ph, 16;\n\tadd.u32 vb, %2, " KEY ";\n\tmov.b64 db, {vb, %3};\n\t"    \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [pl], db, %4, " FIRST ";\n\t"                                            \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ph], db, %4, yes;\n\t"
  asm volatile(
      "{\n\t.reg .pred q, acc, yes;\n\t.reg .b32 ph, pl, vb;\n\t.reg .b64 db;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 acc, %5, 0;\n\tsetp.eq.b32 yes, 0, 0;\n\t"
      DTN_PV_STEP("0", "0", "acc") DTN_PV_STEP("%6", "%7", "yes") DTN_PV_STEP("%8", "%9", "yes") DTN_PV_STEP("%10", "%11", "yes")
      "}" ::"r"(o_tmem), "r"(p_tmem), "r"(v_lo), "r"(A_DESC_HI), "r"(idesc), "r"(accumulate_first), "n"(COL1), "n"(KEY1), "n"(COL2),
      "n"(KEY2), "n"(COL3), "n"(KEY3)
      : "memory");
#undef DTN_PV_STEP
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

// Packed FP32 arithmetic (two lanes per instruction, sm_100): halves the issue slots of the scale-and-shift, the row
// sum and the residual of the probability pass.
__device__ __forceinline__ float2 fma_f32x2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// p - hi for a pair of FP32 values and their packed f16 roundings, exact: the mixed-precision fma of sm_100 takes
// the f16 halves as they are (no conversion of hi back to FP32).
__device__ __forceinline__ float2 residual_after_f16(uint32_t hi_pair, float2 p) {
  float2 r;
  asm("{\n\t.reg .f16 h0, h1, m;\n\tmov.b32 {h0, h1}, %2;\n\tmov.b16 m, 0xBC00;\n\t"   // m = -1.0
      "fma.rn.f32.f16 %0, h0, m, %3;\n\tfma.rn.f32.f16 %1, h1, m, %4;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "r"(hi_pair), "f"(p.x), "f"(p.y));
  return r;
}

// Eight consecutive floats (one 32-byte sector) of one row, scaled, in one store.
__device__ __forceinline__ void store_scaled_sector(float* dst, const uint32_t* r, float scale) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "f"(__uint_as_float(r[0]) * scale),
               "f"(__uint_as_float(r[1]) * scale), "f"(__uint_as_float(r[2]) * scale), "f"(__uint_as_float(r[3]) * scale),
               "f"(__uint_as_float(r[4]) * scale), "f"(__uint_as_float(r[5]) * scale), "f"(__uint_as_float(r[6]) * scale),
               "f"(__uint_as_float(r[7]) * scale)
               : "memory");
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
    // a short burst of polls between looks at the abort flag and the clock: the partner is normally a few hundred
    // cycles away, and every instruction of this loop competes with the softmax arithmetic for issue slots
#pragma unroll 1
    for (int poll = 0; poll < 32; ++poll) {
      float a, b;
      asm volatile("ld.volatile.shared.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "r"(addr) : "memory");
      if (__float_as_int(b) == seq) {
        other = a;
        return true;
      }
    }
    if (*abort_flag) return false;
    if (clock64() - start > ptx::kWaitBudgetCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// The same hand-over through an mbarrier that the two partner warps of a row quarter share (two arrivals per phase,
// one elected lane per warp): the waiting warp sleeps in mbarrier.try_wait instead of polling shared memory, so it
// takes no issue slots from the warps that are still computing. `slot` alternates between two floats per thread: a
// value is overwritten only two exchanges later, after the partner's arrival for the exchange in between, which it
// makes after reading this one.
__device__ __forceinline__ bool exchange_through_barrier(volatile float2* mine, volatile float2* theirs, uint32_t bar, int count,
                                                         float value, int lane, volatile int* abort_flag, float& other) {
  volatile float* out_slot = reinterpret_cast<volatile float*>(mine) + (count & 1);
  volatile float* in_slot = reinterpret_cast<volatile float*>(theirs) + (count & 1);
  *out_slot = value;
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(bar);
  if (!ptx::mbar_wait(bar, (uint32_t)count & 1u, abort_flag)) return false;
  other = *in_slot;
  return true;
}

// Work items: one item = 256 query rows of one query head. A CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...
// and runs them as ONE stream of key steps: barrier phases, the K/V ring and the exchange sequence numbers keep
// counting across items, so the next item's first products are issued while the previous item's output is still being
// written (the per-item prologue, pipeline fill and output no longer leave the tensor core idle). With as many CTAs
// as items the kernel degenerates to one item per CTA.
struct AttnItem {
  int q_row0;     // first query row in the [B*Hq*S, D] view
  int kv_row0;    // first key row in the [B*Hkv*S, D] view
  int q_head, q_row;   // the same as (query head of the batch, row inside it)
  int kv_head;         // key/value head of the batch
};
__device__ __forceinline__ AttnItem attn_item(int item, int qblocks, int Hq, int Hkv, int S, int group_begin,
                                             int item_rows = 2 * A_BM) {
  const int heads_per_group = Hq / Hkv;
  const int head_local = item / qblocks, qb = item % qblocks;
  const int group = group_begin + head_local / heads_per_group;
  const int b = group / Hkv, hkv = group % Hkv;
  const int hq = hkv * heads_per_group + head_local % heads_per_group;
  AttnItem it;
  it.q_row0 = (b * Hq + hq) * S + qb * item_rows;
  it.kv_row0 = (b * Hkv + hkv) * S;
  it.q_head = b * Hq + hq;
  it.q_row = qb * item_rows;
  it.kv_head = b * Hkv + hkv;
  return it;
}

// The softmax + output role of one warp, shared by the one-CTA and the CTA-pair kernels.
// SPLIT warpgroups share one 128-row tile: each owns 128 / SPLIT score columns (and the same share of the output
// columns) of all 128 rows. Partner threads of a row agree on the row maximum through a shared-memory slot (bounded
// spin, no block-wide barrier). Barriers are shared-memory addresses of this CTA, except p_half0 / p_half1 when
// `remote_arrive` is set: then they are cluster addresses of the barriers in the CTA that issues the MMAs.
struct SoftmaxRole {
  uint32_t tmem_base;
  uint32_t s_full, p_half0, p_half1, o_done;
  bool remote_arrive;
  volatile float2* xchg;     // [2 tiles][2 shares][128 rows]
  uint32_t xbar;             // barrier the two partner warps of this warp's (tile, row quarter) exchange through (KEEP form)
  const CUtensorMap* out_map;   // KEEP form: the output as [heads][S][128] FP32, boxes of 32 columns x 32 rows, 128-byte swizzle
  uint32_t out_stage;           // KEEP form: this warp's 4 KiB staging block for its output, in ring slot 0 of the keys (tile 0) or
                                // of the values (tile 1); the block of the slot the item's last step used is A_TILE_BYTES further
  uint32_t staged_bar;          // KEEP form: arrives once the staging block has been read (the slot may be loaded again)
  int valid_last;               // KEEP form: keys of the item's last step that exist (128 unless S is not a multiple of 128)
  float* stage_base;         // 1 KiB per softmax warp
  volatile int* abort_flag;
  int* status;
  float* out;
  float scale_log2e;
  int total_steps, num_kv;
  int first_item, item_stride, qblocks, Hq, Hkv, S, group_begin, item_rows;
  int rows_before_tile;      // first row of this warp's tile inside the work item
  int rows_between_tiles;    // alternating form: row distance from tile 0 to tile 1 inside the work item
};

template <int SPLIT, bool KEEP = false>
__device__ __forceinline__ void softmax_role(const SoftmaxRole& R, int warp, int lane) {
  const uint32_t tmem_base = R.tmem_base;
  volatile int* abort_flag = R.abort_flag;
  int* status = R.status;
  const int total_steps = R.total_steps, num_kv = R.num_kv;
  const float scale_log2e = R.scale_log2e;
  volatile float2* xchg = R.xchg;
  float* out = R.out;
  // SPLIT warpgroups share one tile: each owns 128 / SPLIT score columns (and the same share of
  // the output columns) of all 128 rows. Partner threads of a row agree on the row maximum
  // through a shared-memory slot (bounded spin, no block-wide barrier).
  constexpr int kChunks = 4 / SPLIT;             // 32-column chunks per thread
  // KEEP: the thread's first 32 scores stay in registers between the two passes, the other 32 are fetched a second
  // time while the first are worked on, and the partner threads exchange through a barrier instead of polling. (All
  // 64 scores cannot stay: with 18 warps per CTA one scheduler holds five warps, which caps a thread at 96 registers,
  // and the kept scores spilled: 651 instead of 827 TFLOP/s.)
  constexpr bool kKeep = SPLIT == 2 && KEEP;
  int exchanges = 0;   // kKeep: exchanges through the barrier so far
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
  float m_used = -INFINITY;   // log2-domain maximum the current probabilities are scaled by
  float mass = 0.f;
  // No division inside the loop: with four or five busy warps per scheduler a dependent instruction issues every ten
  // cycles or so, and one integer division is a chain of thirty. j and it count along; the item's output address is
  // worked out during its first step, after the probabilities are handed over, when this warp would wait anyway.
  int j = -1, it = 0;
  float* row_out = nullptr;
  int out_head = 0, out_first_row = 0;
  bool release_pending = false;
  for (int g = 0; g < total_steps; ++g) {
    if (++j == num_kv) {
      j = 0;
      ++it;
    }
    if (j == 0) {   // a new item starts
      m_used = -INFINITY;
      mass = 0.f;
    }
    const bool ready = ptx::mbar_wait(R.s_full, (uint32_t)g & 1u, abort_flag);
    if (!__all_sync(0xffffffffu, ready)) {
      if (lane == 0) atomicExch(status, 0x3100 | t);
      break;
    }
    ptx::tc_fence_after();
    ATRACE(warp, g, 0);
    // pass 1: row maximum of the raw scores (three-input max: two scores per instruction). With two warpgroups per
    // tile a thread owns 64 scores: both loads are issued together and the scores stay in registers for pass 2.
    float mx = -INFINITY;
    bool masked = false;
    uint32_t kept[kKeep ? 64 : 1];
    if constexpr (kKeep) {
      uint32_t (&lo_half)[32] = *reinterpret_cast<uint32_t (*)[32]>(kept);
      uint32_t (&hi_half)[32] = *reinterpret_cast<uint32_t (*)[32]>(kept + 32);
      ptx::tmem_ld_32x32(s_tmem + (uint32_t)(c0 * 32), lo_half);
      ptx::tmem_ld_32x32(s_tmem + (uint32_t)((c0 + 1) * 32), hi_half);
      ptx::tmem_ld_wait();
      // keys past the end of the sequence (the item's last step when S is not a multiple of 128; their K rows were
      // loaded as zeros): their scores become -inf, so they take no part in the maximum and their probabilities are 0
      masked = j == num_kv - 1 && R.valid_last < A_BN;
      if (masked) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (c0 * 32 + i >= R.valid_last) kept[i] = 0xff800000u;
      }
#pragma unroll
      for (int i = 0; i < 64; i += 2) mx = max3(mx, __uint_as_float(kept[i]), __uint_as_float(kept[i + 1]));
    } else {
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(s_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      }
    }
    ATRACE(warp, g, 1);
    if constexpr (SPLIT == 2) {
      float other;
      bool got;
      if constexpr (kKeep) got = exchange_through_barrier(my_slot, peer_slot, R.xbar, exchanges++, mx, lane, abort_flag, other);
      else got = exchange_with_peer(my_slot, peer_slot, mx, 2 * g + 1, abort_flag, other);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) atomicExch(status, 0x3300 | t);
        break;
      }
      mx = fmaxf(mx, other);
    }
    ATRACE(warp, g, 2);
    const float mx2 = mx * scale_log2e;
    const bool grow = (j == 0) || (mx2 > m_used + A_RESCALE_THRESHOLD);
    if (__any_sync(0xffffffffu, grow)) {
      const float m_new = grow ? mx2 : m_used;
      const float alpha = (j == 0) ? 0.f : ex2_approx_ftz(m_used - m_new);   // 1 when this row does not grow
      if (j > 0) {
        ATRACE(warp, g, 6);
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
    ATRACE(warp, g, 3);
    if constexpr (kKeep) {
      // The first 32 scores are still in registers; the other 32 are fetched again while the first are worked on, so
      // no load of this pass is waited for. A piece of 16 scores becomes 8 words of high parts and 8 words of
      // residuals, stored with two 8-column instructions: only 16 result registers are live beside the scores.
      uint32_t (&first)[32] = *reinterpret_cast<uint32_t (*)[32]>(kept);
      uint32_t (&second)[32] = *reinterpret_cast<uint32_t (*)[32]>(kept + 32);
      ptx::tmem_ld_32x16(s_tmem + (uint32_t)((c0 + 1) * 32), second);
      const float2 scale2 = make_float2(scale_log2e, scale_log2e), shift2 = make_float2(shift, shift);
      float2 sums = make_float2(0.f, 0.f);
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        if (piece == 1) ptx::tmem_ld_32x16(s_tmem + (uint32_t)((c0 + 1) * 32 + 16), second + 16);
        if (piece == 2) {
          ptx::tmem_ld_wait();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if ((c0 + 1) * 32 + i >= R.valid_last) second[i] = 0xff800000u;
          }
          mass += sums.x + sums.y;   // per 32 scores, like the form that reads the scores twice: the same bits
          sums = make_float2(0.f, 0.f);
        }
        const uint32_t* src = (piece < 2 ? first : second) + 16 * (piece & 1);
        uint32_t high[8], low[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 x = fma_f32x2(make_float2(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1])), scale2, shift2);
          const float2 p = make_float2(ex2_approx_ftz(x.x), ex2_approx_ftz(x.y));
          sums = add_f32x2(sums, p);
          const __half2 hi = __floats2half2_rn(p.x, p.y);
          high[i] = *reinterpret_cast<const uint32_t*>(&hi);
          const float2 residual = residual_after_f16(high[i], p);
          const __half2 lo = __floats2half2_rn(residual.x, residual.y);
          low[i] = *reinterpret_cast<const uint32_t*>(&lo);
        }
        const uint32_t col = s_tmem + (uint32_t)((c0 + (piece >> 1)) * 32 + (piece & 1) * 8);
        ptx::tmem_st_32x8(col, high);
        ptx::tmem_st_32x8(col + 16u, low);
        if (piece & 1) {   // this warp's share of one half is in tensor memory
          ptx::tmem_st_wait();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            const uint32_t bar = (piece >> 1) ? R.p_half1 : R.p_half0;
            if (R.remote_arrive) ptx::mbar_arrive_cluster(bar);
            else ptx::mbar_arrive(bar);
          }
          ATRACE(warp, g, 4 + (piece >> 1));
        }
      }
      mass += sums.x + sums.y;
    } else
#pragma unroll(SPLIT == 1 ? 4 : 1)   // one warpgroup per tile has registers to spare for overlapping the chunks
    for (int c = c0; c < c0 + kChunks; ++c) {
      uint32_t r[kKeep ? 1 : 32], w[32];
      if constexpr (!kKeep) {
        ptx::tmem_ld_32x32(s_tmem + (uint32_t)(c * 32), *reinterpret_cast<uint32_t (*)[32]>(r));
        ptx::tmem_ld_wait();
      }
      const uint32_t* src = kKeep ? kept + 32 * (c - c0) : r;
      const float2 scale2 = make_float2(scale_log2e, scale_log2e), shift2 = make_float2(shift, shift);
      float2 sums = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 x = fma_f32x2(make_float2(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1])), scale2, shift2);
        const float2 p = make_float2(ex2_approx_ftz(x.x), ex2_approx_ftz(x.y));
        sums = add_f32x2(sums, p);
        const __half2 hi = __floats2half2_rn(p.x, p.y);
        w[i] = *reinterpret_cast<const uint32_t*>(&hi);
        const float2 residual = residual_after_f16(w[i], p);
        const __half2 lo = __floats2half2_rn(residual.x, residual.y);
        w[16 + i] = *reinterpret_cast<const uint32_t*>(&lo);
      }
      mass += sums.x + sums.y;
      ptx::tmem_st_32x32(s_tmem + (uint32_t)(c * 32), w);
      if (((c - c0 + 1) % (kChunks / 2)) == 0) {   // this warp's share of one half is in tensor memory
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          const uint32_t bar = ((c - c0) / (kChunks / 2)) ? R.p_half1 : R.p_half0;
          if (R.remote_arrive) ptx::mbar_arrive_cluster(bar);
          else ptx::mbar_arrive(bar);
        }
        ATRACE(warp, g, 4 + ((c - c0) / (kChunks / 2)));
      }
    }
    if constexpr (kKeep) {
      if (release_pending) {   // the previous item's last store has long read its staging block: the slot may be loaded again
        if (lane == 0) {
          ptx::bulk_wait_read_all();
          ptx::mbar_arrive(R.staged_bar);
        }
        __syncwarp();
        release_pending = false;
      }
    }
    if (j == 0) {
      const AttnItem item = attn_item(R.first_item + it * R.item_stride, R.qblocks, R.Hq, R.Hkv, R.S, R.group_begin, R.item_rows);
      row_out = out + ((int64_t)item.q_row0 + R.rows_before_tile + row_in_tile) * A_D;
      out_head = item.q_head;
      out_first_row = item.q_row + R.rows_before_tile + quarter * 32;   // first of this warp's rows inside the head
    }
    if (j != num_kv - 1) continue;

    // ---- the item's last step: normalise and store its output while the tensor core already works on the other
    // tile and on the next item's scores (the next item's first product into O_t waits for this warp's next arrival
    // on p_half, which comes after the reads below) ----
    bool done = ptx::mbar_wait(R.o_done, (uint32_t)it & 1u, abort_flag);
    if constexpr (SPLIT == 2) {
      float other = 0.f;
      if constexpr (kKeep) done = done && exchange_through_barrier(my_slot, peer_slot, R.xbar, exchanges++, mass, lane, abort_flag, other);
      else done = done && exchange_with_peer(my_slot, peer_slot, mass, 2 * g + 2, abort_flag, other);
      mass += other;
    }
    if (!__all_sync(0xffffffffu, done)) {
      if (lane == 0) atomicExch(status, 0x3200 | t);
      break;
    }
    ptx::tc_fence_after();
    ATRACE(warp, g, 6);
    const float inv = 1.0f / mass;
    if constexpr (kKeep) {
      // The ring slot the item's last step used is free by now -- the keys once the step's score products are done,
      // which o_done(0) implies, the values once both tiles' value products are done, which o_done(1) implies -- and
      // nothing wants it before the second step of the next item. So the warp's 32 rows x 32 columns of output go
      // there (tile 0: keys' slot, tile 1: values' slot; the layout of a 128-byte-swizzled box: 16-byte piece p of
      // row r at position p ^ (r & 7)) and from there to memory as one TMA store: whole lines, nothing for the
      // load/store unit to do, about forty instructions per block. The producer loads the slot again once every warp
      // of the tile has reported that its staging block has been read.
      const uint32_t out_stage = R.out_stage + (uint32_t)(g & 1) * A_TILE_BYTES;
      ATRACE2(g, 0);
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(o_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
        ATRACE2(g, 1 + 3 * (c - c0));
        if (c > c0) {
          if (lane == 0) ptx::bulk_wait_read_all();
          __syncwarp();
        }
        ATRACE2(g, 2 + 3 * (c - c0));
        const uint32_t row_addr = out_stage + (uint32_t)lane * 128u;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)((piece ^ (lane & 7)) * 16)),
                       "f"(__uint_as_float(r[4 * piece]) * inv), "f"(__uint_as_float(r[4 * piece + 1]) * inv),
                       "f"(__uint_as_float(r[4 * piece + 2]) * inv), "f"(__uint_as_float(r[4 * piece + 3]) * inv)
                       : "memory");
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_3d(R.out_map, out_stage, c * 32, out_first_row, out_head);   // rows past the sequence's end are dropped
          ptx::bulk_commit_group();
        }
        ATRACE2(g, 3 + 3 * (c - c0));
      }
      // The staging block is handed back during the next item's first step (see there): its store needs about a
      // thousand cycles to read the block, and the next item's scores are already waiting.
      release_pending = true;
      ATRACE2(g, 7);
    } else {
      // A thread owns one row in tensor memory and writes its share of it as whole 32-byte sectors.
#pragma unroll 1
      for (int c = c0; c < c0 + kChunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(o_tmem + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int sector = 0; sector < 4; ++sector) store_scaled_sector(row_out + c * 32 + sector * 8, r + 8 * sector, inv);
      }
    }
    ATRACE(warp, g, 7);
  }
  if constexpr (kKeep) {
    if (lane == 0) ptx::bulk_wait_all();   // the last item's stores are complete before the CTA may end
  }
}

// Hands `value` to the three threads that own the other column quarters of the same row and folds theirs into it
// (maximum or sum). slots: this tile's [4 quarters][128 rows] block; `mine` is this thread's quarter.
template <bool MAX>
__device__ __forceinline__ bool exchange_four(volatile float2* slots, int mine, int row, float& value, int seq,
                                              volatile int* abort_flag) {
  asm volatile("st.volatile.shared.v2.f32 [%0], {%1, %2};" ::"r"(smem_u32((const void*)(slots + mine * 128 + row))), "f"(value),
               "f"(__int_as_float(seq))
               : "memory");
  float folded = value;
  const long long start = clock64();
#pragma unroll
  for (int other = 1; other < 4; ++other) {
    const uint32_t addr = smem_u32((const void*)(slots + ((mine + other) & 3) * 128 + row));
    while (true) {
      float a, b;
      asm volatile("ld.volatile.shared.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "r"(addr) : "memory");
      if (__float_as_int(b) == seq) {
        folded = MAX ? fmaxf(folded, a) : folded + a;
        break;
      }
      if (*abort_flag) return false;
      if (clock64() - start > ptx::kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  value = folded;
  return true;
}

// Softmax + output with all sixteen warps on one tile at a time. A warp owns 32 rows (its tensor-memory lane quarter)
// and one 32-column quarter of the scores, of BOTH tiles: it serves tile 0's step, then tile 1's, and so on. A tile's
// softmax therefore takes half as long as with eight warps per tile working on both tiles at once -- it has to fit in
// the time the tensor core spends on the other tile's products, or the tensor core waits for it. The thread's 32
// scores are read from tensor memory once and stay in registers between the maximum and the probabilities.
// R.s_full, R.p_half0/1 and R.o_done are tile 0's barriers; tile 1's follow at the distances given below.
struct SoftmaxBarrierStrides {
  uint32_t s_full, p_half, o_done;   // byte distance from a tile-0 barrier to the same barrier of tile 1
};

__device__ __forceinline__ void softmax_role_alternating(const SoftmaxRole& R, const SoftmaxBarrierStrides& strides, int warp, int lane) {
  const uint32_t tmem_base = R.tmem_base;
  volatile int* abort_flag = R.abort_flag;
  int* status = R.status;
  const int total_steps = R.total_steps, num_kv = R.num_kv;
  const float scale_log2e = R.scale_log2e;
  const int quarter = warp & 3;          // tensor-memory lanes [32 * quarter, +32)
  const int cq = (warp >> 2) & 3;        // column quarter: score / output columns [32 * cq, +32)
  const int row_in_tile = quarter * 32 + lane;
  const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
  float* stage = R.stage_base + warp * 256;
  float m_used[2] = {-INFINITY, -INFINITY};
  float mass[2] = {0.f, 0.f};
  bool ok = true;
  for (int g = 0; g < total_steps && ok; ++g) {
    const int j = g % num_kv;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (j == 0) {
        m_used[t] = -INFINITY;
        mass[t] = 0.f;
      }
      const uint32_t s_tmem = tmem_base + lane_field + (uint32_t)(t * 128 + cq * 32);
      const uint32_t o_tmem = tmem_base + lane_field + (uint32_t)(256 + t * 128 + cq * 32);
      volatile float2* slots = R.xchg + t * 4 * 128;
      const bool ready = ptx::mbar_wait(R.s_full + t * strides.s_full, (uint32_t)g & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) atomicExch(status, 0x3100 | t);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      uint32_t r[32], w[32];
      ptx::tmem_ld_32x32(s_tmem, r);
      ptx::tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      const bool got = exchange_four<true>(slots, cq, row_in_tile, mx, 2 * g + 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) atomicExch(status, 0x3300 | t);
        ok = false;
        break;
      }
      const float mx2 = mx * scale_log2e;
      const bool grow = (j == 0) || (mx2 > m_used[t] + A_RESCALE_THRESHOLD);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx2 : m_used[t];
        const float alpha = (j == 0) ? 0.f : ex2_approx_ftz(m_used[t] - m_new);   // 1 when this row does not grow
        if (j > 0) {
          // All earlier products into O_t are complete: s_full(t) of this step was committed after them.
          uint32_t o[32];
          ptx::tmem_ld_32x32(o_tmem, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          ptx::tmem_st_32x32(o_tmem, o);
          ptx::tmem_st_wait();
        }
        mass[t] *= alpha;
        m_used[t] = m_new;
      }
      const float shift = A_BIAS - m_used[t];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = ex2_approx_ftz(fmaf(__uint_as_float(r[2 * i]), scale_log2e, shift));
        const float p1 = ex2_approx_ftz(fmaf(__uint_as_float(r[2 * i + 1]), scale_log2e, shift));
        sum += p0 + p1;
        const __half2 hi = __floats2half2_rn(p0, p1);
        const float2 back = __half22float2(hi);
        const __half2 lo = __floats2half2_rn(p0 - back.x, p1 - back.y);
        w[i] = *reinterpret_cast<const uint32_t*>(&hi);
        w[16 + i] = *reinterpret_cast<const uint32_t*>(&lo);
      }
      mass[t] += sum;
      ptx::tmem_st_32x32(s_tmem, w);
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = ((cq >> 1) ? R.p_half1 : R.p_half0) + t * strides.p_half;   // quarters 0, 1 -> first half of the keys
        if (R.remote_arrive) ptx::mbar_arrive_cluster(bar);
        else ptx::mbar_arrive(bar);
      }
    }
    if (!ok || j != num_kv - 1) continue;

    // ---- the item's last step, both tiles: normalise and store this warp's 32 x 32 block of each output ----
    const int it = g / num_kv;
    const AttnItem item = attn_item(R.first_item + it * R.item_stride, R.qblocks, R.Hq, R.Hkv, R.S, R.group_begin, R.item_rows);
    const int wr_swap = (lane >> 2) & 1;
    const int rd_row = lane >> 1, rd_piece = lane & 1;
#pragma unroll 1
    for (int t = 0; t < 2; ++t) {
      const uint32_t o_tmem = tmem_base + lane_field + (uint32_t)(256 + t * 128 + cq * 32);
      bool done = ptx::mbar_wait(R.o_done + t * strides.o_done, (uint32_t)it & 1u, abort_flag);
      float total = mass[t];
      done = done && exchange_four<false>(R.xchg + t * 4 * 128, cq, row_in_tile, total, 2 * g + 2, abort_flag);
      if (!__all_sync(0xffffffffu, done)) {
        if (lane == 0) atomicExch(status, 0x3200 | t);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const float inv = 1.0f / total;
      float* obase = R.out + ((int64_t)item.q_row0 + R.rows_before_tile + t * R.rows_between_tiles + quarter * 32) * A_D;
      uint32_t o[32];
      ptx::tmem_ld_32x32(o_tmem, o);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<float4*>(stage + lane * 8 + 4 * (i ^ wr_swap)) =
              make_float4(__uint_as_float(o[8 * sub + 4 * i]) * inv, __uint_as_float(o[8 * sub + 4 * i + 1]) * inv,
                          __uint_as_float(o[8 * sub + 4 * i + 2]) * inv, __uint_as_float(o[8 * sub + 4 * i + 3]) * inv);
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int rloc = rd_row + 16 * h;
          const float4 val = *reinterpret_cast<const float4*>(stage + rloc * 8 + 4 * (rd_piece ^ ((rloc >> 2) & 1)));
          *reinterpret_cast<float4*>(obase + (int64_t)rloc * A_D + cq * 32 + sub * 8 + 4 * rd_piece) = val;
        }
        __syncwarp();
      }
    }
  }
}

}  // namespace dtn
