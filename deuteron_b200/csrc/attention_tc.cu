// Grouped-query attention forward on the sm_100a tensor cores (f16 storage, head_dim 128).
//
// One CTA owns 256 query rows of one query head (two 128-row tiles) and walks the keys 128 at a
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
// Warps 0-3 and 4-7: softmax + output for tile 0 and tile 1; warp 8: TMA loads (Q once, then a
// two-slot ring of K and V tiles); warp 9: MMA issue. While one tile's softmax runs, the tensor
// core works on the other tile.
//
// Tensor-memory columns: [0,128) scores/probabilities of tile 0, [128,256) of tile 1,
// [256,384) output of tile 0, [384,512) output of tile 1.
#include <cuda.h>
#include <math.h>

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
constexpr int A_SMEM_BYTES = A_SMEM_TILES * A_TILE_BYTES + 256 + A_XCHG_BYTES + 1024;
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

template <int SPLIT /*warpgroups per 128-row tile: 1 or 2*/>
__global__ void __launch_bounds__(attn_threads(SPLIT), 1)
gqa_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, float* __restrict__ out, int Hq, int Hkv, int S,
              float scale_log2e, int group_begin, int* __restrict__ status) {
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
  const uint32_t q_full = bar_addr;
  auto k_full = [&](int s) { return bar_addr + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar_addr + 8u * (3 + s); };
  auto k_empty = [&](int s) { return bar_addr + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar_addr + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar_addr + 8u * (9 + t); };
  auto p_full = [&](int t) { return bar_addr + 8u * (11 + t); };
  auto o_done = [&](int t) { return bar_addr + 8u * (13 + t); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * 15 + 8);
  volatile float2* xchg = reinterpret_cast<volatile float2*>(bar_ptr + 256);
  constexpr int kTmaWarp = 8 * SPLIT, kMmaWarp = 8 * SPLIT + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_per_group = Hq / Hkv;
  const int group = group_begin + (int)blockIdx.y / heads_per_group;
  const int b = group / Hkv, hkv = group % Hkv;
  const int hq = hkv * heads_per_group + (int)blockIdx.y % heads_per_group;
  const int q_row0 = (b * Hq + hq) * S + (int)blockIdx.x * (2 * A_BM);   // row in the [B*Hq*S, D] view
  const int kv_row0 = (b * Hkv + hkv) * S;
  const int num_kv = S / A_BN;

  for (int i = threadIdx.x; i < 2 * 2 * 128; i += blockDim.x) {   // sequence 0 = empty
    xchg[i].x = 0.f;
    xchg[i].y = 0.f;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < A_KV_STAGES; ++s) {
      ptx::mbar_init(k_full(s), 1);
      ptx::mbar_init(v_full(s), 1);
      ptx::mbar_init(k_empty(s), 1);
      ptx::mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(s_full(t), 1);
      ptx::mbar_init(p_full(t), 4 * SPLIT);   // one arrival per softmax warp
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
      ptx::mbar_expect_tx(q_full, 2 * A_TILE_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_2d(q_addr + t * A_TILE_BYTES + h * A_HALF_BYTES, &tm_q, h * 64, q_row0 + t * A_BM, q_full);
      for (int j = 0; j < num_kv; ++j) {
        const int s = j % A_KV_STAGES;
        const uint32_t ph = (uint32_t)(j / A_KV_STAGES) & 1u;
        if (!ptx::mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1100); break; }
        ptx::mbar_expect_tx(k_full(s), A_TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_2d(k_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_k, h * 64, kv_row0 + j * A_BN, k_full(s));
        if (!ptx::mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1200); break; }
        ptx::mbar_expect_tx(v_full(s), A_TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_2d(v_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_v, h * 64, kv_row0 + j * A_BN, v_full(s));
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------ MMA issuer -----------------------------------------
    if (lane == 0) {
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
      // O_t += P_t V : 8 k-steps of 16 keys; per step the high and the residual plane of P
      auto issue_pv = [&](int t, int s, bool first) {
        const uint32_t va = v_addr + s * A_TILE_BYTES;
        const uint32_t o_tmem = tmem_base + (uint32_t)(256 + t * 128);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t p_col = tmem_base + (uint32_t)(t * 128 + 32 * (kk >> 1) + 8 * (kk & 1));
          const uint64_t vd = umma_desc_mn_sw128(va + (uint32_t)kk * 2048u);
          ptx::umma_ts_f16(o_tmem, p_col + 16u, vd, kIdescPV, (first && kk == 0) ? 0u : 1u);  // residual first
          ptx::umma_ts_f16(o_tmem, p_col, vd, kIdescPV, 1u);
        }
      };
      if (!ptx::mbar_wait(q_full, 0, abort_flag)) { atomicExch(status, 0x2100); ok = false; }
      if (ok && !ptx::mbar_wait(k_full(0), 0, abort_flag)) { atomicExch(status, 0x2200); ok = false; }
      if (ok) {
        ptx::tc_fence_after();
        issue_qk(0, 0);
        ptx::umma_commit<1>(s_full(0));
        issue_qk(1, 0);
        ptx::umma_commit<1>(s_full(1));
        ptx::umma_commit<1>(k_empty(0));
      }
      for (int j = 0; j < num_kv && ok; ++j) {
        const int s = j % A_KV_STAGES, sn = (j + 1) % A_KV_STAGES;
        const uint32_t ph = (uint32_t)(j / A_KV_STAGES) & 1u, phn = (uint32_t)((j + 1) / A_KV_STAGES) & 1u;
        const bool more = j + 1 < num_kv;
        if (!ptx::mbar_wait(v_full(s), ph, abort_flag)) { atomicExch(status, 0x2300); break; }
        if (!ptx::mbar_wait(p_full(0), (uint32_t)j & 1u, abort_flag)) { atomicExch(status, 0x2400); break; }
        ptx::tc_fence_after();
        issue_pv(0, s, j == 0);
        if (more) {
          if (!ptx::mbar_wait(k_full(sn), phn, abort_flag)) { atomicExch(status, 0x2500); break; }
          ptx::tc_fence_after();
          issue_qk(0, sn);
          ptx::umma_commit<1>(s_full(0));
        } else {
          ptx::umma_commit<1>(o_done(0));
        }
        if (!ptx::mbar_wait(p_full(1), (uint32_t)j & 1u, abort_flag)) { atomicExch(status, 0x2600); break; }
        ptx::tc_fence_after();
        issue_pv(1, s, j == 0);
        ptx::umma_commit<1>(v_empty(s));
        if (more) {
          issue_qk(1, sn);
          ptx::umma_commit<1>(s_full(1));
          ptx::umma_commit<1>(k_empty(sn));
        } else {
          ptx::umma_commit<1>(o_done(1));
        }
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
    float m_used = -INFINITY;   // log2-domain maximum the current probabilities are scaled by
    float mass = 0.f;
    bool ok = true;
    for (int j = 0; j < num_kv; ++j) {
      const bool ready = ptx::mbar_wait(s_full(t), (uint32_t)j & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) atomicExch(status, 0x3100 | t);
        ok = false;
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
        const bool got = exchange_with_peer(my_slot, peer_slot, mx, j + 1, abort_flag, other);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) atomicExch(status, 0x3300 | t);
          ok = false;
          break;
        }
        mx = fmaxf(mx, other);
      }
      const float mx2 = mx * scale_log2e;
      const bool grow = (j == 0) || (mx2 > m_used + A_RESCALE_THRESHOLD);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx2 : m_used;
        const float alpha = (j == 0) ? 0.f : ex2_approx(m_used - m_new);   // 1 when this row does not grow
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
          const float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), scale_log2e, shift));
          const float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), scale_log2e, shift));
          mass += p0 + p1;
          const __half2 hi = __floats2half2_rn(p0, p1);
          const float2 back = __half22float2(hi);
          const __half2 lo = __floats2half2_rn(p0 - back.x, p1 - back.y);
          w[i] = *reinterpret_cast<const uint32_t*>(&hi);
          w[16 + i] = *reinterpret_cast<const uint32_t*>(&lo);
        }
        ptx::tmem_st_32x32(s_tmem + (uint32_t)(c * 32), w);
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(p_full(t));
    }
    if (ok) {
      bool ready = ptx::mbar_wait(o_done(t), 0, abort_flag);
      if constexpr (SPLIT == 2) {
        float other = 0.f;
        ready = ready && exchange_with_peer(my_slot, peer_slot, mass, num_kv + 1, abort_flag, other);
        mass += other;
      }
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) atomicExch(status, 0x3200 | t);
      } else {
        ptx::tc_fence_after();
        const float inv = 1.0f / mass;
        // Output through a 4 KiB per-warp staging block (in this tile's Q buffer, which no MMA reads any
        // more): each thread owns one row in tensor memory, but a warp-wide store should cover whole rows,
        // so the 32x32 block is written row-per-thread with an XOR swizzle and read back four rows per
        // instruction, 128 contiguous bytes per row.
        float* stage = reinterpret_cast<float*>(base_ptr + t * A_TILE_BYTES) + (warp % (4 * SPLIT)) * (32 * 32);
        const int tile_row0 = (int)blockIdx.x * (2 * A_BM) + t * A_BM + quarter * 32;
        float* obase = out + ((int64_t)(b * Hq + hq) * S + tile_row0) * A_D;
        const int sub_row = lane >> 3, piece = lane & 7;
#pragma unroll 1
        for (int c = c0; c < c0 + kChunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(o_tmem + (uint32_t)(c * 32), r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(stage + lane * 32 + 4 * (i ^ (lane & 7))) =
                make_float4(__uint_as_float(r[4 * i]) * inv, __uint_as_float(r[4 * i + 1]) * inv,
                            __uint_as_float(r[4 * i + 2]) * inv, __uint_as_float(r[4 * i + 3]) * inv);
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int rloc = rr + sub_row;
            const float4 val = *reinterpret_cast<const float4*>(stage + rloc * 32 + 4 * (piece ^ (rloc & 7)));
            *reinterpret_cast<float4*>(obase + (int64_t)rloc * A_D + c * 32 + 4 * piece) = val;
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
  const int64_t heads = (ge - gb) * (Hq / Hkv);
  DTN_REQUIRE(heads <= 65535, DTN_ERR_UNSUPPORTED, "gqa: too many heads for one launch");
  dim3 grid((unsigned)(S / (2 * A_BM)), (unsigned)heads);
  const float scale_log2e = scale * 1.4426950408889634f;
  gqa_tc_kernel<SPLIT><<<grid, attn_threads(SPLIT), A_SMEM_BYTES, s>>>(mq, mk, mv, out, (int)Hq, (int)Hkv, (int)S, scale_log2e, (int)gb,
                                                      status);
  DTN_LAUNCH_CHECK("gqa_tc_kernel");
  return DTN_OK;
}

int gqa_tc_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                  int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s) {
  return split == 2 ? gqa_tc_launch_t<2>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s)
                    : gqa_tc_launch_t<1>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);
}

}  // namespace dtn
