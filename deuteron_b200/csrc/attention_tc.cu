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

#include "attention_tc.cuh"

namespace dtn {

template <int SPLIT /*warpgroups per 128-row tile: 1 or 2*/, bool KEEP = false /*scores stay in registers between the passes*/>
__global__ void __launch_bounds__(attn_threads(SPLIT), 1)
gqa_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_out, float* __restrict__ out, int Hq,
              int Hkv, int S,
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
  auto staged = [&](int t) { return bar_addr + 8u * (22 + t); };   // KEEP: the tile's output staging (a K or V ring slot) has been read
  auto x_bar = [&](int t, int quarter) { return bar_addr + 8u * (24 + 4 * t + quarter); };   // partner warps of a row quarter
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * 20 + 8);
  volatile float2* xchg = reinterpret_cast<volatile float2*>(bar_ptr + 256);
  float* stage_base = reinterpret_cast<float*>(bar_ptr + 256 + A_XCHG_BYTES);   // 1 KiB per softmax warp
  constexpr int kTmaWarp = attn_softmax_warps(SPLIT), kMmaWarp = attn_softmax_warps(SPLIT) + 1;
#ifdef DTN_ATTN_TRACE
  const uint32_t dbg_bar = bar_addr + 256 + A_XCHG_BYTES;   // in the staging area, which the traced form does not use
#define DTN_DBG_COMMIT(b) ptx::umma_commit_led(leader, dbg_bar + 8u * (b))
#else
#define DTN_DBG_COMMIT(b)
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // S need not be a multiple of the tile sizes: the tensor maps are [heads][S][128], so rows past a head's end load
  // as zeros and are dropped by the output store; the softmax masks the keys that do not exist (KEEP form only: the
  // other forms store their output with plain stores and take only multiples of 256)
  const int qblocks = (S + 2 * A_BM - 1) / (2 * A_BM);
  const int num_kv = (S + A_BN - 1) / A_BN;
  const int my_items = ((int)blockIdx.x < total_items) ? (total_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total_steps = my_items * num_kv;

  for (int i = threadIdx.x; i < A_XCHG_BYTES / 8; i += blockDim.x) {   // sequence 0 = empty
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
      ptx::mbar_init(p_half(t, 0), attn_p_half_arrivals(SPLIT));   // one arrival per softmax warp that writes this half
      ptx::mbar_init(p_half(t, 1), attn_p_half_arrivals(SPLIT));
      ptx::mbar_init(o_done(t), 1);
#ifdef DTN_ATTN_TRACE
      if (t == 0) for (int b = 0; b < 6; ++b) ptx::mbar_init(dbg_bar + 8u * b, 1);
#endif
      ptx::mbar_init(staged(t), attn_softmax_warps(SPLIT) / 2);
      for (int quarter = 0; quarter < 4; ++quarter) ptx::mbar_init(x_bar(t, quarter), 2);
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
          // KEEP: the previous item's output was staged in the slots its last step used, which are this item's second
          // step's: tile 0's in the keys' slot, tile 1's in the values' slot
          if (KEEP && it > 0 && j == 1 && !ptx::mbar_wait(staged(0), (uint32_t)(it - 1) & 1u, abort_flag)) { atomicExch(status, 0x1400); ok = false; break; }
          ptx::mbar_expect_tx(k_full(s), A_TILE_BYTES);
          for (int h = 0; h < 2; ++h)
            ptx::tma_load_3d(k_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_k, h * 64, j * A_BN, item.kv_head, k_full(s));
          if (j == 0) {
            // this item's queries, right after its first keys: a buffer is free once the previous item's last score
            // product has read it, which is about one step before the first product of this item wants it. The tiles
            // were asked into L2 one item earlier, so the load does not wait for HBM.
            for (int t = 0; t < 2 && ok; ++t) {
              if (it > 0 && !ptx::mbar_wait(q_empty(t), (uint32_t)(it - 1) & 1u, abort_flag)) { atomicExch(status, 0x1300); ok = false; break; }
              ptx::mbar_expect_tx(q_full(t), A_TILE_BYTES);
              for (int h = 0; h < 2; ++h)
                ptx::tma_load_3d(q_addr + t * A_TILE_BYTES + h * A_HALF_BYTES, &tm_q, h * 64, item.q_row + t * A_BM, item.q_head, q_full(t));
            }
            if (!ok) break;
            if (it + 1 < my_items) {
              const AttnItem next = attn_item((int)blockIdx.x + (it + 1) * (int)gridDim.x, qblocks, Hq, Hkv, S, group_begin);
              for (int t = 0; t < 2; ++t)
                for (int h = 0; h < 2; ++h) ptx::tma_prefetch_3d(&tm_q, h * 64, next.q_row + t * A_BM, next.q_head);
            }
          }
          if (!ptx::mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1200); ok = false; break; }
          if (KEEP && it > 0 && j == 1 && !ptx::mbar_wait(staged(1), (uint32_t)(it - 1) & 1u, abort_flag)) { atomicExch(status, 0x1500); ok = false; break; }
          ptx::mbar_expect_tx(v_full(s), A_TILE_BYTES);
          for (int h = 0; h < 2; ++h)
            ptx::tma_load_3d(v_addr + s * A_TILE_BYTES + h * A_HALF_BYTES, &tm_v, h * 64, j * A_BN, item.kv_head, v_full(s));
        }
      }
    }
#ifdef DTN_ATTN_TRACE
    else if (lane == 1 && blockIdx.x == 0) {
      bool fine = true;
      for (int g = 0; g < total_steps && fine; ++g)
        for (int b = 0; b < 6; ++b) {
          if (!ptx::mbar_wait(dbg_bar + 8u * b, (uint32_t)g & 1u, abort_flag)) { fine = false; break; }
          if (g >= DTN_ATTN_TRACE && g < DTN_ATTN_TRACE + 32) g_attn_trace[((g - DTN_ATTN_TRACE) * 32 + 21) * 8 + b] = clock64();
        }
    }
#endif
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------ MMA issuer -----------------------------------------
    // All 32 lanes walk the loop and wait on the barriers; lane 0 alone issues. Control flow and operands are
    // uniform across the warp, so descriptors and addresses can live in uniform registers.
    if (total_steps > 0) {
      constexpr uint32_t kIdescQK = attn_idesc(0);
      constexpr uint32_t kIdescPV = attn_idesc(1);
      const uint32_t leader = lane == 0 ? 1u : 0u;
      const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
      bool ok = true;
      auto failed = [&](int code) {
        if (lane == 0) atomicExch(status, code);
        return false;
      };
      auto wait_all = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)); };
      static_assert(A_KV_STAGES == 2, "the issue loops select between two K/V slots");
      auto issue_qk = [&](int t, int s) {
        issue_score_products(tmem + (uint32_t)(t * 128), desc_lo_k_major(q_addr + t * A_TILE_BYTES), desc_lo_k_major(k_addr + s * A_TILE_BYTES),
                             kIdescQK);
      };
      // The probabilities arrive in two halves, so the value products of the first half can run while the second is
      // still being computed. SPLIT == 2: warpgroup 0 writes the 32-key chunks 0, 1 and warpgroup 1 chunks 2, 3, each
      // in order -> halves {0, 2} and {1, 3}; otherwise chunks are finished in order -> halves {0, 1} and {2, 3}.
      auto issue_pv = [&](int t, int s, bool first, int half) {
        const uint32_t o_tmem = tmem + (uint32_t)(256 + t * 128);
        const uint32_t v_lo = desc_lo_mn_major(v_addr + s * A_TILE_BYTES);
        const uint32_t accumulate = (first && half == 0) ? 0u : 1u;
        if constexpr (SPLIT == 2)   // chunks half and 2 + half: columns 32 * chunk (+8 for the chunk's second k-step), keys 32 * chunk
          issue_value_products<8, 128, 64, 512, 72, 640>(o_tmem, tmem + (uint32_t)(t * 128 + 32 * half), v_lo + (uint32_t)(256 * half), kIdescPV,
                                                         accumulate);
        else                        // chunks 2 * half and 2 * half + 1
          issue_value_products<8, 128, 32, 256, 40, 384>(o_tmem, tmem + (uint32_t)(t * 128 + 64 * half), v_lo + (uint32_t)(512 * half), kIdescPV,
                                                         accumulate);
      };
      // scores of tile t for the step after (j, it): the next step of this item, or the first of the next item.
      // Steps, items and ring slots are counted along; the loop holds no division (see softmax_role).
      auto next_scores = [&](int t, int jn, int itn, int sn, uint32_t k_parity) -> bool {
        if (jn == 0 && !wait_all(q_full(t), (uint32_t)itn & 1u)) return failed(0x2100 | t);
        if (t == 0 && !wait_all(k_full(sn), k_parity)) return failed(0x2500);
        ptx::tc_fence_after();
        issue_qk(t, sn);
        ptx::umma_commit_led(leader, s_full(t));
        if (t == 1) ptx::umma_commit_led(leader, k_empty(sn));
        if (jn == num_kv - 1) ptx::umma_commit_led(leader, q_empty(t));   // the item's last read of this query tile
        return true;
      };
      ok = next_scores(0, 0, 0, 0, 0u) && next_scores(1, 0, 0, 0, 0u);
      int j = 0, it = 0;
      for (int g = 0; g < total_steps && ok; ++g) {
        const int s = g & 1;
        const uint32_t ph = (uint32_t)(g >> 1) & 1u;
        const bool more = g + 1 < total_steps, first = j == 0, last = j == num_kv - 1;
        const int jn = last ? 0 : j + 1, itn = last ? it + 1 : it, sn = s ^ 1;
        const uint32_t k_parity = (uint32_t)((g + 1) >> 1) & 1u;
        ATRACE(17, g, 0);
        if (!wait_all(v_full(s), ph)) { failed(0x2300); break; }
        if (!wait_all(p_half(0, 0), (uint32_t)g & 1u)) { failed(0x2400); break; }
        ptx::tc_fence_after();
        ATRACE(17, g, 1);
        if (early_pv) issue_pv(0, s, first, 0);
        DTN_DBG_COMMIT(0);
        if (!wait_all(p_half(0, 1), (uint32_t)g & 1u)) { failed(0x2400); break; }
        ptx::tc_fence_after();
        ATRACE(17, g, 2);
        if (!early_pv) issue_pv(0, s, first, 0);
        issue_pv(0, s, first, 1);
        DTN_DBG_COMMIT(1);
        if (last) ptx::umma_commit_led(leader, o_done(0));
        // At the end of an item the next item's queries may not have arrived yet: then the item's remaining value
        // products go first, so that its output can be normalised and stored while the queries are on their way.
        const bool scores_later = last && more && !__all_sync(0xffffffffu, ptx::mbar_test_wait(q_full(0), (uint32_t)itn & 1u));
        if (more && !scores_later && !next_scores(0, jn, itn, sn, k_parity)) break;
        DTN_DBG_COMMIT(2);
        ATRACE(17, g, 3);
        if (!wait_all(p_half(1, 0), (uint32_t)g & 1u)) { failed(0x2600); break; }
        ptx::tc_fence_after();
        ATRACE(17, g, 4);
        if (early_pv) issue_pv(1, s, first, 0);
        DTN_DBG_COMMIT(3);
        if (!wait_all(p_half(1, 1), (uint32_t)g & 1u)) { failed(0x2600); break; }
        ptx::tc_fence_after();
        ATRACE(17, g, 5);
        if (!early_pv) issue_pv(1, s, first, 0);
        issue_pv(1, s, first, 1);
        DTN_DBG_COMMIT(4);
        ptx::umma_commit_led(leader, v_empty(s));
        if (last) ptx::umma_commit_led(leader, o_done(1));
        if (scores_later && !next_scores(0, jn, itn, sn, k_parity)) break;
        if (more && !next_scores(1, jn, itn, sn, k_parity)) break;
        DTN_DBG_COMMIT(5);
        ATRACE(17, g, 6);
        j = jn;
        it = itn;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax + output -----------------------------------
    const int t = SPLIT == 4 ? 0 : warp / (4 * SPLIT);   // tile of this warp
    SoftmaxRole role;
    role.tmem_base = tmem_base;
    role.s_full = s_full(t);
    role.p_half0 = p_half(t, 0);
    role.p_half1 = p_half(t, 1);
    role.o_done = o_done(t);
    role.remote_arrive = false;
    role.xchg = xchg;
    role.xbar = x_bar(t, warp & 3);
    role.out_map = &tm_out;
    role.out_stage = (t == 0 ? k_addr : v_addr) + (uint32_t)(warp & 7) * 4096u;   // SPLIT == 2: the tile's eight warps, 4 KiB each
    role.staged_bar = staged(t);
    role.valid_last = S - (num_kv - 1) * A_BN;
    role.stage_base = stage_base;
    role.abort_flag = abort_flag;
    role.status = status;
    role.out = out;
    role.scale_log2e = scale_log2e;
    role.total_steps = total_steps;
    role.num_kv = num_kv;
    role.first_item = (int)blockIdx.x;
    role.item_stride = (int)gridDim.x;
    role.qblocks = qblocks;
    role.Hq = Hq;
    role.Hkv = Hkv;
    role.S = S;
    role.group_begin = group_begin;
    role.item_rows = 2 * A_BM;
    role.rows_before_tile = t * A_BM;
    role.rows_between_tiles = A_BM;
    if constexpr (SPLIT == 4) {
      role.s_full = s_full(0);
      role.p_half0 = p_half(0, 0);
      role.p_half1 = p_half(0, 1);
      role.o_done = o_done(0);
      role.rows_before_tile = 0;
      const SoftmaxBarrierStrides strides = {s_full(1) - s_full(0), p_half(1, 0) - p_half(0, 0), o_done(1) - o_done(0)};
      softmax_role_alternating(role, strides, warp, lane);
    } else {
      softmax_role<SPLIT, KEEP>(role, warp, lane);
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

// [heads][S][128] f16, box = 64 columns (128 bytes) x 128 rows of one head, 128-byte swizzle.
static int make_rows_map(CUtensorMap* map, const void* base, int64_t S, int64_t heads) {
  EncodeTiledFn enc = attn_encode_fn();
  DTN_REQUIRE(enc != nullptr, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {(cuuint64_t)A_D, (cuuint64_t)S, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {(cuuint64_t)A_D * 2, (cuuint64_t)S * A_D * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DTN_OK;
}

// [heads][S][128] FP32 output, box = 32 columns (128 bytes) x 32 rows of one head, 128-byte swizzle.
static int make_output_map(CUtensorMap* map, const void* base, int64_t S, int64_t heads) {
  EncodeTiledFn enc = attn_encode_fn();
  DTN_REQUIRE(enc != nullptr, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {(cuuint64_t)A_D, (cuuint64_t)S, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {(cuuint64_t)A_D * 4, (cuuint64_t)S * A_D * 4};
  const cuuint32_t box[3] = {32, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
  return DTN_OK;
}

// The tensor-core kernels take f16 storage and head_dim 128. Sequence length: a multiple of 256, or, for the form with
// kept scores (which masks missing keys and stores through a tensor map), anything from 256 up.
bool gqa_tc_ragged_supported(int64_t S, int64_t D, int storage) { return storage == DTN_STORAGE_F16 && D == A_D && S >= 2 * A_BM; }
bool gqa_tc_supported(int64_t S, int64_t D, int storage) {
  return storage == DTN_STORAGE_F16 && D == A_D && S >= 2 * A_BM && S % (2 * A_BM) == 0;
}

template <int SPLIT, bool KEEP = false>
static int gqa_tc_launch_t(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                           int64_t S, float scale, int64_t gb, int64_t ge, cudaStream_t s) {
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_rows_map(&mq, q, S, B * Hq))) return rc;
  if ((rc = make_rows_map(&mk, k, S, B * Hkv))) return rc;
  if ((rc = make_rows_map(&mv, v, S, B * Hkv))) return rc;
  CUtensorMap mo = mq;   // only the KEEP form stores through a tensor map
  if (KEEP && (rc = make_output_map(&mo, out, S, B * Hq))) return rc;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(gqa_tc_kernel<SPLIT, KEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, A_SMEM_BYTES));
    attr_dev = dev;
  }
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gqa: could not allocate the device status word");
  const int64_t items = (ge - gb) * (Hq / Hkv) * ((S + 2 * A_BM - 1) / (2 * A_BM));
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
  gqa_tc_kernel<SPLIT, KEEP><<<(unsigned)ctas, attn_threads(SPLIT), A_SMEM_BYTES, s>>>(mq, mk, mv, mo, out, (int)Hq, (int)Hkv, (int)S, scale_log2e,
                                                                                 (int)gb, (int)items, early_pv, status);
  DTN_LAUNCH_CHECK("gqa_tc_kernel");
  return DTN_OK;
}

#ifdef DTN_ATTN_TRACE
extern "C" int dtn_attn_trace_copy(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_attn_trace, sizeof(g_attn_trace));
}
#endif

int gqa_tc_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                  int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s) {
  if (split == 4) return gqa_tc_launch_t<4>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);
  if (split == 3) return gqa_tc_launch_t<2, true>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);   // two warpgroups, kept scores
  return split == 2 ? gqa_tc_launch_t<2>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s)
                    : gqa_tc_launch_t<1>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);
}

}  // namespace dtn
