// Grouped-query attention forward on CTA pairs (tcgen05.mma.cta_group::2), f16 storage, head_dim 128.
//
// Same algorithm, softmax code and tensor-memory layout as attention_tc.cu; what changes is who holds
// the operands. A pair of CTAs (a cluster of two) works on 512 query rows of one head: two 256-row
// super-tiles, of which each CTA owns 128 rows (its own queries in shared memory, its own scores,
// probabilities and output accumulator in tensor memory). Every product is one 256-row instruction
// issued by the leader CTA for both:
//   S = Q K^T   B operand = the 128 keys of the step, 64 in each CTA's shared memory
//   O += P V    B operand = the 128 value columns, 64 in each CTA's shared memory
// so each CTA loads and reads only half of every K and V tile. With one CTA per tile the score product
// reads 128 B/clk from shared memory (its whole bandwidth); here it reads 96 B/clk, and the K/V traffic
// from L2 halves. The freed shared memory makes the K/V ring four steps deep.
//
// Barriers: loads of both CTAs complete on the leader's barriers (it posts the byte count of the
// pair); the leader's MMA warp releases buffers and publishes scores with commits that arrive at the
// same barrier in both CTAs; the softmax warps of both CTAs arrive on the leader's probability
// barriers. No TMA multicast is used.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>

#include <mutex>

#include "attention_tc.cuh"

namespace dtn {

constexpr int P_KV_STAGES = 4;
constexpr int P_KV_BYTES = 16 * 1024;   // this CTA's half of a K tile (64 keys x 128 d) or of a V tile (128 keys x 64 d)
constexpr int P_SMEM_TILES_BYTES = 2 * A_TILE_BYTES + 2 * P_KV_STAGES * P_KV_BYTES;
constexpr int P_SMEM_BYTES = P_SMEM_TILES_BYTES + 256 + A_XCHG_BYTES + A_STAGE_BYTES + 1024;
constexpr int P_ITEM_ROWS = 4 * A_BM;   // 512 query rows per pair and work item

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  // acquire at cluster scope: the arrivals come from the other CTA as well
  auto probe = [&]() {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
  };
  if (probe()) return true;
  const long long start = clock64();
  while (true) {
    if (probe()) return true;
    if (*abort_flag) return false;
    if (clock64() - start > ptx::kWaitBudgetCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// D[tmem] (+)= A[tmem] * B[smem] on a CTA pair (each CTA reads its own rows of A from its tensor memory).
__device__ __forceinline__ void umma_ts_f16_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int SPLIT>
__global__ void __launch_bounds__(attn_threads(SPLIT), 1)
gqa_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, float* __restrict__ out, int Hq, int Hkv, int S,
                   float scale_log2e, int group_begin, int total_items, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t q_addr = base;                                   // 2 tiles of this CTA's 128 rows
  const uint32_t k_addr = base + 2 * A_TILE_BYTES;                // P_KV_STAGES half tiles
  const uint32_t v_addr = k_addr + P_KV_STAGES * P_KV_BYTES;      // P_KV_STAGES half tiles
  const uint32_t bar_addr = base + P_SMEM_TILES_BYTES;
  uint8_t* bar_ptr = base_ptr + P_SMEM_TILES_BYTES;
  auto q_full = [&](int t) { return bar_addr + 8u * (0 + t); };
  auto q_empty = [&](int t) { return bar_addr + 8u * (2 + t); };
  auto s_full = [&](int t) { return bar_addr + 8u * (4 + t); };
  auto o_done = [&](int t) { return bar_addr + 8u * (6 + t); };
  auto p_half = [&](int t, int h) { return bar_addr + 8u * (8 + 2 * t + h); };
  auto k_full = [&](int s) { return bar_addr + 8u * (12 + s); };
  auto v_full = [&](int s) { return bar_addr + 8u * (12 + P_KV_STAGES + s); };
  auto k_empty = [&](int s) { return bar_addr + 8u * (12 + 2 * P_KV_STAGES + s); };
  auto v_empty = [&](int s) { return bar_addr + 8u * (12 + 3 * P_KV_STAGES + s); };
  constexpr int kBarriers = 12 + 4 * P_KV_STAGES;
  static_assert(kBarriers * 8 + 16 <= 256, "barrier block too small");
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * kBarriers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * kBarriers + 8);
  volatile float2* xchg = reinterpret_cast<volatile float2*>(bar_ptr + 256);
  float* stage_base = reinterpret_cast<float*>(bar_ptr + 256 + A_XCHG_BYTES);
  constexpr int kTmaWarp = 8 * SPLIT, kMmaWarp = 8 * SPLIT + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)ptx::cluster_ctarank();
  const int pair = (int)blockIdx.x >> 1, num_pairs = (int)gridDim.x >> 1;
  const int qblocks = S / P_ITEM_ROWS;
  const int num_kv = S / A_BN;
  const int my_items = pair < total_items ? (total_items - 1 - pair) / num_pairs + 1 : 0;
  const int total_steps = my_items * num_kv;

  for (int i = threadIdx.x; i < A_XCHG_BYTES / 8; i += blockDim.x) {
    xchg[i].x = 0.f;
    xchg[i].y = 0.f;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < P_KV_STAGES; ++s) {
      ptx::mbar_init(k_full(s), 1);
      ptx::mbar_init(v_full(s), 1);
      ptx::mbar_init(k_empty(s), 1);
      ptx::mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(q_full(t), 1);
      ptx::mbar_init(q_empty(t), 1);
      ptx::mbar_init(s_full(t), 1);
      ptx::mbar_init(o_done(t), 1);
      ptx::mbar_init(p_half(t, 0), 2 * 4 * SPLIT);   // one arrival per softmax warp of both CTAs (used in the leader)
      ptx::mbar_init(p_half(t, 1), 2 * 4 * SPLIT);
    }
    ptx::mbar_fence_init();
    ptx::fence_proxy_async_smem();
    ptx::tma_prefetch_desc(&tm_q);
    ptx::tma_prefetch_desc(&tm_k);
    ptx::tma_prefetch_desc(&tm_v);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc<2>(smem_u32(tmem_holder), 512);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();   // the peer's barriers are initialised before anything is sent to them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == kTmaWarp) {
    // ------------------------------------ TMA producer (both CTAs) ---------------------------
    if (lane == 0) {
      const uint32_t lead_q_full0 = ptx::map_to_cta(q_full(0), 0);
      const uint32_t lead_k_full0 = ptx::map_to_cta(k_full(0), 0);
      const uint32_t lead_v_full0 = ptx::map_to_cta(v_full(0), 0);
      int g = 0;
      bool ok = true;
      for (int it = 0; it < my_items && ok; ++it) {
        const AttnItem item = attn_item(pair + it * num_pairs, qblocks, Hq, Hkv, S, group_begin, P_ITEM_ROWS);
        for (int j = 0; j < num_kv; ++j, ++g) {
          const int s = g % P_KV_STAGES;
          const uint32_t ph = (uint32_t)(g / P_KV_STAGES) & 1u;
          if (!ptx::mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1100); ok = false; break; }
          if (rank == 0) ptx::mbar_expect_tx(k_full(s), 2 * P_KV_BYTES);
          for (int h = 0; h < 2; ++h)   // this CTA's 64 keys, two 64-element halves of the head dimension
            ptx::tma_load_2d_pair(k_addr + s * P_KV_BYTES + h * (P_KV_BYTES / 2), &tm_k, h * 64,
                                  item.kv_row0 + j * A_BN + rank * 64, lead_k_full0 + 8u * s);
          if (!ptx::mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { atomicExch(status, 0x1200); ok = false; break; }
          if (rank == 0) ptx::mbar_expect_tx(v_full(s), 2 * P_KV_BYTES);
          // this CTA's 64 value columns of all 128 keys
          ptx::tma_load_2d_pair(v_addr + s * P_KV_BYTES, &tm_v, rank * 64, item.kv_row0 + j * A_BN, lead_v_full0 + 8u * s);
          if (j == 0) {
            for (int t = 0; t < 2 && ok; ++t) {
              if (it > 0 && !ptx::mbar_wait(q_empty(t), (uint32_t)(it - 1) & 1u, abort_flag)) { atomicExch(status, 0x1300); ok = false; break; }
              if (rank == 0) ptx::mbar_expect_tx(q_full(t), 2 * A_TILE_BYTES);
              for (int h = 0; h < 2; ++h)
                ptx::tma_load_2d_pair(q_addr + t * A_TILE_BYTES + h * A_HALF_BYTES, &tm_q, h * 64,
                                      item.q_row0 + t * (2 * A_BM) + rank * A_BM, lead_q_full0 + 8u * t);
            }
            if (!ok) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------ MMA issuer (leader CTA only) -----------------------
    if (lane == 0 && rank == 0 && total_steps > 0) {
      constexpr uint32_t kIdescQK = ptx::umma_idesc(0, 256, 128);
      constexpr uint32_t kIdescPV = ptx::umma_idesc(0, 256, 128) | (1u << 16);   // B (values) is MN-major
      bool ok = true;
      // S_t = Q_t K^T : 8 k-steps of 16 along the head dimension
      auto issue_qk = [&](int t, int s) {
        const uint32_t qa = q_addr + t * A_TILE_BYTES, ka = k_addr + s * P_KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t q_off = (uint32_t)(kk >> 2) * A_HALF_BYTES + (uint32_t)(kk & 3) * 32u;
          const uint32_t k_off = (uint32_t)(kk >> 2) * (P_KV_BYTES / 2) + (uint32_t)(kk & 3) * 32u;
          ptx::umma_ss<0, 2>(tmem_base + (uint32_t)(t * 128), ptx::umma_desc_sw128(qa + q_off),
                             ptx::umma_desc_sw128(ka + k_off), kIdescQK, kk ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int s, bool first, int half) {
        const uint32_t va = v_addr + s * P_KV_BYTES;
        const uint32_t o_tmem = tmem_base + (uint32_t)(256 + t * 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int chunk = SPLIT == 2 ? 2 * (i >> 1) + half : 2 * half + (i >> 1);
          const int kk = 2 * chunk + (i & 1);
          const uint32_t p_col = tmem_base + (uint32_t)(t * 128 + 32 * (kk >> 1) + 8 * (kk & 1));
          const uint64_t vd = umma_desc_mn_sw128(va + (uint32_t)kk * 2048u);
          umma_ts_f16_pair(o_tmem, p_col + 16u, vd, kIdescPV, (first && half == 0 && i == 0) ? 0u : 1u);
          umma_ts_f16_pair(o_tmem, p_col, vd, kIdescPV, 1u);
        }
      };
      auto next_scores = [&](int t, int g) -> bool {
        const int gn = g + 1, jn = gn % num_kv, sn = gn % P_KV_STAGES;
        if (jn == 0 && !ptx::mbar_wait(q_full(t), (uint32_t)(gn / num_kv) & 1u, abort_flag)) { atomicExch(status, 0x2100 | t); return false; }
        if (t == 0 && !ptx::mbar_wait(k_full(sn), (uint32_t)(gn / P_KV_STAGES) & 1u, abort_flag)) { atomicExch(status, 0x2500); return false; }
        ptx::tc_fence_after();
        issue_qk(t, sn);
        ptx::umma_commit<2>(s_full(t));
        if (t == 1) ptx::umma_commit<2>(k_empty(sn));
        if (jn == num_kv - 1) ptx::umma_commit<2>(q_empty(t));
        return true;
      };
      ok = next_scores(0, -1) && next_scores(1, -1);
      for (int g = 0; g < total_steps && ok; ++g) {
        const int s = g % P_KV_STAGES, j = g % num_kv;
        const uint32_t ph = (uint32_t)(g / P_KV_STAGES) & 1u;
        const bool more = g + 1 < total_steps, first = j == 0, last = j == num_kv - 1;
        if (!ptx::mbar_wait(v_full(s), ph, abort_flag)) { atomicExch(status, 0x2300); break; }
        if (!mbar_wait_cluster(p_half(0, 0), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2400); break; }
        ptx::tc_fence_after();
        issue_pv(0, s, first, 0);
        if (!mbar_wait_cluster(p_half(0, 1), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2400); break; }
        ptx::tc_fence_after();
        issue_pv(0, s, first, 1);
        if (last) ptx::umma_commit<2>(o_done(0));
        if (more && !next_scores(0, g)) break;
        if (!mbar_wait_cluster(p_half(1, 0), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2600); break; }
        ptx::tc_fence_after();
        issue_pv(1, s, first, 0);
        if (!mbar_wait_cluster(p_half(1, 1), (uint32_t)g & 1u, abort_flag)) { atomicExch(status, 0x2600); break; }
        ptx::tc_fence_after();
        issue_pv(1, s, first, 1);
        ptx::umma_commit<2>(v_empty(s));
        if (last) ptx::umma_commit<2>(o_done(1));
        if (more && !next_scores(1, g)) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax + output (both CTAs) -----------------------
    const int t = warp / (4 * SPLIT);
    SoftmaxRole role;
    role.tmem_base = tmem_base;
    role.s_full = s_full(t);
    role.p_half0 = ptx::map_to_cta(p_half(t, 0), 0);
    role.p_half1 = ptx::map_to_cta(p_half(t, 1), 0);
    role.o_done = o_done(t);
    role.remote_arrive = true;
    role.xchg = xchg;
    role.stage_base = stage_base;
    role.abort_flag = abort_flag;
    role.status = status;
    role.out = out;
    role.scale_log2e = scale_log2e;
    role.total_steps = total_steps;
    role.num_kv = num_kv;
    role.first_item = pair;
    role.item_stride = num_pairs;
    role.qblocks = qblocks;
    role.Hq = Hq;
    role.Hkv = Hkv;
    role.S = S;
    role.group_begin = group_begin;
    role.item_rows = P_ITEM_ROWS;
    role.rows_before_tile = t * (2 * A_BM) + rank * A_BM;
    role.rows_between_tiles = 2 * A_BM;
    softmax_role<SPLIT>(role, warp, lane);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  ptx::cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers or read its memory
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<2>(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*PairEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PairEncodeTiledFn pair_encode_fn() {
  static PairEncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PairEncodeTiledFn>(p);
  });
  return fn;
}

// [rows, 128] f16 matrix, box = 64 columns (128 bytes) x box_rows rows, 128-byte swizzle.
static int make_pair_map(CUtensorMap* map, const void* base, int64_t rows, int box_rows) {
  PairEncodeTiledFn enc = pair_encode_fn();
  DTN_REQUIRE(enc != nullptr, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)A_D, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)A_D * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DTN_REQUIRE(r == CUDA_SUCCESS, DTN_ERR_CUDA, "gqa: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DTN_OK;
}

bool gqa_tc_pair_supported(int64_t S, int64_t D, int storage) {
  return storage == DTN_STORAGE_F16 && D == A_D && S >= P_ITEM_ROWS && S % P_ITEM_ROWS == 0;
}

template <int SPLIT>
static int gqa_tc_pair_launch_t(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                                int64_t S, float scale, int64_t gb, int64_t ge, cudaStream_t s) {
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_pair_map(&mq, q, B * Hq * S, 128))) return rc;
  if ((rc = make_pair_map(&mk, k, B * Hkv * S, 64))) return rc;    // a CTA's half of a K tile: 64 keys
  if ((rc = make_pair_map(&mv, v, B * Hkv * S, 128))) return rc;   // a CTA's half of a V tile: 128 keys x 64 columns
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(gqa_tc_pair_kernel<SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
    attr_dev = dev;
  }
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gqa: could not allocate the device status word");
  const int64_t items = (ge - gb) * (Hq / Hkv) * (S / P_ITEM_ROWS);
  DTN_REQUIRE(items < (1LL << 31) && B * Hq * S < (1LL << 31), DTN_ERR_UNSUPPORTED, "gqa: too many query rows for one launch");
  int64_t pairs = sm_count() / 2;
  if (items < pairs) pairs = items;
  const float scale_log2e = scale * 1.4426950408889634f;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(attn_threads(SPLIT));
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DTN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gqa_tc_pair_kernel<SPLIT>, mq, mk, mv, out, (int)Hq, (int)Hkv, (int)S, scale_log2e, (int)gb,
                                    (int)items, status));
  return DTN_OK;
}

int gqa_tc_pair_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                       int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s) {
  return split == 2 ? gqa_tc_pair_launch_t<2>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s)
                    : gqa_tc_pair_launch_t<1>(q, k, v, out, B, Hq, Hkv, S, scale, gb, ge, s);
}

}  // namespace dtn
