// Compensated FP32 GEMM for mid-size problems: one kernel, operand split inside the producer warps,
// products on tcgen05 with the accumulator in tensor memory.
//
// Between the single-kernel mma.sync path (up to about 512^3) and the sizes where a separate split
// pass is a few percent of the run time (4096^3 and up), the split pass and its round trip through
// the operand planes are a third of the time. Here eight producer warps read the FP32 tiles of A and
// B straight from global memory, round them to a high part and a residual in registers (the same
// arithmetic as the split kernels, so the operands of every product are the same bits) and write the
// four planes into shared memory in the layouts tcgen05.mma reads: A K-major (128-byte rows, 128-byte
// swizzle), B MN-major (rows of 128 bytes along n, one row per k, 128-byte swizzle), which is the
// order B is stored in, so no transposition is needed. One thread of a ninth warp issues the three
// products per k-step in the usual order (lo*hi, hi*lo, hi*hi); the producer warps read the
// accumulator back and store C at the end. One output tile per CTA.
//
// Measured on B200 it only matches the two-kernel path up to 1024^3 (18.2 against 17.1 us) and loses beyond
// (2048^3: 84 against 48 us): with one 128 x 64 or 128 x 128 tile per CTA the operands are re-read from L2
// 16 to 32 times, FP32 operands are as many bytes as the two bf16 planes, and the run time is those bytes at
// about 6.4 TB/s. Larger tiles cannot take the split in: a 256 x 256 CTA-pair tile already reads its operands
// at 94 of the 128 bytes per clock shared memory delivers, and the producers' 64 KiB of stores per k-block
// would push it past that. The kernel therefore stays an explicit variant (one launch, no workspace).
#include "sm100_ptx.cuh"

namespace dtn {

// PW producer warps (8 or 16), which also run the epilogue, then one warp that issues the products and owns the tensor memory.
template <int BN, int PW>
struct FusedCfg {
  static constexpr int kThreads = (PW + 1) * 32;
  static constexpr int kBK = 64;                             // k per k-block = bf16 elements per 128-byte row of A
  static constexpr int kPer16 = 8;                           // operand elements per 16-byte piece
  static constexpr int kNBlock = 64;                         // n per 128-byte row of B
  static constexpr int kABytes = 128 * 128;                  // A plane: 128 rows of 128 bytes
  static constexpr int kBBlockBytes = kBK * 128;             // B plane, one n-block: kBK rows (k) of 128 bytes
  static constexpr int kBBytes = (BN / kNBlock) * kBBlockBytes;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes > 4 ? 4 : (192 * 1024) / kStageBytes;
  static constexpr int kAUnits = 128 * 8 / (PW * 32);              // 16-byte pieces of A per thread and k-block
  static constexpr int kBUnits = kBK * (BN / kPer16) / (PW * 32);  // of B
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
  static_assert(BN == 64 || BN == 128, "tile width");
  static_assert(kStages >= 3, "ring too shallow");
};

// Shared-memory descriptor of an MN-major operand with the 128-byte swizzle: rows of 128 bytes along n, one row per
// k; groups of eight rows 1024 bytes apart (stride offset), blocks of one row width along n `block_bytes` apart
// (leading offset).
__device__ __forceinline__ uint64_t fused_desc_mn_sw128(uint32_t smem_addr, uint32_t block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)(block_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// hi = bf16_rn(v), lo = bf16_rn(v - hi) for two values, packed (first value in the low half).
__device__ __forceinline__ void fused_split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const float ha = __uint_as_float(hi << 16), hb = __uint_as_float(hi & 0xffff0000u);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - ha, b - hb);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// One 16-byte piece of each plane from eight FP32 values.
__device__ __forceinline__ void fused_split_piece(const float4 (&v)[2], uint4& hi, uint4& lo) {
  fused_split_bf16(v[0].x, v[0].y, hi.x, lo.x);
  fused_split_bf16(v[0].z, v[0].w, hi.y, lo.y);
  fused_split_bf16(v[1].x, v[1].y, hi.z, lo.z);
  fused_split_bf16(v[1].z, v[1].w, hi.w, lo.w);
}

template <int BN, int PW>
__global__ void __launch_bounds__((PW + 1) * 32, 1)
gemm_x3_fused_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                     int64_t lda, int64_t ldb, int64_t ldc, int c_vec_ok, int* __restrict__ status) {
  using Cfg = FusedCfg<BN, PW>;
  constexpr int kStages = Cfg::kStages, BK = Cfg::kBK, P16 = Cfg::kPer16, V = P16 / 4;
  constexpr int kProducerThreads = PW * 32;
  constexpr int kBPiecesPerRow = BN / P16;
  constexpr uint32_t kIdesc = ptx::umma_idesc(1, 128, BN) | (1u << 16);   // bf16 operands, B MN-major

  extern __shared__ uint8_t fused_smem[];
  const uint32_t raw_addr = smem_u32(fused_smem);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* bar_ptr = fused_smem + (tiles_addr - raw_addr) + kStages * Cfg::kStageBytes;
  const uint32_t bar_addr = tiles_addr + kStages * Cfg::kStageBytes;
  // barrier block (8-byte slots): full[kStages] (one arrival per producer warp), empty[kStages], accumulator complete
  auto full_bar = [&](int s) { return bar_addr + 8u * s; };
  auto empty_bar = [&](int s) { return bar_addr + 8u * (kStages + s); };
  const uint32_t done_bar = bar_addr + 8u * (2 * kStages);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_ptr + 8 * (2 * kStages + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * kStages + 1) + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * BN;
  const int num_kb = (K + BK - 1) / BK;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), PW);
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(done_bar, 1);
    ptx::mbar_fence_init();
  }
  if (warp == PW) {
    ptx::tmem_alloc<1>(smem_u32(tmem_holder), BN);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < PW) {
    // ------------------------------- producers ----------------------------------------------
    // Piece u of a tile belongs to thread u % 256. A: row u / 8, piece u % 8 of the row's eight. B: k row
    // u / kBPiecesPerRow, piece u % kBPiecesPerRow along n. Eight (A) or kBPiecesPerRow (B) neighbouring threads read
    // one contiguous row segment.
    // Everything that does not change from one k-block to the next is worked out once: where the piece comes from,
    // whether its row (A) or columns (B) exist, its k offset inside the block and where it goes in a stage.
    constexpr int kUnits = Cfg::kAUnits + Cfg::kBUnits;
    const float4* src[kUnits];
    uint32_t dst[kUnits];
    int k_in_block[kUnits];
#pragma unroll
    for (int i = 0; i < Cfg::kAUnits; ++i) {
      const int u = i * kProducerThreads + tid, row = u >> 3, piece = u & 7;
      const bool in = m0 + row < M;
      src[i] = reinterpret_cast<const float4*>(A + (int64_t)(in ? m0 + row : 0) * lda + piece * P16);
      k_in_block[i] = in ? piece * P16 : (1 << 30);   // an absent row never passes the k < K test
      dst[i] = (uint32_t)(row * 128 + ((piece ^ (row & 7)) << 4));
    }
#pragma unroll
    for (int i = 0; i < Cfg::kBUnits; ++i) {
      const int u = i * kProducerThreads + tid, krow = u / kBPiecesPerRow, pc = u % kBPiecesPerRow;
      const int n = pc * P16, block = n / Cfg::kNBlock, piece = (n % Cfg::kNBlock) / P16;
      const bool in = n0 + n < N;
      src[Cfg::kAUnits + i] = reinterpret_cast<const float4*>(B + (int64_t)krow * ldb + (in ? n0 + n : 0));
      k_in_block[Cfg::kAUnits + i] = in ? krow : (1 << 30);
      dst[Cfg::kAUnits + i] =
          (uint32_t)(2 * Cfg::kABytes + block * Cfg::kBBlockBytes + krow * 128 + ((piece ^ (krow & 7)) << 4));
    }
    const int64_t a_step = BK / 4, b_step = (int64_t)BK * ldb / 4;   // float4 per k-block (ldb is a multiple of 4)

    float4 regs[2][kUnits][V];
    auto load = [&](int kb, float4 (&r)[kUnits][V]) {
      const int k_left = K - kb * BK;
      const int64_t a_at = kb * a_step, b_at = kb * b_step;
#pragma unroll
      for (int i = 0; i < kUnits; ++i) {
        const float4* p = src[i] + (i < Cfg::kAUnits ? a_at : b_at);
        const bool in = k_in_block[i] < k_left;
#pragma unroll
        for (int v = 0; v < V; ++v) r[i][v] = in ? __ldg(p + v) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    };
    auto store = [&](int stage, const float4 (&r)[kUnits][V]) {
      const uint32_t base = tiles_addr + stage * Cfg::kStageBytes;
#pragma unroll
      for (int i = 0; i < kUnits; ++i) {
        uint4 hi, lo;
        fused_split_piece(r[i], hi, lo);
        st_shared_v4(base + dst[i], hi);                                                  // high plane
        st_shared_v4(base + dst[i] + (i < Cfg::kAUnits ? Cfg::kABytes : Cfg::kBBytes), lo);   // residual plane behind it
      }
    };
    // hands k-block kb (held in r) to the tensor core; false when a wait ran out
    auto publish = [&](int kb, const float4 (&r)[kUnits][V]) -> bool {
      const int stage = kb % kStages;
      const uint32_t phase = (uint32_t)(kb / kStages) & 1u;
      const bool free_slot = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
      if (!__all_sync(0xffffffffu, free_slot)) {
        if (lane == 0) atomicExch(status, 0x5100 | (int)(blockIdx.x & 0xff));
        return false;
      }
      store(stage, r);
      ptx::fence_proxy_async_smem();   // the tensor core reads shared memory through the async proxy
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(full_bar(stage));
      return true;
    };
    bool ok = true;
    load(0, regs[0]);
    for (int kb = 0; kb < num_kb && ok; kb += 2) {
      // the next k-block's loads are in flight while this one is converted
      if (kb + 1 < num_kb) load(kb + 1, regs[1]);
      ok = publish(kb, regs[0]);
      if (!ok || kb + 1 >= num_kb) break;
      if (kb + 2 < num_kb) load(kb + 2, regs[0]);
      ok = publish(kb + 1, regs[1]);
    }

    // ------------------------------- epilogue -----------------------------------------------
    const bool ready = ok && ptx::mbar_wait(done_bar, 0u, abort_flag);
    if (!__all_sync(0xffffffffu, ready)) {
      if (lane == 0 && ok) atomicExch(status, 0x5300 | (int)(blockIdx.x & 0xff));
    } else {
      ptx::tc_fence_after();
      const int quarter = warp & 3, part = warp >> 2;   // tensor-memory lanes [32 * quarter, +32); 32-column chunks part, part + PW / 4, ...
      const int row = m0 + quarter * 32 + lane;
      float* crow = C + (int64_t)row * ldc + n0;
#pragma unroll 1
      for (int c = part; c < BN / 32; c += PW / 4) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
        ptx::tmem_ld_wait();
        if (row < M) {
          if (c_vec_ok && n0 + c * 32 + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(crow + c * 32 + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c * 32 + j < N) crow[c * 32 + j] = __uint_as_float(r[j]);
          }
        }
      }
    }
  } else if (lane == 0) {
    // ------------------------------- MMA issuer ---------------------------------------------
    bool ok = true;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int stage = kb % kStages;
      const uint32_t phase = (uint32_t)(kb / kStages) & 1u;
      if (!ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
        atomicExch(status, 0x5200 | (int)(blockIdx.x & 0xff));
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t a_hi = tiles_addr + stage * Cfg::kStageBytes, a_lo = a_hi + Cfg::kABytes;
      const uint32_t b_hi = a_lo + Cfg::kABytes, b_lo = b_hi + Cfg::kBBytes;
      const uint64_t da_hi = ptx::umma_desc_sw128(a_hi), da_lo = ptx::umma_desc_sw128(a_lo);
      const uint64_t db_hi = fused_desc_mn_sw128(b_hi, Cfg::kBBlockBytes), db_lo = fused_desc_mn_sw128(b_lo, Cfg::kBBlockBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // one k-step of 16: 32 bytes along A's swizzled rows (+2 in the address field); 16 rows of 128 bytes of B
        const uint64_t oa = (uint64_t)(2 * k), ob = (uint64_t)(k * (BK / 4) * 128 / 16);
        ptx::umma_ss<0, 1>(tmem_base, da_lo + oa, db_hi + ob, kIdesc, (kb | k) != 0 ? 1u : 0u);
        ptx::umma_ss<0, 1>(tmem_base, da_hi + oa, db_lo + ob, kIdesc, 1u);
        ptx::umma_ss<0, 1>(tmem_base, da_hi + oa, db_hi + ob, kIdesc, 1u);
      }
      ptx::umma_commit<1>(empty_bar(stage));   // frees the slot once the products have read it
    }
    if (ok) ptx::umma_commit<1>(done_bar);
  }

  // ------------------------------- teardown -------------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out: give products already issued time to finish before shared and tensor memory are released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == PW) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, BN);
  }
}

template <int BN, int PW>
static int launch_fused(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                        int64_t ldc, cudaStream_t s) {
  using Cfg = FusedCfg<BN, PW>;
  auto kernel = gemm_x3_fused_kernel<BN, PW>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_dev = dev;
  }
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "gemm: could not allocate the device status word");
  const dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + 127) / 128));
  DTN_REQUIRE(grid.y <= 65535, DTN_ERR_UNSUPPORTED, "gemm: M too large for the fused-split kernel");
  const int c_vec_ok = aligned_to(C, 16) && (ldc % 4 == 0);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, s>>>(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc, c_vec_ok, status);
  DTN_LAUNCH_CHECK("gemm_x3_fused_kernel");
  return DTN_OK;
}

// Whether the fused-split kernel can take the problem: bf16x3 only (B is consumed in its stored, n-contiguous order,
// which for 32-bit operands needs a different swizzle), 128-bit loads of whole 16-byte operand pieces.
bool gemm_fused_supported(int mode, const float* A, const float* B, int64_t N, int64_t K, int64_t lda, int64_t ldb) {
  return mode == DTN_GEMM_BF16X3 && aligned_to(A, 16) && aligned_to(B, 16) && lda % 4 == 0 && ldb % 4 == 0 && K % 8 == 0 &&
         N % 8 == 0;
}

// bn: 64 or 128 columns per tile; 0 picks 64 while 128-wide tiles would leave SMs without one.
int gemm_fused_launch(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, cudaStream_t s, int bn) {
  DTN_REQUIRE(gemm_fused_supported(mode, A, B, N, K, lda, ldb), DTN_ERR_UNSUPPORTED,
              "gemm: the fused-split kernel takes bf16x3 with 16-byte aligned A and B, leading dimensions that are multiples "
              "of 4 and N, K multiples of 8");
  if (bn == 0) bn = ((M + 127) / 128) * ((N + 127) / 128) >= sm_count() ? 128 : 64;
  // sixteen producer warps for the wide tile (measured 84 against 144 us at 2048^3), eight for the narrow one (no difference)
  return bn == 128 ? launch_fused<128, 16>(A, B, C, M, N, K, lda, ldb, ldc, s) : launch_fused<64, 8>(A, B, C, M, N, K, lda, ldb, ldc, s);
}

}  // namespace dtn
