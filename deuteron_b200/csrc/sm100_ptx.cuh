// Thin inline-PTX wrappers for the sm_100a units the tensor-core kernels use: mbarrier,
// TMA tile loads (cp.async.bulk.tensor), tensor memory (tcgen05.alloc/ld) and the
// tcgen05.mma issue/commit path. Every wait is bounded: it gives up after a cycle budget
// and reports failure instead of spinning forever.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "dtn_common.cuh"

namespace dtn {
namespace ptx {

// Cycle budget of one bounded wait (about half a second at B200 clocks). A healthy kernel
// waits microseconds; a wait that reaches this budget is reported, not retried.
constexpr long long kWaitBudgetCycles = 1000000000LL;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on a barrier that may live in another CTA of the cluster (shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// The same test without waiting at all (try_wait may sleep for a few microseconds before it answers "not yet").
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait. Returns false if the budget ran out or another role raised `abort_flag`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kWaitBudgetCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while the kernel before it in the stream is still running; grid_dependency_wait() blocks until
// that kernel has completed and its writes are visible. launch_dependents() lets the next kernel start.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tile load into this CTA's shared memory, completion counted on this CTA's barrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
      "%3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// The same with a third coordinate (a tile of one matrix out of a stack of them: rows past the matrix's own extent
// are filled with zeros by a load and dropped by a store, whatever lies behind them in memory).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x),
               "r"(y), "r"(z)
               : "memory");
}
// Asks for the same tile to be brought into L2 only (no destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
}
// Same for a CTA pair: the barrier may be the peer CTA's (shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], "
      "[%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}

// 2-D tile store from this CTA's shared memory, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(x), "r"(y), "r"(z), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Blocks until the stores of this thread's groups have READ their shared-memory source (the source may be reused).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Blocks until they are complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tensor memory -------------------------------------------------------------------
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem),
                 "r"(ncols)
                 : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base+i), r[j] = column j.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 columns load into r[0..16).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 columns store (registers -> tensor memory), same mapping as tmem_ld_32x32.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 32 lanes x 8 columns store: registers r[0..8) of lane l go to columns [c, c + 8) of tensor-memory lane l.
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- tcgen05.mma ---------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes and are
// stored with the 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B
// writes): 8-row groups are 1024 bytes apart (stride offset), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                  // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
  d |= (uint64_t)1 << 46;                  // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16 / kind::tf32 with FP32 accumulation, both operands
// K-major. fmt: 0 = f16, 1 = bf16, 2 = tf32.
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int m, int n) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]. KIND: 0 = kind::f16 (f16/bf16 operands), 1 = kind::tf32.
template <int KIND, int CTAS>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (KIND == 0 && CTAS == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (KIND == 0 && CTAS == 2)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (KIND == 1 && CTAS == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem] (A operand read from tensor memory), one CTA, kind::f16.
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same instructions issued by one lane of a warp whose 32 lanes all walk the issue loop: `leader` is 1 in the
// issuing lane and 0 in the others. With the loop's control flow and operands uniform across the warp the descriptors
// and addresses stay in uniform registers, which is where the instruction takes them from.
__device__ __forceinline__ void umma_ss_f16_led(uint32_t leader, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void umma_ts_f16_led(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void umma_commit_led(uint32_t leader, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar),
      "r"(leader)
      : "memory");
}

// The two 32-bit words of umma_desc_sw128: the high word is the same for every K-major, 128-byte-swizzled operand.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_sw128(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }

// One 128-byte k-block of a compensated product on one CTA or a CTA pair: four k-steps of 16 (32 bytes: +2 in the address
// field), per step lo*hi, hi*lo, hi*hi into the same accumulator. All 32 lanes of the issuing warp reach this block;
// `elect.sync` picks the lane that issues all twelve instructions, and every operand is uniform across the warp, so
// descriptors and addresses stay in uniform registers. KIND: 0 = bf16 planes (kind::f16), 1 = tf32 planes.
template <int KIND, int CTAS>
__device__ __forceinline__ void umma_x3_kblock(uint32_t d_tmem, uint32_t a_hi, uint32_t a_lo, uint32_t b_hi, uint32_t b_lo,
                                                    uint32_t idesc, uint32_t accumulate_first) {
#define DTN_X3_STEP(MMA, OFF, FIRST)                                                                                      \
  "add.u32 ah, %1, " #OFF ";\n\tadd.u32 al, %2, " #OFF ";\n\tadd.u32 bh, %3, " #OFF ";\n\tadd.u32 bl, %4, " #OFF ";\n\t" \
  "mov.b64 dah, {ah, %5};\n\tmov.b64 dal, {al, %5};\n\tmov.b64 dbh, {bh, %5};\n\tmov.b64 dbl, {bl, %5};\n\t"          \
  "@q " MMA " [%0], dal, dbh, %6, " FIRST ";\n\t"                                                                         \
  "@q " MMA " [%0], dah, dbl, %6, yes;\n\t"                                                                               \
  "@q " MMA " [%0], dah, dbh, %6, yes;\n\t"
#define DTN_X3_BLOCK(MMA)                                                                                        \
  asm volatile(                                                                                                  \
      "{\n\t.reg .pred q, acc, yes;\n\t.reg .b32 ah, al, bh, bl;\n\t.reg .b64 dah, dal, dbh, dbl;\n\t"          \
      "elect.sync _|q, 0xffffffff;\n\t"                                                                          \
      "setp.ne.b32 acc, %7, 0;\n\tsetp.eq.b32 yes, 0, 0;\n\t"                                                    \
      DTN_X3_STEP(MMA, 0, "acc") DTN_X3_STEP(MMA, 2, "yes") DTN_X3_STEP(MMA, 4, "yes") DTN_X3_STEP(MMA, 6, "yes") \
      "}" ::"r"(d_tmem), "r"(a_hi), "r"(a_lo), "r"(b_hi), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(accumulate_first) \
      : "memory")
  if constexpr (KIND == 0 && CTAS == 2) DTN_X3_BLOCK("tcgen05.mma.cta_group::2.kind::f16");
  else if constexpr (KIND == 1 && CTAS == 2) DTN_X3_BLOCK("tcgen05.mma.cta_group::2.kind::tf32");
  else if constexpr (KIND == 0) DTN_X3_BLOCK("tcgen05.mma.cta_group::1.kind::f16");
  else DTN_X3_BLOCK("tcgen05.mma.cta_group::1.kind::tf32");
#undef DTN_X3_BLOCK
#undef DTN_X3_STEP
}
// umma_commit issued by the elected lane of a warp whose 32 lanes all reach it.
template <int CTAS>
__device__ __forceinline__ void umma_commit_elected(uint32_t bar) {
  if constexpr (CTAS == 1) {
    umma_commit_led(1u, bar);
  } else {
    const uint16_t mask = 3;
    asm volatile(
        "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}" ::"r"(bar),
        "h"(mask)
        : "memory");
  }
}

// Make `bar` complete one arrival once every tcgen05.mma issued so far by this thread
// has finished. With CTAS == 2 the arrival is delivered to the barrier at the same
// shared-memory offset in both CTAs of the pair.
template <int CTAS>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (CTAS == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
  } else {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], "
        "%1;" ::"r"(bar),
        "h"(mask)
        : "memory");
  }
}

}  // namespace ptx
}  // namespace dtn
