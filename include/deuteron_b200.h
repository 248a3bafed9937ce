/*
 * deuteron_b200 — C ABI of the B200 (sm_100a) kernels that stand in for the code the
 * Deuteron compiler emits for its hot workloads.
 *
 * Conventions
 *   - Every function returns an int status: 0 = ok, non-zero = DTN_ERR_* below.
 *     dtn_last_error() gives the text of the calling thread's last failure.
 *   - Pointers are DEVICE pointers unless a parameter says "host". The caller owns every
 *     buffer. Buffers must not overlap. Nothing here allocates or frees device memory
 *     (except where a function's comment says otherwise) and nothing synchronises the
 *     stream: work is enqueued on `stream` (a cudaStream_t passed as void*, NULL = the
 *     legacy default stream) and the call returns.
 *   - Matrices are row-major with a leading dimension in ELEMENTS.
 *   - Functions are re-entrant per stream. One-time kernel attribute set-up is guarded
 *     internally.
 *
 * Each entry point names the part of the reference (stashuk-olek/deuteron, paths relative
 * to that project) whose emitted kernel it replaces.
 */
#ifndef DEUTERON_B200_H
#define DEUTERON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DTN_OK 0
#define DTN_ERR_INVALID 1   /* bad argument (null pointer, negative size, bad enum, misalignment) */
#define DTN_ERR_CUDA 2      /* a CUDA runtime/driver call failed; see dtn_last_error */
#define DTN_ERR_WORKSPACE 3 /* workspace missing or too small */
#define DTN_ERR_UNSUPPORTED 4 /* shape outside what the kernels implement */
#define DTN_ERR_DEVICE 5    /* a kernel reported a bounded wait that ran out */

/* contraction_precision of compiler/options.py:5-28 */
#define DTN_GEMM_F32 0
#define DTN_GEMM_TF32X3 1
#define DTN_GEMM_BF16X3 2
/* FP32 multiply-adds whose k range may be cut into partial sums that are added in a fixed order: the arithmetic of
 * the reference's split-K kernels (partial products added into a zeroed output, compiler/passes/gridfold.py:23-129),
 * whose k order is not the sequential one either. Same result on every run. */
#define DTN_GEMM_F32_SPLITK 3

/* reduction operator of dtn_row_reduce_f32 */
#define DTN_REDUCE_SUM 0
#define DTN_REDUCE_MAX 1
#define DTN_REDUCE_SUMSQ 2
#define DTN_REDUCE_SOFTMAX 3 /* dtn_row_fused only: row maximum and the sum of exp(x - maximum) */

/* kind of an extra input of dtn_row_fused */
#define DTN_ROW_INPUT_SCALAR 0    /* one-element f32 buffer, broadcast (constants arrive this way) */
#define DTN_ROW_INPUT_COLUMNS 1   /* f32[cols], indexed by the column (a weight vector) */
#define DTN_ROW_INPUT_IMMEDIATE 2 /* a literal of the IR; the value is taken from input_immediate */

/* storage type of attention operands */
#define DTN_STORAGE_F32 0
#define DTN_STORAGE_F16 1

/* binary / unary elementwise operators (compiler/codegen/lower.py:258-291) */
#define DTN_EW_ADD 0
#define DTN_EW_SUB 1
#define DTN_EW_MUL 2
#define DTN_EW_DIV 3
#define DTN_EW_MAX 4
#define DTN_EW_MIN 5
#define DTN_EW_RELU 6
#define DTN_EW_EXP 7
#define DTN_EW_SQRT 8
#define DTN_EW_RSQRT 9
#define DTN_EW_RCP 10
#define DTN_EW_NEG 11
#define DTN_EW_ABS 12
#define DTN_EW_COPY 13

/* Library version: major*10000 + minor*100 + patch. No reference counterpart
 * (the reference reports compiler/_version.py). */
int dtn_version(void);

/* Copies the calling thread's last error text (NUL terminated, truncated to n) into buf.
 * Mirrors the name+string that benchmark.py:46-52 attaches to CudaError. */
int dtn_last_error(char* buf, size_t n);

/* Reads and clears the device-side status word that kernels with bounded waits write
 * when a wait runs out. This call synchronises `stream`. *status_out = 0 when clean.
 * No reference counterpart (its kernels have no device-side waits on async units). */
int dtn_device_status(int* status_out /* host */, void* stream);

/* What the kernels of a call cost, for result records that carry those fields (benchmark.py:218-220 of the
 * reference reads them from its one PTX entry with cuFuncGetAttribute). dtn_capture_begin puts `stream` (not the
 * default stream) into capture; the caller then makes the library calls it wants described, which are recorded, not
 * run; dtn_capture_end ends the capture and reports, over the kernels recorded: how many, the largest register count
 * per thread, the largest static and the largest dynamic shared-memory size. Any output pointer may be NULL. */
int dtn_capture_begin(void* stream);
int dtn_capture_end(void* stream, int* kernels_out /* host */, int* max_registers_out /* host */,
                    int* max_static_smem_out /* host */, int* max_dynamic_smem_out /* host */);

/* Exercises the bounded-wait reporting path without any fault: one CTA waits, for at most
 * `budget_cycles` clock cycles, on a barrier that nothing completes, then records status 0x7100 in
 * the device status word and returns. dtn_device_status then reports it. No reference counterpart. */
int dtn_selftest_wait_timeout(long long budget_cycles, void* stream);

/* out[i] = x[i] + y[i], i < n.  Replaces the elementwise kernel emitted by
 * Lowering.tile / Load / Write (compiler/codegen/lower.py:434-495, 600-638) after
 * vectorize_elementwise (compiler/passes/vectorize.py:160-178) for
 * examples/vector_add/vector_add.ir.json. Bit-exact IEEE add. Any 4-byte aligned pointers. */
int dtn_add_f32(const float* x, const float* y, float* out, int64_t n, void* stream);

/* out[i] = op(x[i], y[i]) (binary ops) or op(x[i]) (unary ops, y ignored, may be NULL).
 * Operator table of Lowering.arithmetic (compiler/codegen/lower.py:258-291). exp uses
 * ex2.approx(x*log2(e)) and rcp/rsqrt the approximate forms, as approximate_math=True does. */
int dtn_elementwise_f32(int op, const float* x, const float* y, float* out, int64_t n, void* stream);

/* A chain of elementwise operators over f16 / f32 buffers in one pass: out[i] = program(inputs[..][i]).
 * Replaces the kernels the reference emits for Load / Assign... / Write tiles with more than one
 * operator, among them the f16 storage "affine" and "cancellation" kernels of
 * examples/f16_storage.py:36-54 (typing rules compiler/storage.py:27-58: arithmetic only in explicit
 * FP32, conversion at the load and at the store, Lowering.convert compiler/codegen/lower.py:249-256).
 *   inputs[k] (host array of n_inputs device pointers) fills register k: f16 (input_f16[k] = 1) or
 *   f32, a buffer of n elements or, with input_scalar[k] = 1, one element that is broadcast.
 *   Instruction j computes register dsts[j] = ops[j](register as[j], register bs[j]) (DTN_EW_* codes,
 *   unary operators ignore bs[j]); 8 registers, at most 24 instructions, each operator rounds once in
 *   FP32 (no fused multiply-add). Register out_reg is stored to out[i] as f32, or narrowed to f16
 *   (round-to-nearest-even) when out_f16 = 1. ops/dsts/as/bs/input_f16/input_scalar are host arrays.
 * Pointers need only their natural alignment. */
int dtn_elementwise_program(const unsigned char* ops, const unsigned char* dsts, const unsigned char* as,
                            const unsigned char* bs, int n_instr, const void* const* inputs,
                            const unsigned char* input_f16, const unsigned char* input_scalar,
                            int n_inputs, int out_reg, void* out, int out_f16, int64_t n, void* stream);

/* f16 storage kernels (compiler/storage.py:5-59, Lowering.convert compiler/codegen/lower.py:249-256,
 * shapes of examples/f16_storage.py:19-60). f16 values travel as uint16_t bit patterns.
 *   copy  : bit-preserving 16-bit move
 *   widen : exact f16 -> f32
 *   narrow: f32 -> f16 round-to-nearest-even, overflow to +-inf, subnormals kept, NaN -> NaN
 * Pointers need only their natural alignment (2 bytes for f16, 4 for f32), like the
 * scalar-aligned accesses of compiler/codegen/lower.py:604,623. */
int dtn_f16_copy(const uint16_t* src, uint16_t* dst, int64_t n, void* stream);
int dtn_f16_widen(const uint16_t* src, float* dst, int64_t n, void* stream);
int dtn_f16_narrow(const float* src, uint16_t* dst, int64_t n, void* stream);

/* out[r] = reduce_op over x[r, 0..cols) for r < rows; x has leading dimension ldx.
 * Replaces the coalesced reduction of striped_reduction (compiler/transforms.py:62-95),
 * Lowering.loop / register_reduction (compiler/codegen/lower.py:293-327, 348-421) and the
 * warp-shuffle + tree tail (compiler/codegen/lower.py:517-569). SUM and SUMSQ are
 * reassociated FP32 sums; MAX is the NaN-suppressing maxnum of lower.py:275-278 with
 * identity -inf. */
int dtn_row_reduce_f32(int op, const float* x, float* out, int64_t rows, int64_t cols,
                       int64_t ldx, void* stream);

/* Row reduction, a scalar stage and an elementwise stage over the same row in one launch:
 * row softmax, RMS norm, L2 norm, mean. Replaces the kernels the reference builds from a reduction
 * loop, a shuffle/tree tail and a consumer loop with load forwarding
 * (compiler/passes/regforward.py:150-269) and with the softmax normaliser
 * (compiler/passes/hybrid_normalizer.py:45-183).
 *   reduce_op: DTN_REDUCE_SUM / SUMSQ / MAX / SOFTMAX over x[r, 0..cols), leading dimension ldx.
 *   Program registers (12): 0 = reduced value, 1 = sum of exp(x - max) (SOFTMAX, else 0),
 *   2 = the row element (elementwise stage), 3 + i = extra input i, the rest are temporaries.
 *   Instructions [0, n_scalar_instr) run once per row, [n_scalar_instr, n_instr) once per element;
 *   instruction j is dsts[j] = ops[j](as[j], bs[j]) with DTN_EW_* codes. At most 32 instructions
 *   and 5 extra inputs.
 *   ldo > 0: out[r, c] = register out_reg after the elementwise stage. ldo == 0: out[r] = register
 *   out_reg after the scalar stage (n_scalar_instr must equal n_instr).
 * exp is ex2.approx(x * log2 e), sqrt/rsqrt/reciprocal/divide are the approximate instructions, as in
 * the reference's default approximate_math lowering (compiler/codegen/lower.py:259-289,
 * compiler/ptx.py:41). Rows of up to 8192 aligned values are read from memory once. */
int dtn_row_fused(int reduce_op, const float* x, int64_t rows, int64_t cols, int64_t ldx,
                  const void* const* inputs, const unsigned char* input_kind,
                  const float* input_immediate, int n_inputs, const unsigned char* ops,
                  const unsigned char* dsts, const unsigned char* as, const unsigned char* bs,
                  int n_scalar_instr, int n_instr, int out_reg, float* out, int64_t ldo, void* stream);

/* Bytes of scratch dtn_gemm_x3 needs for (mode, M, N, K): the bf16 (or tf32) high and
 * residual planes of A and of B transposed. 0 for DTN_GEMM_F32. */
int dtn_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, size_t* bytes_out /* host */);

/* C[M,N] = A[M,K] * B[K,N], FP32 in / FP32 out / FP32 accumulate, row-major.
 *   DTN_GEMM_BF16X3: each operand v is split hi = bf16_rn(v), lo = bf16_rn(v - hi) and the
 *     products lo_A*hi_B, hi_A*lo_B, hi_A*hi_B are accumulated in that order per k-step
 *     (TensorEmitter.bf16 / packed_store / _emit_packed, compiler/codegen/tensor.py:55-64,
 *     104-119, 121-190; stage_register_loads, compiler/passes/regstage.py:70-245).
 *   DTN_GEMM_TF32X3: hi = tf32_rna(v), lo = tf32_rna(v - hi), same three products
 *     (compiler/codegen/tensor.py:50-53, 192-245).
 *   DTN_GEMM_F32: plain FP32 FMA, k accumulated in sequence (generic Lowering.body,
 *     compiler/codegen/lower.py:600-653); DTN_GEMM_F32_SPLITK: the same with partial sums over slices of k.
 * The result store replaces TensorEmitter._store (compiler/codegen/tensor.py:255-267).
 * `workspace` must be 1024-byte aligned and at least dtn_gemm_workspace_bytes large for the
 * x3 modes (ignored for F32). A column block of B / C is addressed by offsetting the
 * pointers and keeping ldb / ldc. */
int dtn_gemm_x3(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N,
                int64_t K, int64_t lda, int64_t ldb, int64_t ldc, void* workspace,
                size_t workspace_bytes, void* stream);

/* dtn_gemm_x3 in separately launchable parts, so that a caller can time them apart or reuse
 * operand planes between calls. `phase` is a mask: 1 = split the operands into the workspace,
 * 2 = run the product kernel on the planes in the workspace (3 = both, what dtn_gemm_x3 does);
 * with 4 the A planes already in the workspace are kept (A is not split again), with 8 the B
 * planes are kept. The B planes sit at the start of the workspace, at a place that depends on
 * (mode, N, K) only, and the A planes after them: a caller that walks row blocks of A (of any
 * heights) against one B splits B once (1|4: only B is split) and passes 3|8 for every block,
 * with the same workspace pointer. Kept A planes are valid only for an unchanged (mode, M, N, K).
 * With 4 or 8 set the call always runs the split kernels and the tensor-memory product kernel,
 * never the single-kernel forms (which write no planes). No reference counterpart (the
 * reference splits inside its single kernel). */
int dtn_gemm_x3_phase(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N,
                      int64_t K, int64_t lda, int64_t ldb, int64_t ldc, void* workspace,
                      size_t workspace_bytes, int phase, void* stream);

/* The compensated GEMM for callers that must not allocate device memory. It has no counterpart in
 * the reference; it exists for hosts that cannot give dtn_gemm_x3 a workspace: programs that
 * handed all device memory to their own pool at start-up and forbid cudaMalloc afterwards (an
 * inference server's arena, a plugin sandbox), and latency-critical loops that cannot afford the
 * device-wide synchronisation a cudaMalloc or cudaFree implies. Same arithmetic as
 * dtn_gemm_x3(mode, ...) for DTN_GEMM_BF16X3 and DTN_GEMM_TF32X3, always through the split
 * kernels and the tensor-memory product kernel: bit-identical to dtn_gemm_x3 whenever that call
 * takes the same path (tile variants 1, 2, 3, 5; the automatic choice above about 520^3
 * multiply-adds and more than 16 rows). Where dtn_gemm_x3 picks its single-kernel forms (small or
 * skinny products, variants 4 and 6) the two agree to the tolerance of the mode, not bit for bit
 * (the k order of the accumulation differs); variants 4 and 6 count as "automatic" here. The
 * operand planes go to a fixed 32 MiB array that is part of the library image (every GPU that
 * loads the library holds those 32 MiB until the process exits). This function calls no
 * cudaMalloc, cudaFree or any other allocating routine. K = 0 zero-fills C.
 *   - Limit: the planes of (mode, M, N, K) — dtn_gemm_workspace_bytes tells how many bytes — must
 *     fit 32 MiB (bf16x3: 2048^3; tf32x3: about 1448^3). Larger problems are rejected with
 *     DTN_ERR_WORKSPACE and a message that names both sizes.
 *   - The first call on a device looks up the array's device address (with that device current).
 *     Make that first call outside any stream capture.
 *   - All calls on a device share the one array. Calls that can overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it: serialise them. Nothing in the
 *     array needs clearing between calls; every byte that is read is rewritten first.
 *   - A bounded wait that runs out inside this variant is recorded in a status word of its own
 *     (also part of the library image), read with dtn_gemm_x3_static_status. */
int dtn_gemm_x3_static(int mode, const float* A, const float* B, float* C, int64_t M, int64_t N,
                       int64_t K, int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* Reads and clears the status word of dtn_gemm_x3_static on the current device: 0 when every wait
 * of its kernels completed, else the code of the wait that ran out (the result is then
 * incomplete). Synchronises `stream`; allocates nothing. No counterpart in the reference. */
int dtn_gemm_x3_static_status(int* status_out /* host */, void* stream);

/* Copies the block src[rows, cols] (row-major FP32, leading dimension lds) to the same extent at each of the n_dst
 * (at most 7) destination pointers, all with leading dimension ldd: the block is read once and written n_dst times,
 * 16 bytes per thread when every pointer is 16-byte aligned and lds, ldd, cols are multiples of 4. The destinations
 * may be peer-mapped memory of other GPUs: this is the exchange step of a column-sharded GEMM whose full result is
 * wanted on every GPU (a rank pushes its finished rows into the peers' copies while it multiplies the rest).
 * `dsts` is a host array. No reference counterpart (the reference runs one GPU per problem,
 * benchmark.py:546-551). */
int dtn_push_block(const float* src, int64_t lds, float* const* dsts, int n_dst, int64_t ldd,
                   int64_t rows, int64_t cols, void* stream);

/* The tile schedule the CTA-pair GEMM kernel uses for an M x N output on `pairs` CTA pairs (a B200 has 74): host
 * arithmetic only, no GPU needed. The kernel walks `*rounds_out` rounds; in round j pair w multiplies the tile
 * entries_out[j * pairs + w] = band | (first column / 32) << 12 | (width / 32) << 24 (band = 256 rows; 0 = nothing
 * in that round). Bands are cut into pieces of 64..256 columns so that the pairs finish together: *longest_out is the
 * largest sum of (width + fixed cost) over the pairs, *longest_uniform_out the same for plain 256-wide tiles.
 * *rounds_out = 0 means the kernel keeps the plain walk (the cut would save under 3 %, or the table would not fit).
 * Tile width does not change any output bit. entries_out may be NULL. No reference counterpart (the reference's
 * schedule is one 32x64 tile per CTA, compiler/passes/contraction.py:135-213). */
int dtn_gemm_tile_schedule(int64_t M, int64_t N, int pairs, uint32_t* entries_out /* host */, int capacity,
                           int* rounds_out /* host */, double* longest_out /* host */,
                           double* longest_uniform_out /* host */);

/* Copies `height` rows of `width_bytes` each between host and device memory whose rows lie `src_pitch` / `dst_pitch`
 * bytes apart (a column block of a row-major matrix): one cudaMemcpy2DAsync on `stream`, host to device when
 * to_device is non-zero, else device to host. The host runner uses it to feed B and return C by column blocks
 * (the copies the reference's runner makes whole, benchmark.py:225-235,269-274). */
int dtn_copy_block(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t height, int to_device,
                   void* stream);

/* How the streamed kernel for at most 16 rows (variant 10) cuts a product among `workers` CTAs: host arithmetic only.
 * Work units are 64 k-rows x 128 columns of B, numbered column block by column block with k fastest; CTA w takes units
 * [unit_begin_out[w], unit_begin_out[w + 1]) (workers + 1 entries). first_out[c] .. last_out[c] are the CTAs that
 * contribute partial sums to column block c (ceil(N / 128) entries each); they are added in that order. Any output
 * pointer may be NULL. 1 <= workers <= number of units. No reference counterpart. */
int dtn_gemm_skinny_plan(int64_t N, int64_t K, int workers, int64_t* unit_begin_out /* host */, int* first_out /* host */,
                         int* last_out /* host */);

/* Selects the tensor-core GEMM variant for the calling host thread (other threads keep their own
 * selection, initially 0; for experiments and tests):
 *   0 = automatic, 1 = one-CTA 128x128 tile, 2 = one-CTA 128x256 tile, 3 = two-CTA 256x256 tile,
 *   4 = the single-kernel path for small problems (operand split inside the kernel, warp-level
 *   mma.sync products, no workspace; what automatic picks up to about 520^3 multiply-adds and for
 *   at most 16 rows), 5 = one-CTA 128x64 tile (automatic when 128x128 tiles would occupy at most
 *   half of the SMs), 6 = one tcgen05 kernel with the operand split in its producer warps (no
 *   workspace, one launch; bf16x3 with 16-byte aligned A and B, lda and ldb multiples of 4, N and
 *   K multiples of 8, else DTN_ERR_UNSUPPORTED), 7 = the stream kernel: two-CTA tiles 256 rows tall from the
 *   schedule of dtn_gemm_tile_schedule, with the split of A running inside the kernel beside the products (what
 *   automatic picks where it picked 3 before; 3 remains as the plain two-kernel form; 8 and 9 pin where the operand
 *   splits run), 10 = the streamed kernel for at most 16 rows wherever it applies (B brought in once by TMA in equal
 *   shares per SM, partial sums of a column block added in a fixed order through the workspace; needs 16-byte
 *   aligned A and B with lda and ldb multiples of 4, else DTN_ERR_UNSUPPORTED; what automatic picks for at most 16
 *   rows once B has 12 Mi elements).
 * No reference counterpart. */
int dtn_gemm_set_variant(int variant);

/* Single-head attention in the reference's example layout (examples/attention.py:59-66):
 * q[rows,depth], kt[depth,keys], v[keys,cols], out[rows,cols], all FP32 row-major.
 * out = softmax(q*kt*scale) * v with the staged recurrence of RecurrenceEmitter.emit
 * (compiler/passes/recurrence.py:609-706): scores, warp max, ex2.approx((s-m)*log2e),
 * warp sum, probability*value pass, reciprocal suffix (compiler/codegen/lower.py:264-270). */
int dtn_attention_f32(const float* q, const float* kt, const float* v, float* out,
                      int64_t rows, int64_t keys, int64_t depth, int64_t cols, float scale,
                      void* stream);

/* Grouped-query attention forward, non-causal.
 * q[B,Hq,S,D], k[B,Hkv,S,D], v[B,Hkv,S,D] in `storage` (f16 bit patterns or f32),
 * out[B,Hq,S,D] FP32. Query head h reads kv head h / (Hq/Hkv). FP32 compute with the online
 * form of the recurrence above (stage_recurrences, compiler/passes/recurrence.py:47-388).
 * `group_begin`/`group_end` select a range of the B*Hkv (batch, kv-head) groups, so that a
 * rank of a multi-GPU job computes only its groups; pass 0 and B*Hkv for all. */
int dtn_gqa_fwd(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq,
                int64_t Hkv, int64_t S, int64_t D, float scale, int storage,
                int64_t group_begin, int64_t group_end, void* stream);

/* Selects the attention kernel for the calling host thread: 0 = automatic, 1 = FP32 CUDA-core kernel,
 * 2 = tensor-core kernel (f16 storage, D = 128, S a multiple of 256), 3 = the same with two
 * softmax warpgroups per query tile, 4 and 5 = the CTA-pair form of 2 and 3 (S a multiple of 512; same results,
 * measured slower, kept for comparison), 6 = variant 3's shape with all sixteen softmax warps serving one tile at a
 * time (measured slower too), 7 = variant 3 with half of a thread's scores kept in registers between the maximum and
 * the probabilities and the output written by TMA stores: the automatic choice for f16 storage, D = 128 and any
 * S >= 256 (keys past the end of a sequence are masked, rows past it are neither read nor written: the tensor maps
 * are per head). Variants 3 and 7 give the same bits.
 * No reference counterpart. */
int dtn_gqa_set_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif /* DEUTERON_B200_H */
