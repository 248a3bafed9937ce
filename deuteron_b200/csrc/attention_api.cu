// dtn_gqa_fwd: argument checks and kernel selection for grouped-query attention.
#include "dtn_common.cuh"

namespace dtn {

int gqa_f32_launch(const void* q, const void* k, const void* v, float* out, int64_t Hq, int64_t Hkv, int64_t S,
                   int64_t D, float scale, int storage, int64_t gb, int64_t ge, cudaStream_t s);
int gqa_tc_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                  int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s);
bool gqa_tc_supported(int64_t S, int64_t D, int storage);
bool gqa_tc_ragged_supported(int64_t S, int64_t D, int storage);
int gqa_tc_pair_launch(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                       int64_t S, float scale, int64_t gb, int64_t ge, int split, cudaStream_t s);
bool gqa_tc_pair_supported(int64_t S, int64_t D, int storage);

static thread_local int g_gqa_variant = 0;   // selection of dtn_gqa_set_variant, one value per host thread

}  // namespace dtn

extern "C" {

int dtn_gqa_set_variant(int variant) {
  DTN_REQUIRE(variant >= 0 && variant <= 7, DTN_ERR_INVALID, "gqa: variant must be 0..7");
  dtn::g_gqa_variant = variant;
  return DTN_OK;
}

int dtn_gqa_fwd(const void* q, const void* k, const void* v, float* out, int64_t B, int64_t Hq, int64_t Hkv,
                int64_t S, int64_t D, float scale, int storage, int64_t group_begin, int64_t group_end,
                void* stream) {
  using namespace dtn;
  DTN_REQUIRE(B >= 0 && Hq >= 0 && Hkv >= 0 && S >= 0 && D >= 0, DTN_ERR_INVALID, "gqa: negative extent");
  DTN_REQUIRE(storage == DTN_STORAGE_F16 || storage == DTN_STORAGE_F32, DTN_ERR_INVALID, "gqa: unknown storage %d",
              storage);
  if (B == 0 || Hq == 0 || S == 0 || D == 0) return DTN_OK;
  DTN_REQUIRE(Hkv > 0 && Hq % Hkv == 0, DTN_ERR_INVALID, "gqa: query heads must be a multiple of kv heads");
  DTN_REQUIRE(group_begin >= 0 && group_begin <= group_end && group_end <= B * Hkv, DTN_ERR_INVALID,
              "gqa: group range [%lld, %lld) outside [0, %lld]", (long long)group_begin, (long long)group_end,
              (long long)(B * Hkv));
  if (group_begin == group_end) return DTN_OK;
  DTN_REQUIRE(q && k && v && out, DTN_ERR_INVALID, "gqa: null pointer");
  DTN_REQUIRE(aligned_to(q, 16) && aligned_to(k, 16) && aligned_to(v, 16) && aligned_to(out, 16), DTN_ERR_INVALID,
              "gqa: tensors must be 16-byte aligned");
  DTN_REQUIRE(S < (1LL << 31), DTN_ERR_UNSUPPORTED, "gqa: sequence length must fit 31 bits");
  cudaStream_t s = as_stream(stream);
  int variant = g_gqa_variant;
  // Two softmax warpgroups per tile with the first half of a thread's scores kept in registers are the default, for
  // any sequence length from 256 up (it masks missing keys and clips missing rows; the other forms want multiples)
  // (4096 keys: 997 against 959 TFLOP/s for the form that reads the scores twice, 2048 keys: 890 against 847, 512
  // keys: equal; alternating runs in one process, identical output bits).
  if (variant == 0) variant = gqa_tc_ragged_supported(S, D, storage) ? 7 : 1;
  if (variant == 7) {   // two softmax warpgroups per tile, scores kept in registers between the two passes
    DTN_REQUIRE(gqa_tc_ragged_supported(S, D, storage), DTN_ERR_UNSUPPORTED,
                "gqa: the tensor-core kernel needs f16 storage, head_dim 128 and S of at least 256");
    return gqa_tc_launch(q, k, v, out, B, Hq, Hkv, S, scale, group_begin, group_end, 3, s);
  }
  if (variant == 6) {   // all sixteen softmax warps on one tile at a time
    DTN_REQUIRE(gqa_tc_supported(S, D, storage), DTN_ERR_UNSUPPORTED,
                "gqa: the tensor-core kernel needs f16 storage, head_dim 128 and S a multiple of 256");
    return gqa_tc_launch(q, k, v, out, B, Hq, Hkv, S, scale, group_begin, group_end, 4, s);
  }
  if (variant >= 4) {   // CTA pairs (4: one softmax warpgroup per tile, 5: two)
    DTN_REQUIRE(gqa_tc_pair_supported(S, D, storage), DTN_ERR_UNSUPPORTED,
                "gqa: the CTA-pair kernel needs f16 storage, head_dim 128 and S a multiple of 512");
    return gqa_tc_pair_launch(q, k, v, out, B, Hq, Hkv, S, scale, group_begin, group_end, variant == 5 ? 2 : 1, s);
  }
  if (variant >= 2) {
    DTN_REQUIRE(gqa_tc_supported(S, D, storage), DTN_ERR_UNSUPPORTED,
                "gqa: the tensor-core kernel needs f16 storage, head_dim 128 and S a multiple of 256");
    return gqa_tc_launch(q, k, v, out, B, Hq, Hkv, S, scale, group_begin, group_end, variant == 3 ? 2 : 1, s);
  }
  return gqa_f32_launch(q, k, v, out, Hq, Hkv, S, D, scale, storage, group_begin, group_end, s);
}

}  // extern "C"
