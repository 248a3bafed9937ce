// Tensor-core grouped-query attention (f16 storage, head_dim 128). Placeholder selection
// logic until the kernel lands: reports "not supported" so that dtn_gqa_fwd uses the FP32 kernel.
#include "dtn_common.cuh"

namespace dtn {

bool gqa_tc_supported(int64_t S, int64_t D, int storage) {
  (void)S; (void)D; (void)storage;
  return false;
}

int gqa_tc_launch(const void*, const void*, const void*, float*, int64_t, int64_t, int64_t, float, int64_t,
                  int64_t, cudaStream_t) {
  set_error("gqa: the tensor-core kernel is not built");
  return DTN_ERR_UNSUPPORTED;
}

}  // namespace dtn
