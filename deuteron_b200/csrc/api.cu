// Library-level entry points: version, error text, device status word.
#include <stdarg.h>
#include <stdlib.h>

#include <mutex>

#include "dtn_common.cuh"

namespace dtn {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

const char* get_error() { return g_error; }

// One status word per device, allocated the first time a kernel with bounded waits runs
// there. Kept for the life of the process.
static std::mutex g_status_mutex;
static int* g_status_words[64] = {nullptr};

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return nullptr;
    g_status_words[dev] = p;
  }
  return g_status_words[dev];
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace dtn

extern "C" {

int dtn_version(void) { return 100; /* 0.1.0 */ }

int dtn_last_error(char* buf, size_t n) {
  if (!buf || n == 0) return DTN_ERR_INVALID;
  strncpy(buf, dtn::get_error(), n - 1);
  buf[n - 1] = '\0';
  return DTN_OK;
}

int dtn_device_status(int* status_out, void* stream) {
  DTN_REQUIRE(status_out != nullptr, DTN_ERR_INVALID, "dtn_device_status: status_out is null");
  int* word = dtn::device_status_word();
  DTN_REQUIRE(word != nullptr, DTN_ERR_CUDA, "dtn_device_status: no status word on this device");
  cudaStream_t s = dtn::as_stream(stream);
  int host = 0;
  DTN_CUDA_CHECK(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  DTN_CUDA_CHECK(cudaStreamSynchronize(s));
  if (host != 0) DTN_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(int), s));
  *status_out = host;
  return DTN_OK;
}

int dtn_capture_begin(void* stream) {
  cudaStream_t s = dtn::as_stream(stream);
  DTN_REQUIRE(s != nullptr, DTN_ERR_INVALID, "dtn_capture_begin: a stream of its own is needed (not the default stream)");
  DTN_CUDA_CHECK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  return DTN_OK;
}

int dtn_capture_end(void* stream, int* kernels_out, int* max_registers_out, int* max_static_smem_out,
                    int* max_dynamic_smem_out) {
  cudaStream_t s = dtn::as_stream(stream);
  cudaGraph_t graph = nullptr;
  DTN_CUDA_CHECK(cudaStreamEndCapture(s, &graph));
  DTN_REQUIRE(graph != nullptr, DTN_ERR_CUDA, "dtn_capture_end: the capture produced no graph");
  size_t count = 0;
  cudaError_t err = cudaGraphGetNodes(graph, nullptr, &count);
  int kernels = 0, regs = 0, static_smem = 0, dynamic_smem = 0;
  if (err == cudaSuccess && count > 0) {
    cudaGraphNode_t* nodes = static_cast<cudaGraphNode_t*>(malloc(count * sizeof(cudaGraphNode_t)));
    if (nodes != nullptr && (err = cudaGraphGetNodes(graph, nodes, &count)) == cudaSuccess) {
      for (size_t i = 0; i < count && err == cudaSuccess; ++i) {
        cudaGraphNodeType type;
        if ((err = cudaGraphNodeGetType(nodes[i], &type)) != cudaSuccess || type != cudaGraphNodeTypeKernel) continue;
        cudaKernelNodeParams params = {};
        if ((err = cudaGraphKernelNodeGetParams(nodes[i], &params)) != cudaSuccess) break;
        cudaFuncAttributes attributes = {};
        if ((err = cudaFuncGetAttributes(&attributes, params.func)) != cudaSuccess) break;
        ++kernels;
        if (attributes.numRegs > regs) regs = attributes.numRegs;
        if ((int)attributes.sharedSizeBytes > static_smem) static_smem = (int)attributes.sharedSizeBytes;
        if ((int)params.sharedMemBytes > dynamic_smem) dynamic_smem = (int)params.sharedMemBytes;
      }
    }
    free(nodes);
  }
  cudaGraphDestroy(graph);
  if (err != cudaSuccess) {
    dtn::set_error("dtn_capture_end: %s (%s)", cudaGetErrorName(err), cudaGetErrorString(err));
    return DTN_ERR_CUDA;
  }
  if (kernels_out) *kernels_out = kernels;
  if (max_registers_out) *max_registers_out = regs;
  if (max_static_smem_out) *max_static_smem_out = static_smem;
  if (max_dynamic_smem_out) *max_dynamic_smem_out = dynamic_smem;
  return DTN_OK;
}

/* A block of `height` rows of `width_bytes` each between host and device memory with different row pitches (a column
 * block of a row-major matrix), asynchronous on `stream` when the host side is page-locked: one cudaMemcpy2DAsync. */
int dtn_copy_block(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t height, int to_device,
                   void* stream) {
  if (width_bytes == 0 || height == 0) return DTN_OK;
  DTN_REQUIRE(dst != nullptr && src != nullptr && dst_pitch >= width_bytes && src_pitch >= width_bytes, DTN_ERR_INVALID,
              "copy_block: null pointer or pitch below the row width");
  DTN_CUDA_CHECK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height,
                                   to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, dtn::as_stream(stream)));
  return DTN_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Self-test of the bounded-wait reporting path: a CTA waits on an mbarrier that nothing ever
// completes, with a small cycle budget; when the budget runs out it records a status code and
// returns normally, exactly as the tensor-core kernels do when one of their waits runs out.
// ---------------------------------------------------------------------------------------
namespace dtn {

__global__ void bounded_wait_selftest_kernel(long long budget_cycles, int* status) {
  __shared__ __align__(8) unsigned long long barrier;
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(&barrier));
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr) : "memory");
    const long long start = clock64();
    bool completed = false;
    while (!completed) {
      unsigned ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(addr)
          : "memory");
      completed = ok != 0;
      if (!completed && clock64() - start > budget_cycles) break;
    }
    if (!completed) atomicExch(status, 0x7100);
  }
}

}  // namespace dtn

extern "C" int dtn_selftest_wait_timeout(long long budget_cycles, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(budget_cycles > 0 && budget_cycles <= 2000000000LL, DTN_ERR_INVALID,
              "selftest: budget must be between 1 and 2e9 cycles");
  int* status = device_status_word();
  DTN_REQUIRE(status != nullptr, DTN_ERR_CUDA, "selftest: no status word on this device");
  bounded_wait_selftest_kernel<<<1, 32, 0, as_stream(stream)>>>(budget_cycles, status);
  DTN_LAUNCH_CHECK("bounded_wait_selftest_kernel");
  return DTN_OK;
}
