// Library-level entry points: version, error text, device status word.
#include <stdarg.h>

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

}  // extern "C"
