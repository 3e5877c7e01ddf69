// Host-side plumbing shared by the entry points: error text, device status word,
// launch counter, ABI version.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace nvllm {

static thread_local char tl_error[512] = "";
static std::atomic<int64_t> g_launches{0};

// One status word per device: the symbol is instantiated in every context that loads the
// module, and its address differs per device.
__device__ int g_status_word = 0;
constexpr int kMaxDevices = 64;
static int* g_status_addr[kMaxDevices] = {nullptr};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return code;
}

int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (!g_status_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_status_addr[dev] = static_cast<int*>(p);
  }
  return g_status_addr[dev];
}

int num_sms() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return 0;
  }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return 0;
    }
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* s = std::getenv("NVLLM_PDL");
    return s && s[0] == '1';
  }();
  return on;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return NVLLM_OK;
}

}  // namespace nvllm

extern "C" {

const char* nvllm_last_error(void) { return nvllm::tl_error; }

int nvllm_read_status(int32_t* host_out) {
  if (!host_out) return nvllm::fail(NVLLM_E_NULL, "nvllm_read_status: host_out is NULL");
  int* dev = nvllm::status_word();
  if (!dev) return nvllm::fail(NVLLM_E_NO_DEVICE, "nvllm_read_status: no CUDA device is usable");
  int32_t v = 0;
  cudaError_t e = cudaMemcpy(&v, dev, sizeof(v), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemset(dev, 0, sizeof(int));
  if (e != cudaSuccess) return nvllm::fail(NVLLM_E_CUDA, "nvllm_read_status: %s", cudaGetErrorString(e));
  *host_out = v;
  return NVLLM_OK;
}

int nvllm_abi_version(void) { return 2; }

int64_t nvllm_launch_count(void) { return nvllm::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
