// Library-level pieces of the C ABI: version, error text, device query,
// launch counter and the per-device error word.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace grmx {

namespace {
thread_local char g_last_error[512] = {0};
std::atomic<int64_t> g_launches{0};

// Sticky error bits written by kernels (bad gather index, bounded wait expired).
__device__ uint32_t g_device_error_word = 0;

constexpr int kMaxDevices = 64;
uint32_t* g_error_word_ptr[kMaxDevices] = {nullptr};
std::mutex g_error_word_mutex;
}  // namespace

char* last_error_buffer() { return g_last_error; }

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
  va_end(args);
  return code;
}

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "%s: CUDA launch failed: %s", what, cudaGetErrorString(err));
  }
  note_launch();
  return GRMX_OK;
}

uint32_t* device_error_word_ptr() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_error_word_mutex);
  if (g_error_word_ptr[device] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_error_word) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_error_word_ptr[device] = static_cast<uint32_t*>(ptr);
  }
  return g_error_word_ptr[device];
}

}  // namespace grmx

extern "C" {

int grmx_version(void) { return 100; }

const char* grmx_last_error(void) { return grmx::last_error_buffer(); }

int64_t grmx_launch_count(void) { return grmx::g_launches.load(std::memory_order_relaxed); }

int grmx_query_device(int device, grmx_device_info* out) {
  if (out == nullptr) return grmx::fail(GRMX_ERR_ARG, "grmx_query_device: out is NULL");
  cudaDeviceProp prop;
  cudaError_t err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return grmx::fail(GRMX_ERR_DEVICE, "grmx_query_device: %s", cudaGetErrorString(err));
  }
  out->device = device;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  out->max_smem_per_block = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->has_tcgen05 = prop.major == 10 ? 1 : 0;
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  return GRMX_OK;
}

int grmx_device_error_word(uint32_t* out, void* stream) {
  if (out == nullptr) return grmx::fail(GRMX_ERR_ARG, "grmx_device_error_word: out is NULL");
  uint32_t* word = grmx::device_error_word_ptr();
  if (word == nullptr) return grmx::fail(GRMX_ERR_DEVICE, "grmx_device_error_word: no device error word");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(out, word, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    return grmx::fail(GRMX_ERR_LAUNCH, "grmx_device_error_word: %s", cudaGetErrorString(err));
  }
  return GRMX_OK;
}

int grmx_device_error_reset(void* stream) {
  uint32_t* word = grmx::device_error_word_ptr();
  if (word == nullptr) return grmx::fail(GRMX_ERR_DEVICE, "grmx_device_error_reset: no device error word");
  cudaError_t err = cudaMemsetAsync(word, 0, sizeof(uint32_t), static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    return grmx::fail(GRMX_ERR_LAUNCH, "grmx_device_error_reset: %s", cudaGetErrorString(err));
  }
  return GRMX_OK;
}

}  // extern "C"
