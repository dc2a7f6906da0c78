// Host-side helpers shared by the tcgen05 kernels: the driver entry point for tensor-map
// encoding, a per-thread cache of encoded maps, the device check, the bounded-wait self-test
// and the rules that decide whether a call can take the tensor-core scan.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace tc {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    } else {
      cudaGetLastError();
    }
  });
  return fn;
}

namespace {

// Encoding a tensor map is a driver call of a few microseconds, and a scan needs four of them;
// callers that run the same buffers again and again (a segment loop, a serving step) would pay
// that on every call.  The last few encodings are kept per thread, keyed by everything that
// goes into them.
struct MapKey {
  const void* base;
  int64_t B, T, D;
  int kind;   // 0: load map (64 x 128 box, 128-byte swizzle), 1: store map (32 x 128 box, 64-byte swizzle)
  bool operator==(const MapKey& o) const {
    return base == o.base && B == o.B && T == o.T && D == o.D && kind == o.kind;
  }
};
constexpr int kMapCacheSlots = 16;
struct MapCache {
  MapKey keys[kMapCacheSlots];
  CUtensorMap maps[kMapCacheSlots];
  int used = 0;
  int next = 0;
};

bool encode_token_map(CUtensorMap* map, const MapKey& key) {
  thread_local MapCache cache;
  for (int i = 0; i < cache.used; ++i) {
    if (cache.keys[i] == key) {
      *map = cache.maps[i];
      return true;
    }
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(key.D), static_cast<cuuint64_t>(key.T),
                              static_cast<cuuint64_t>(key.B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(key.D) * 2, static_cast<cuuint64_t>(key.T) * key.D * 2};
  const cuuint32_t box[3] = {key.kind == 0 ? 64u : 32u, 128, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const bool ok =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(key.base), dims, strides, box, elem_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, key.kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
             key.kind == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  if (ok) {
    const int slot = cache.next;
    cache.keys[slot] = key;
    cache.maps[slot] = *map;
    cache.next = (slot + 1) % kMapCacheSlots;
    if (cache.used < kMapCacheSlots) ++cache.used;
  }
  return ok;
}

}  // namespace

bool make_token_map(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t D) {
  return encode_token_map(map, MapKey{base, B, T, D, 0});
}

bool make_token_half_map(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t D) {
  return encode_token_map(map, MapKey{base, B, T, D, 1});
}

namespace {

// Four warps wait on a barrier that nothing completes.  The first to run out of polls raises the
// abort flag, the others see it at their next check, and the CTA reports through the error word.
__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(uint32_t limit, uint32_t* error_word) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  mbar_wait(&bar, 0, &abort_flag, limit);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
}

}  // namespace

int launch_bounded_wait_selftest(uint32_t limit, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 128, 0, stream>>>(limit, device_error_word_ptr());
  return check_launch("bounded_wait_selftest");
}

bool device_is_sm100() {
  static int cached[64] = {0};   // 0 unknown, 1 yes, 2 no
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return false;
  if (cached[device] == 0) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    cached[device] = major == 10 ? 1 : 2;
  }
  return cached[device] == 1;
}

}  // namespace tc

using namespace tc;

bool scan_tcgen05_supported(const ScanParams& p, int io_dtype, int state_dtype, const char** why) {
  if (io_dtype != GRMX_BF16 || state_dtype != GRMX_F32) {
    *why = "needs bf16 tokens and an fp32 state";
    return false;
  }
  if (!scan_tcgen05_pipe_supported(p)) {
    *why = "d_k and d_v must be multiples of 64 (d_k <= 1024, d_v <= 4096)";
    return false;
  }
  if (p.T < 1) {
    *why = "no tokens";
    return false;
  }
  if (p.B > 0x7fffffffLL || p.T > 0x7fff0000LL) {
    *why = "B or T exceeds the tensor-map coordinate range";
    return false;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(p.keys) | reinterpret_cast<uintptr_t>(p.values) |
                          reinterpret_cast<uintptr_t>(p.queries) | reinterpret_cast<uintptr_t>(p.hidden_out) |
                          reinterpret_cast<uintptr_t>(p.memory_out);
  if (align & 15u) {
    *why = "tensors must be 16-byte aligned";
    return false;
  }
  if (!device_is_sm100()) {
    *why = "the current device is not sm_100";
    return false;
  }
  if (encode_tiled_fn() == nullptr) {
    *why = "cuTensorMapEncodeTiled is unavailable";
    return false;
  }
  *why = "";
  return true;
}

int launch_scan_tcgen05(const ScanParams& p, cudaStream_t stream) {
  if (scan_tcgen05_square_supported(p)) return launch_scan_tcgen05_square(p, stream);
  if (scan_tcgen05_wide_supported(p)) return launch_scan_tcgen05_wide(p, stream);
  return launch_scan_tcgen05_selfcut(p, stream);
}

}  // namespace grmx
