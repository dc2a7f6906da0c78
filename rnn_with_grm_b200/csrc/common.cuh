// Shared helpers of the grmx kernels: error reporting, element-type traits,
// launch accounting.  Internal to the library; the public surface is grmx.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "grmx.h"

namespace grmx {

// ---- host-side error text (thread local, so concurrent callers do not mix) ----
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
void note_launch(int n = 1);

// Checks the launch status of the kernel just enqueued.
int check_launch(const char* what);

// Device error word (one per device, lives in the library image).
uint32_t* device_error_word_ptr();

#define GRMX_REQUIRE(cond, ...)                          \
  do {                                                   \
    if (!(cond)) return ::grmx::fail(GRMX_ERR_ARG, __VA_ARGS__); \
  } while (0)

// ---- element conversion ----
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

inline size_t dtype_size(int dtype) { return dtype == GRMX_F32 ? 4 : 2; }
inline bool dtype_valid(int dtype) {
  return dtype == GRMX_F32 || dtype == GRMX_BF16 || dtype == GRMX_F16;
}

constexpr uint32_t kErrGatherIndex = 1u;
constexpr uint32_t kErrBoundedWait = 2u;

}  // namespace grmx
