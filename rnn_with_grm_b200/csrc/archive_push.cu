// One segment-end state into its slot of the archive ring and, in the same pass, into the bf16 copy
// of the ring that the dense retrieval multiplies with (the state is read once instead of being
// converted again with every later segment that retrieves from it).
// Semantics: the append of grm/core/paper_grm.py:31-44, 721-725 on a preallocated device ring.
#include "common.cuh"

namespace grmx {
namespace {

constexpr int kThreads = 256;

template <int VEC>
__global__ void __launch_bounds__(kThreads)
archive_push_kernel(const float* __restrict__ memory, float* __restrict__ archive,
                    __nv_bfloat16* __restrict__ shadow, int64_t units, int64_t row_units, int64_t S, int64_t slot) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= units) return;
  const int64_t b = i / row_units;
  const int64_t dst = ((b * S + slot) * row_units + (i - b * row_units)) * VEC;
  if constexpr (VEC == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(memory) + i);
    *reinterpret_cast<float4*>(archive + dst) = v;
    if (shadow != nullptr) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(shadow + dst) = packed;
    }
  } else {
    const float v = __ldg(memory + i);
    archive[dst] = v;
    if (shadow != nullptr) shadow[dst] = __float2bfloat16_rn(v);
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_archive_push(const float* memory, float* archive, void* archive_bf16, int64_t B, int64_t S,
                                 int64_t slot, int64_t row_elems, void* stream) {
  using namespace grmx;
  const char* who = "grmx_archive_push";
  GRMX_REQUIRE(B >= 0 && S >= 0 && row_elems >= 0, "%s: negative size", who);
  GRMX_REQUIRE(slot >= 0 && slot < S, "%s: slot %lld outside [0, %lld)", who, (long long)slot, (long long)S);
  if (B * row_elems == 0) return GRMX_OK;
  GRMX_REQUIRE(memory && archive, "%s: NULL pointer", who);
  const uintptr_t bases = reinterpret_cast<uintptr_t>(memory) | reinterpret_cast<uintptr_t>(archive) |
                          (reinterpret_cast<uintptr_t>(archive_bf16) << 1);   // 8-byte stores into the bf16 ring
  const bool vec = row_elems % 4 == 0 && (bases & 15u) == 0;
  const int64_t row_units = vec ? row_elems / 4 : row_elems;
  const int64_t units = B * row_units;
  const int64_t blocks = (units + kThreads - 1) / kThreads;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "%s: grid too large", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* shadow = static_cast<__nv_bfloat16*>(archive_bf16);
  if (vec) {
    archive_push_kernel<4><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(memory, archive, shadow, units, row_units, S, slot);
  } else {
    archive_push_kernel<1><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(memory, archive, shadow, units, row_units, S, slot);
  }
  return check_launch("archive_push");
}
