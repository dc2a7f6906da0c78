// out[b,j,:] = memories[b, indices[b,j], :]  -- a pure HBM copy.
//
// Each CTA moves one 16 KiB piece of one selected matrix: 256 threads, four
// 16-byte loads issued per thread before the first store.  The index is read
// once per thread (one cached word).  Rows whose size or alignment rules out
// 16-byte accesses fall back to 4- or 2-byte units.
// Semantics: grm/core/cuda_ops.py:265-284 (per-batch index_select).
#include "common.cuh"

namespace grmx {
namespace {

constexpr int kThreads = 256;
constexpr int kUnitsPerThread = 4;
constexpr int kUnitsPerCta = kThreads * kUnitsPerThread;

template <typename U>
__device__ __forceinline__ U zero_unit();
template <>
__device__ __forceinline__ uint4 zero_unit<uint4>() { return make_uint4(0, 0, 0, 0); }
template <>
__device__ __forceinline__ uint32_t zero_unit<uint32_t>() { return 0u; }
template <>
__device__ __forceinline__ uint16_t zero_unit<uint16_t>() { return 0; }

template <typename U>
__global__ void __launch_bounds__(kThreads)
batched_gather_kernel(const U* __restrict__ memories, const int64_t* __restrict__ indices,
                      U* __restrict__ out, int64_t S, int64_t J, int64_t row_units,
                      int64_t pieces_per_row, uint32_t* __restrict__ error_word) {
  const int64_t out_row = blockIdx.x / pieces_per_row;  // b*J + j
  const int64_t piece = blockIdx.x % pieces_per_row;
  const int64_t b = out_row / J;
  const int64_t seg = indices[out_row];
  const bool valid = seg >= 0 && seg < S;
  if (!valid && seg != -1 && threadIdx.x == 0 && piece == 0 && error_word != nullptr) {
    atomicOr(error_word, kErrGatherIndex);
  }
  const U* src = memories + (b * S + (valid ? seg : 0)) * row_units;
  U* dst = out + out_row * row_units;
  const int64_t u0 = piece * kUnitsPerCta + threadIdx.x;

  U v[kUnitsPerThread];
#pragma unroll
  for (int i = 0; i < kUnitsPerThread; ++i) {
    const int64_t u = u0 + (int64_t)i * kThreads;
    v[i] = (valid && u < row_units) ? __ldg(src + u) : zero_unit<U>();
  }
#pragma unroll
  for (int i = 0; i < kUnitsPerThread; ++i) {
    const int64_t u = u0 + (int64_t)i * kThreads;
    if (u < row_units) dst[u] = v[i];
  }
}

template <typename U>
int launch(const void* memories, const int64_t* indices, void* out, int64_t B, int64_t S, int64_t J,
           int64_t row_bytes, cudaStream_t stream) {
  const int64_t row_units = row_bytes / static_cast<int64_t>(sizeof(U));
  const int64_t pieces = (row_units + kUnitsPerCta - 1) / kUnitsPerCta;
  const int64_t blocks = B * J * pieces;
  if (blocks > 0x7fffffffLL) return fail(GRMX_ERR_UNSUPPORTED, "batched_gather: grid too large");
  batched_gather_kernel<U><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
      static_cast<const U*>(memories), indices, static_cast<U*>(out), S, J, row_units, pieces,
      device_error_word_ptr());
  return check_launch("batched_gather");
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_batched_gather(const void* memories, const int64_t* indices, void* out,
                                   int64_t B, int64_t S, int64_t J, int64_t row_elems,
                                   int elem_size, void* stream) {
  using namespace grmx;
  GRMX_REQUIRE(B >= 0 && S >= 0 && J >= 0 && row_elems >= 0, "grmx_batched_gather: negative size");
  GRMX_REQUIRE(elem_size == 2 || elem_size == 4, "grmx_batched_gather: elem_size must be 2 or 4");
  if (B * J * row_elems == 0) return GRMX_OK;
  GRMX_REQUIRE(indices && out, "grmx_batched_gather: NULL tensor pointer");
  GRMX_REQUIRE(S == 0 || memories != nullptr, "grmx_batched_gather: NULL memories");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = row_elems * elem_size;
  const uintptr_t align = reinterpret_cast<uintptr_t>(memories) | reinterpret_cast<uintptr_t>(out);
  if (row_bytes % 16 == 0 && (align & 15u) == 0) {
    return launch<uint4>(memories, indices, out, B, S, J, row_bytes, s);
  }
  if (row_bytes % 4 == 0 && (align & 3u) == 0) {
    return launch<uint32_t>(memories, indices, out, B, S, J, row_bytes, s);
  }
  return launch<uint16_t>(memories, indices, out, B, S, J, row_bytes, s);
}
