// L2-normalisation of the key / query projections in one pass: out[n,:] = x[n,:] / max(||x[n,:]||, eps),
// optionally rounding fp32 input to bf16 on the way out (the form the tensor-core scan reads).
// Replaces the three passes of F.normalize (norm, clamp, divide) at grm/core/paper_grm.py:491-493.
// A group of G lanes owns a row and keeps it in registers between the sum of squares and the scaling;
// 16-byte loads; the sum is fp32 whatever the input type.
#include "common.cuh"

namespace grmx {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxPieces = 4;   // 16-byte pieces per lane: rows up to 32 * 4 * 16 bytes

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float (&out)[16 / sizeof(T)]) {
  if constexpr (sizeof(T) == 4) {
    out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
    out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] = __uint_as_float(w[j] << 16);
      out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
}

template <typename TOut, int VEC>
__device__ __forceinline__ void store_scaled(TOut* p, const float (&x)[VEC], float scale) {
  if constexpr (sizeof(TOut) == 4) {
    static_assert(VEC == 4, "fp32 out comes from fp32 in");
    *reinterpret_cast<float4*>(p) = make_float4(x[0] * scale, x[1] * scale, x[2] * scale, x[3] * scale);
  } else {
    uint32_t w[VEC / 2];
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(x[2 * j] * scale, x[2 * j + 1] * scale);
      w[j] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    if constexpr (VEC == 8) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    else *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  }
}

// G lanes per row (a power of two), `pieces` 16-byte pieces per row
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kThreads)
normalize_rows_kernel(const TIn* __restrict__ x, TOut* __restrict__ out, int64_t N, int K, int pieces, int G,
                      float eps) {
  constexpr int VEC = 16 / sizeof(TIn);
  const int lane = threadIdx.x & 31;
  const int in_group = lane & (G - 1);
  const int64_t row = ((int64_t)blockIdx.x * kThreads + threadIdx.x) / G;
  const bool live = row < N;
  const TIn* src = x + (live ? row : 0) * (int64_t)K;
  uint4 raw[kMaxPieces];
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const int piece = in_group + i * G;
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (live && piece < pieces) raw[i] = __ldg(reinterpret_cast<const uint4*>(src) + piece);
    float v[VEC];
    unpack16<TIn>(raw[i], v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) sq = fmaf(v[j], v[j], sq);
  }
  // every lane of the warp takes part; the exchange stays inside the group of G lanes
  for (int o = G >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float scale = 1.0f / fmaxf(sqrtf(sq), eps);
  if (!live) return;
  TOut* dst = out + row * (int64_t)K;
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const int piece = in_group + i * G;
    if (piece < pieces) {
      float v[VEC];
      unpack16<TIn>(raw[i], v);
      store_scaled<TOut, VEC>(dst + piece * VEC, v, scale);
    }
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_normalize_rows(const void* x, void* out, int64_t N, int64_t K, float eps, int in_dtype,
                                   int out_dtype, void* stream) {
  using namespace grmx;
  const char* who = "grmx_normalize_rows";
  GRMX_REQUIRE(N >= 0 && K >= 0, "%s: negative size", who);
  const bool f32 = in_dtype == GRMX_F32 && out_dtype == GRMX_F32;
  const bool b16 = in_dtype == GRMX_BF16 && out_dtype == GRMX_BF16;
  const bool cast = in_dtype == GRMX_F32 && out_dtype == GRMX_BF16;
  GRMX_REQUIRE(f32 || b16 || cast, "%s: dtypes must be f32->f32, bf16->bf16 or f32->bf16", who);
  if (N * K == 0) return GRMX_OK;
  GRMX_REQUIRE(x && out, "%s: NULL pointer", who);
  const int per16 = in_dtype == GRMX_F32 ? 4 : 8;
  if (K % per16 != 0 || K / per16 > 32 * kMaxPieces ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: rows must be whole 16-byte pieces, at most %d of them, 16-byte aligned", who,
                32 * kMaxPieces);
  }
  const int pieces = static_cast<int>(K / per16);
  int G = 1;
  while (G < 32 && G < pieces) G <<= 1;
  const int64_t blocks = (N * G + kThreads - 1) / kThreads;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "%s: grid too large", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(blocks);
  const int k = static_cast<int>(K);
  if (f32) {
    normalize_rows_kernel<float, float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(out), N, k, pieces, G, eps);
  } else if (b16) {
    normalize_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), N, k, pieces, G, eps);
  } else {
    normalize_rows_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, s>>>(
        static_cast<const float*>(x), static_cast<__nv_bfloat16*>(out), N, k, pieces, G, eps);
  }
  return check_launch("normalize_rows");
}
