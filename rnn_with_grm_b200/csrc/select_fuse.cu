// Selection half of the fused retrieval when the candidates have already been applied to the query.
//
// With per-token routing every token of a segment chooses among the same few archived matrices, so
// the caller applies the query to all of them with one batched GEMM (states[b,q,s,:] = M[b,s] q[b,q])
// and what is left of RetrievedStateFusion (grm/core/aggregator.py:104-105, 116-118) is, per token:
// pick R of the S candidate states, weight them by the gates, add the online state, LayerNorm.
// One warp per token; the row stays in registers between the sum and the normalisation.
#include "common.cuh"

namespace grmx {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kMaxPerLane = 32;   // register path covers H <= 1024
constexpr int kMaxRoutes = 32;

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
__device__ __forceinline__ void store_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
select_fuse_kernel(const T* __restrict__ states, const int64_t* __restrict__ indices,
                   const float* __restrict__ gates, const T* __restrict__ online,
                   const float* __restrict__ ln_weight, const float* __restrict__ ln_bias, float ln_eps,
                   T* __restrict__ out, int64_t BQ, int S, int R, int H, int mode,
                   uint32_t* __restrict__ error_word) {
  const int lane = threadIdx.x & 31;
  const int64_t bq = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (bq >= BQ) return;   // whole warps leave together; no CTA barrier below

  // this token's routes: lane r holds route r
  int64_t my_idx = -1;
  float my_gate = 0.0f;
  if (lane < R) {
    my_idx = indices[bq * R + lane];
    if (my_idx >= S || my_idx < -1) {
      if (error_word != nullptr) atomicOr(error_word, kErrGatherIndex);
      my_idx = -1;
    }
    my_gate = my_idx >= 0 ? gates[bq * R + lane] : 0.0f;
  }
  const bool live = __ballot_sync(0xffffffffu, my_idx >= 0) != 0u;
  const T* cand = states + bq * (int64_t)S * H;
  const bool fuse = mode == GRMX_FUSE_RESIDUAL_LN;

  float x[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) x[i] = 0.0f;
  for (int r = 0; r < R; ++r) {                             // gate-weighted sum in route order
    // every lane takes part in the shuffles, whatever part of the row it owns
    const int64_t idx = __shfl_sync(0xffffffffu, my_idx, r);
    const float gate = __shfl_sync(0xffffffffu, my_gate, r);
    if (idx < 0) continue;                                   // the same for all lanes
    const T* row = cand + idx * H;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int h = lane + 32 * i;
      if (h < H) x[i] = fmaf(gate, load_as_float(row + h), x[i]);
    }
  }
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int h = lane + 32 * i;
    if (fuse && h < H) x[i] += load_as_float(online + bq * H + h);
    sum += x[i];
  }
  if (!fuse || !live) {
    // the contribution alone, or (nothing archived for this token) the online state untouched
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int h = lane + 32 * i;
      if (h < H) store_from_float(out + bq * H + h, x[i]);
    }
    return;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / (float)H;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int h = lane + 32 * i;
    if (h < H) {
      const float d = x[i] - mean;
      sq = fmaf(d, d, sq);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / (float)H + ln_eps);
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int h = lane + 32 * i;
    if (h < H) {
      float y = (x[i] - mean) * rstd;
      if (ln_weight != nullptr) y *= ln_weight[h];
      if (ln_bias != nullptr) y += ln_bias[h];
      store_from_float(out + bq * H + h, y);
    }
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_select_fuse(const void* states, const int64_t* indices, const float* gates,
                                const void* online, const float* ln_weight, const float* ln_bias,
                                float ln_eps, void* out, int64_t B, int64_t Q, int64_t S, int64_t R,
                                int64_t H, int dtype, int mode, void* stream) {
  using namespace grmx;
  const char* who = "grmx_select_fuse";
  GRMX_REQUIRE(B >= 0 && Q >= 0 && S >= 0 && R >= 0 && H >= 0, "%s: negative size", who);
  GRMX_REQUIRE(mode == GRMX_FUSE_CONTRIB || mode == GRMX_FUSE_RESIDUAL_LN, "%s: mode must be contrib or residual_ln", who);
  GRMX_REQUIRE(dtype == GRMX_F32 || dtype == GRMX_BF16, "%s: dtype must be f32 or bf16", who);
  GRMX_REQUIRE(R <= kMaxRoutes, "%s: R %lld exceeds %d routes", who, (long long)R, kMaxRoutes);
  GRMX_REQUIRE(H <= 32 * kMaxPerLane, "%s: H %lld exceeds %d", who, (long long)H, 32 * kMaxPerLane);
  GRMX_REQUIRE(S <= 0x7fffffffLL, "%s: S too large", who);
  if (B * Q * H == 0) return GRMX_OK;
  GRMX_REQUIRE(out != nullptr, "%s: out is NULL", who);
  GRMX_REQUIRE(R == 0 || (indices && gates), "%s: NULL indices or gates", who);
  GRMX_REQUIRE(R == 0 || S == 0 || states, "%s: NULL states", who);
  GRMX_REQUIRE(mode != GRMX_FUSE_RESIDUAL_LN || online, "%s: NULL online state", who);
  const int64_t BQ = B * Q;
  const int64_t blocks = (BQ + kWarpsPerCta - 1) / kWarpsPerCta;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "%s: grid too large", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* err = device_error_word_ptr();
  if (dtype == GRMX_F32) {
    select_fuse_kernel<float><<<static_cast<unsigned>(blocks), kWarpsPerCta * 32, 0, s>>>(
        static_cast<const float*>(states), indices, gates, static_cast<const float*>(online), ln_weight, ln_bias,
        ln_eps, static_cast<float*>(out), BQ, (int)S, (int)R, (int)H, mode, err);
  } else {
    select_fuse_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), kWarpsPerCta * 32, 0, s>>>(
        static_cast<const __nv_bfloat16*>(states), indices, gates, static_cast<const __nv_bfloat16*>(online),
        ln_weight, ln_bias, ln_eps, static_cast<__nv_bfloat16*>(out), BQ, (int)S, (int)R, (int)H, mode, err);
  }
  return check_launch("select_fuse");
}
