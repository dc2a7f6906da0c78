// Retrieval without the gathered tensor: for every (batch row, query) read the
// selected archive matrices once, apply the query, weight by the gates and,
// optionally, add the online state and layer-normalise.
//
// One CTA per query.  A group of G lanes owns a matrix row h and walks the R
// routes for it, so up to R independent 16-byte loads are in flight per lane
// and the gate-weighted sum over routes is accumulated in route order by one
// owner (deterministic).  Bytes moved per query: R*H*K*4 read, H*4 (or R*H*4)
// written -- the reference chain writes and re-reads the gathered R*H*K*4 too
// (grm/core/paper_grm.py:229-234,301-307).
#include "common.cuh"

namespace grmx {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxRoutes = 32;

template <int VEC>
__device__ __forceinline__ void load_row_chunk(const float* p, float (&out)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
    out[0] = __ldg(p);
  }
}

__device__ __forceinline__ float block_sum(float v, float* s_red) {
  // fixed-order reduction: warp shuffles, then warp 0 adds the 8 partials
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_red[warp] = v;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total += s_red[w];
  return total;
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
retrieve_fuse_kernel(const float* __restrict__ archive, const int64_t* __restrict__ indices,
                     const float* __restrict__ gates, const float* __restrict__ queries,
                     const float* __restrict__ online, const float* __restrict__ ln_weight,
                     const float* __restrict__ ln_bias, float ln_eps, float* __restrict__ out,
                     int64_t S, int64_t Q, int R, int H, int K, int G, int mode,
                     uint32_t* __restrict__ error_word) {
  extern __shared__ float s_mem[];
  float* s_q = s_mem;             // [K]
  float* s_x = s_mem + K;         // [H]
  __shared__ int64_t s_idx[kMaxRoutes];
  __shared__ float s_gate[kMaxRoutes];
  __shared__ float s_red[kThreads / 32];
  __shared__ int s_live;

  const int64_t bq = blockIdx.x;
  const int64_t b = bq / Q;
  if (threadIdx.x == 0) s_live = 0;
  __syncthreads();
  if (threadIdx.x < R) {
    int64_t seg = indices[bq * R + threadIdx.x];
    if (seg >= S || seg < -1) {
      if (error_word != nullptr) atomicOr(error_word, kErrGatherIndex);
      seg = -1;
    }
    s_idx[threadIdx.x] = seg;
    s_gate[threadIdx.x] = gates != nullptr ? gates[bq * R + threadIdx.x] : 0.0f;
    if (seg >= 0) atomicOr(&s_live, 1);
  }
  for (int k = threadIdx.x; k < K; k += kThreads) s_q[k] = queries[bq * K + k];
  __syncthreads();

  const bool live = s_live != 0;
  const float* arch_b = archive + b * S * (int64_t)H * K;
  const int lane_in_group = threadIdx.x % G;
  const int group = threadIdx.x / G;
  const int groups = kThreads / G;
  const int iters = (H + groups - 1) / groups;

  for (int it = 0; it < iters; ++it) {
    const int h = it * groups + group;
    float contrib = 0.0f;
    // four routes at a time so that their loads are all issued before use
    for (int r0 = 0; r0 < R; r0 += 4) {
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const float* row[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t seg = r0 + u < R ? s_idx[r0 + u] : -1;
        row[u] = (seg >= 0 && h < H) ? arch_b + (seg * H + h) * (int64_t)K : nullptr;
      }
      for (int k0 = lane_in_group * VEC; k0 < K; k0 += G * VEC) {
        float m[4][VEC];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (row[u] != nullptr) {
            load_row_chunk<VEC>(row[u] + k0, m[u]);
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) m[u][j] = 0.0f;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[u] = fmaf(m[u][j], s_q[k0 + j], acc[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float a = acc[u];
        for (int o = G >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        const int r = r0 + u;
        if (r < R) {
          if (mode == GRMX_FUSE_RETRIEVED) {
            if (lane_in_group == 0 && h < H) out[(bq * R + r) * (int64_t)H + h] = a;
          } else if (s_idx[r] >= 0) {
            contrib = fmaf(s_gate[r], a, contrib);
          }
        }
      }
    }
    if (mode != GRMX_FUSE_RETRIEVED && lane_in_group == 0 && h < H) {
      if (mode == GRMX_FUSE_CONTRIB) {
        out[bq * H + h] = contrib;
      } else {
        s_x[h] = online[bq * H + h] + contrib;
      }
    }
  }
  if (mode != GRMX_FUSE_RESIDUAL_LN) return;
  __syncthreads();

  if (!live) {  // nothing archived for this query: the online state passes through
    for (int h = threadIdx.x; h < H; h += kThreads) out[bq * H + h] = online[bq * H + h];
    return;
  }
  float part = 0.0f;
  for (int h = threadIdx.x; h < H; h += kThreads) part += s_x[h];
  const float mean = block_sum(part, s_red) / (float)H;
  part = 0.0f;
  for (int h = threadIdx.x; h < H; h += kThreads) {
    const float d = s_x[h] - mean;
    part = fmaf(d, d, part);
  }
  const float var = block_sum(part, s_red) / (float)H;
  const float rstd = rsqrtf(var + ln_eps);
  for (int h = threadIdx.x; h < H; h += kThreads) {
    float y = (s_x[h] - mean) * rstd;
    if (ln_weight != nullptr) y *= ln_weight[h];
    if (ln_bias != nullptr) y += ln_bias[h];
    out[bq * H + h] = y;
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_retrieve_fuse(const float* archive, const int64_t* indices, const float* gates,
                                  const float* queries, const float* online, const float* ln_weight,
                                  const float* ln_bias, float ln_eps, void* out, int64_t B, int64_t S,
                                  int64_t Q, int64_t R, int64_t H, int64_t K, int mode, void* stream) {
  using namespace grmx;
  const char* who = "grmx_retrieve_fuse";
  GRMX_REQUIRE(B >= 0 && S >= 0 && Q >= 0 && R >= 0 && H >= 0 && K >= 0, "%s: negative size", who);
  GRMX_REQUIRE(mode == GRMX_FUSE_RETRIEVED || mode == GRMX_FUSE_CONTRIB || mode == GRMX_FUSE_RESIDUAL_LN,
               "%s: bad mode %d", who, mode);
  GRMX_REQUIRE(R <= kMaxRoutes, "%s: R %lld exceeds %d routes", who, (long long)R, kMaxRoutes);
  GRMX_REQUIRE(H <= 8192 && K <= 2048, "%s: H or K too large for one CTA per query", who);
  if (B * Q * H == 0) return GRMX_OK;
  if (mode == GRMX_FUSE_RETRIEVED && R == 0) return GRMX_OK;
  GRMX_REQUIRE(out != nullptr, "%s: out is NULL", who);
  GRMX_REQUIRE(R == 0 || (indices && queries), "%s: NULL indices or queries", who);
  GRMX_REQUIRE(R == 0 || S == 0 || archive, "%s: NULL archive", who);
  GRMX_REQUIRE(mode == GRMX_FUSE_RETRIEVED || R == 0 || gates, "%s: NULL gates", who);
  GRMX_REQUIRE(mode != GRMX_FUSE_RESIDUAL_LN || online, "%s: NULL online state", who);
  const int64_t blocks = B * Q;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "%s: grid too large", who);
  const bool vec = K % 4 == 0 && (reinterpret_cast<uintptr_t>(archive) & 15u) == 0;
  const int VEC = vec ? 4 : 1;
  int G = 1;
  while (G < 32 && G * VEC < K) G <<= 1;
  const size_t smem = sizeof(float) * (size_t)(K + H);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* err = device_error_word_ptr();
  if (vec) {
    retrieve_fuse_kernel<4><<<static_cast<unsigned>(blocks), kThreads, smem, s>>>(
        archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps, static_cast<float*>(out),
        S, Q, (int)R, (int)H, (int)K, G, mode, err);
  } else {
    retrieve_fuse_kernel<1><<<static_cast<unsigned>(blocks), kThreads, smem, s>>>(
        archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps, static_cast<float*>(out),
        S, Q, (int)R, (int)H, (int)K, G, mode, err);
  }
  return check_launch("retrieve_fuse");
}
