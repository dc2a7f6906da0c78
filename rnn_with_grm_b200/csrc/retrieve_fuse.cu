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
constexpr int kRows = 2;               // matrix rows per lane group with loads in flight together

template <int VEC>
__device__ __forceinline__ void load_row_chunk(const float* p, float (&out)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
    out[0] = __ldg(p);
  }
}

// VEC floats per load, G lanes per matrix row (G * VEC divides into K in whole steps or covers it
// once), kPerRoute: the per-route products are the result (mode "retrieved"); otherwise the gate
// weights are applied lane by lane before the one reduction per row.
template <int VEC, int G, bool kPerRoute>
__global__ void __launch_bounds__(kThreads)
retrieve_fuse_kernel(const float* __restrict__ archive, const int64_t* __restrict__ indices,
                     const float* __restrict__ gates, const float* __restrict__ queries,
                     const float* __restrict__ online, const float* __restrict__ ln_weight,
                     const float* __restrict__ ln_bias, float ln_eps, float* __restrict__ out,
                     int64_t S, int64_t Q, int R, int H, int K, int mode,
                     uint32_t* __restrict__ error_word) {
  extern __shared__ float s_mem[];
  float* s_q = s_mem;             // [K]
  float* s_x = s_mem + K;         // [H]
  __shared__ int64_t s_idx[kMaxRoutes];
  __shared__ float s_gate[kMaxRoutes];
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
  constexpr int groups = kThreads / G;
  const int iters = (H + groups - 1) / groups;

  // kRows matrix rows per group at a time, four routes each: all of their loads (kRows x 4 x 16 bytes
  // per lane) are issued before the first use.  The kernel is bound by instruction issue, not by
  // bytes in flight, so the loops below are fully unrolled over compile-time lane counts, and for the
  // fused modes the gate-weighted sum over routes is formed per lane (in route order) before the
  // single reduction of a row over its G lanes.
  for (int it0 = 0; it0 < iters; it0 += kRows) {
    float contrib[kRows];
#pragma unroll
    for (int v = 0; v < kRows; ++v) contrib[v] = 0.0f;
    for (int r0 = 0; r0 < R; r0 += 4) {
      float acc[kRows][4];
      const float* row[kRows][4];
      float gate[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t seg = r0 + u < R ? s_idx[r0 + u] : -1;
        gate[u] = seg >= 0 ? s_gate[r0 + u] : 0.0f;
        const float* mat = seg >= 0 ? arch_b + seg * H * (int64_t)K : nullptr;
#pragma unroll
        for (int v = 0; v < kRows; ++v) {
          const int h = (it0 + v) * groups + group;
          row[v][u] = (mat != nullptr && h < H) ? mat + h * (int64_t)K : nullptr;
          acc[v][u] = 0.0f;
        }
      }
      for (int k0 = lane_in_group * VEC; k0 < K; k0 += G * VEC) {
        float m[kRows][4][VEC];
#pragma unroll
        for (int v = 0; v < kRows; ++v) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (row[v][u] != nullptr) {
              load_row_chunk<VEC>(row[v][u] + k0, m[v][u]);
            } else {
#pragma unroll
              for (int j = 0; j < VEC; ++j) m[v][u][j] = 0.0f;
            }
          }
        }
        float qv[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) qv[j] = s_q[k0 + j];
#pragma unroll
        for (int v = 0; v < kRows; ++v) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[v][u] = fmaf(m[v][u][j], qv[j], acc[v][u]);
          }
        }
      }
#pragma unroll
      for (int v = 0; v < kRows; ++v) {
        if constexpr (kPerRoute) {
          const int h = (it0 + v) * groups + group;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float a = acc[v][u];
#pragma unroll
            for (int o = G >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (r0 + u < R && lane_in_group == 0 && h < H) out[(bq * R + r0 + u) * (int64_t)H + h] = a;
          }
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) contrib[v] = fmaf(gate[u], acc[v][u], contrib[v]);
        }
      }
    }
    if constexpr (!kPerRoute) {
#pragma unroll
      for (int v = 0; v < kRows; ++v) {
        const int h = (it0 + v) * groups + group;
        float a = contrib[v];
#pragma unroll
        for (int o = G >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane_in_group == 0 && h < H) {
          if (mode == GRMX_FUSE_CONTRIB) {
            out[bq * H + h] = a;
          } else {
            s_x[h] = online[bq * H + h] + a;
          }
        }
      }
    }
  }
  if (mode != GRMX_FUSE_RESIDUAL_LN) return;
  __syncthreads();

  if (!live) {  // nothing archived for this query: the online state passes through
    for (int h = threadIdx.x; h < H; h += kThreads) out[bq * H + h] = online[bq * H + h];
    return;
  }
  // LayerNorm over the H values of the row by the first warp alone (fixed-order shuffles): the other
  // warps are done and free their slots instead of waiting at four more CTA barriers
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  float part = 0.0f;
  for (int h = lane; h < H; h += 32) part += s_x[h];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  const float mean = part / (float)H;
  part = 0.0f;
  for (int h = lane; h < H; h += 32) {
    const float d = s_x[h] - mean;
    part = fmaf(d, d, part);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  const float rstd = rsqrtf(part / (float)H + ln_eps);
  for (int h = lane; h < H; h += 32) {
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
  // fused modes: two steps over K per lane, i.e. fewer reduction steps per byte.  The per-route mode
  // keeps one step per lane: its results are defined to equal gather followed by apply-query bit for bit.
  if (mode != GRMX_FUSE_RETRIEVED && G >= 4 && K % (G / 2 * VEC) == 0) G >>= 1;
  const size_t smem = sizeof(float) * (size_t)(K + H);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* err = device_error_word_ptr();
  const bool per_route = mode == GRMX_FUSE_RETRIEVED;
#define GRMX_FUSE_LAUNCH(V, GG)                                                                                     \
  do {                                                                                                              \
    if (per_route) {                                                                                                \
      retrieve_fuse_kernel<V, GG, true><<<static_cast<unsigned>(blocks), kThreads, smem, s>>>(                      \
          archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps, static_cast<float*>(out), S, Q,     \
          (int)R, (int)H, (int)K, mode, err);                                                                       \
    } else {                                                                                                        \
      retrieve_fuse_kernel<V, GG, false><<<static_cast<unsigned>(blocks), kThreads, smem, s>>>(                     \
          archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps, static_cast<float*>(out), S, Q,     \
          (int)R, (int)H, (int)K, mode, err);                                                                       \
    }                                                                                                               \
  } while (0)
  if (vec) {
    switch (G) {
      case 1: GRMX_FUSE_LAUNCH(4, 1); break;
      case 2: GRMX_FUSE_LAUNCH(4, 2); break;
      case 4: GRMX_FUSE_LAUNCH(4, 4); break;
      case 8: GRMX_FUSE_LAUNCH(4, 8); break;
      case 16: GRMX_FUSE_LAUNCH(4, 16); break;
      default: GRMX_FUSE_LAUNCH(4, 32); break;
    }
  } else {
    switch (G) {
      case 1: GRMX_FUSE_LAUNCH(1, 1); break;
      case 2: GRMX_FUSE_LAUNCH(1, 2); break;
      case 4: GRMX_FUSE_LAUNCH(1, 4); break;
      case 8: GRMX_FUSE_LAUNCH(1, 8); break;
      case 16: GRMX_FUSE_LAUNCH(1, 16); break;
      default: GRMX_FUSE_LAUNCH(1, 32); break;
    }
  }
#undef GRMX_FUSE_LAUNCH
  return check_launch("retrieve_fuse");
}
