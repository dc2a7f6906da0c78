// Sparse top-k routing over archived segment keys: scores, selection, gates.
//
// One warp per (batch row, query).  Lane l scores keys l, l+32, ... with a
// strictly sequential fp32 fused multiply-add over the feature index, so the
// score of a key is a pure function of its inputs (no dependence on the warp
// shape) and the host restatement can reproduce it bit for bit.  Selection is
// R rounds of a warp arg-max over a 64-bit key (ordered score bits, then the
// complemented index) which resolves equal scores to the lower index.
//
// Semantics follow TopKMemoryRetriever.forward (grm/core/gating_unit.py:67-91)
// and _route_chunk (grm/core/paper_grm.py:570-588): identity order when every
// visible key is selected, softmax over the selected scores only.
#include <math_constants.h>

#include "common.cuh"

namespace grmx {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kMaxTopK = 32;

// Monotone map from float to uint32: NaN highest, then +inf ... -inf; both
// zeros share one key so that they tie like they do under float comparison.
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  if (v != v) return 0xffffffffu;
  if (v == 0.0f) return 0x80000000u;
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__global__ void __launch_bounds__(kThreads)
topk_route_kernel(const float* __restrict__ queries, const float* __restrict__ keys,
                  const int32_t* __restrict__ visible, int64_t BQ, int64_t Q, int S, int D,
                  int top_k, float scale, float temperature, const float* __restrict__ given_scores,
                  int64_t* __restrict__ indices_out, float* __restrict__ gates_out,
                  float* __restrict__ scores_out) {
  extern __shared__ float s_scores[];  // [kWarpsPerCta][S] then taken flags
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t bq = (int64_t)blockIdx.x * kWarpsPerCta + warp;
  if (bq >= BQ) return;  // whole warps leave together; no CTA barrier below
  const int64_t b = bq / Q;
  const int64_t q = bq % Q;
  float* sc = s_scores + (size_t)warp * S;
  uint8_t* taken = reinterpret_cast<uint8_t*>(s_scores + (size_t)kWarpsPerCta * S) + (size_t)warp * S;

  int n_vis = S;
  if (visible != nullptr) {
    n_vis = visible[q];
    n_vis = n_vis < 0 ? 0 : (n_vis > S ? S : n_vis);
  }
  const float* qv = queries + bq * D;
  const float* kb = keys + b * (int64_t)S * D;
  const bool vec4 = D % 4 == 0 && ((reinterpret_cast<uintptr_t>(queries) | reinterpret_cast<uintptr_t>(keys)) & 15u) == 0;

  for (int s = lane; s < S; s += 32) {
    float score;
    if (given_scores != nullptr) {
      score = given_scores[bq * S + s];
    } else {
      const float* kr = kb + (int64_t)s * D;
      float acc = 0.0f;
      if (vec4) {
        // same sequential order over d as the scalar loop (the order is part of the contract), but
        // the key row comes in 16-byte pieces, eight of them in flight before the first use
        for (int d0 = 0; d0 < D; d0 += 32) {
          float4 k4[8], q4[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (d0 + 4 * i < D) {
              k4[i] = __ldg(reinterpret_cast<const float4*>(kr + d0) + i);
              q4[i] = __ldg(reinterpret_cast<const float4*>(qv + d0) + i);
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (d0 + 4 * i < D) {
              acc = fmaf(q4[i].x, k4[i].x, acc);
              acc = fmaf(q4[i].y, k4[i].y, acc);
              acc = fmaf(q4[i].z, k4[i].z, acc);
              acc = fmaf(q4[i].w, k4[i].w, acc);
            }
          }
        }
      } else {
        for (int d = 0; d < D; ++d) acc = fmaf(__ldg(qv + d), __ldg(kr + d), acc);
      }
      score = acc * scale;
    }
    sc[s] = score;
    taken[s] = 0;
    if (scores_out != nullptr) scores_out[bq * S + s] = score;
  }
  __syncwarp();

  const int R = top_k < n_vis ? top_k : n_vis;
  int64_t* idx_row = indices_out + bq * top_k;
  float* gate_row = gates_out + bq * top_k;

  // lane r ends up holding route r
  int my_index = -1;
  float my_score = 0.0f;
  if (R == n_vis) {
    if (lane < R) {
      my_index = lane;
      my_score = sc[lane];
    }
  } else {
    for (int r = 0; r < R; ++r) {
      unsigned long long best = 0ull;
      for (int s = lane; s < n_vis; s += 32) {
        if (!taken[s]) {
          const unsigned long long key =
              ((unsigned long long)ordered_bits(sc[s]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)s);
          best = key > best ? key : best;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
      }
      const int win = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
      if (lane == 0) taken[win] = 1;
      if (lane == r) {
        my_index = win;
        my_score = sc[win];
      }
      __syncwarp();
    }
  }

  // softmax over the R selected scores
  const float x = lane < R ? my_score / temperature : -CUDART_INF_F;
  float mx = x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  // fmaxf drops NaN; put it back so a NaN score poisons the row as softmax does
  const unsigned nan_mask = __ballot_sync(0xffffffffu, lane < R && x != x);
  float e = lane < R ? expf(x - mx) : 0.0f;
  float sum = e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  float gate = e / sum;
  if (nan_mask != 0u) gate = CUDART_NAN_F;
  if (lane < top_k) {
    idx_row[lane] = lane < R ? (int64_t)my_index : (int64_t)-1;
    gate_row[lane] = lane < R ? gate : 0.0f;
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_topk_route(const float* queries, const float* keys, const int32_t* visible,
                               int64_t B, int64_t Q, int64_t S, int64_t D, int top_k, float scale,
                               float temperature, int64_t* indices_out, float* gates_out,
                               float* scores_out, void* stream) {
  using namespace grmx;
  GRMX_REQUIRE(B >= 0 && Q >= 0 && S >= 0 && D >= 0, "grmx_topk_route: negative size");
  GRMX_REQUIRE(top_k >= 0 && top_k <= kMaxTopK, "grmx_topk_route: top_k %d outside [0, %d]", top_k, kMaxTopK);
  GRMX_REQUIRE(S <= 2048, "grmx_topk_route: S %lld exceeds 2048 segments", (long long)S);
  GRMX_REQUIRE(D <= 0x7fffffffLL, "grmx_topk_route: D too large");
  if (B * Q == 0 || top_k == 0) return GRMX_OK;
  GRMX_REQUIRE(indices_out && gates_out, "grmx_topk_route: NULL output pointer");
  GRMX_REQUIRE(S == 0 || D == 0 || (queries && keys), "grmx_topk_route: NULL input pointer");
  const int64_t BQ = B * Q;
  const int64_t blocks = (BQ + kWarpsPerCta - 1) / kWarpsPerCta;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "grmx_topk_route: grid too large");
  const size_t smem = (size_t)kWarpsPerCta * S * (sizeof(float) + 1) + 16;
  topk_route_kernel<<<static_cast<unsigned>(blocks), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      queries, keys, visible, BQ, Q, static_cast<int>(S), static_cast<int>(D), top_k, scale,
      temperature, nullptr, indices_out, gates_out, scores_out);
  return check_launch("topk_route");
}

extern "C" int grmx_topk_select(const float* scores, const int32_t* visible, int64_t B, int64_t Q,
                                int64_t S, int top_k, float temperature, int64_t* indices_out,
                                float* gates_out, void* stream) {
  using namespace grmx;
  GRMX_REQUIRE(B >= 0 && Q >= 0 && S >= 0, "grmx_topk_select: negative size");
  GRMX_REQUIRE(top_k >= 0 && top_k <= kMaxTopK, "grmx_topk_select: top_k %d outside [0, %d]", top_k, kMaxTopK);
  GRMX_REQUIRE(S <= 2048, "grmx_topk_select: S %lld exceeds 2048 segments", (long long)S);
  if (B * Q == 0 || top_k == 0) return GRMX_OK;
  GRMX_REQUIRE(indices_out && gates_out, "grmx_topk_select: NULL output pointer");
  GRMX_REQUIRE(S == 0 || scores, "grmx_topk_select: NULL scores");
  const int64_t BQ = B * Q;
  const int64_t blocks = (BQ + kWarpsPerCta - 1) / kWarpsPerCta;
  GRMX_REQUIRE(blocks <= 0x7fffffffLL, "grmx_topk_select: grid too large");
  const size_t smem = (size_t)kWarpsPerCta * S * (sizeof(float) + 1) + 16;
  // S == 0 leaves nothing to read; pass any non-null marker so the kernel skips scoring
  const float* given = scores != nullptr ? scores : reinterpret_cast<const float*>(indices_out);
  topk_route_kernel<<<static_cast<unsigned>(blocks), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      nullptr, nullptr, visible, BQ, Q, static_cast<int>(S), 0, top_k, 1.0f, temperature, given,
      indices_out, gates_out, nullptr);
  return check_launch("topk_select");
}
