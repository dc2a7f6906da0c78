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

#include <mutex>

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

// Selection and gates of one query by one whole warp: sc[S] holds the scores, taken[S] is scratch.
__device__ __forceinline__ void select_and_gate(const float* sc, uint8_t* taken, int n_vis, int top_k,
                                                float temperature, int lane, int64_t* idx_row,
                                                float* gate_row) {
  const int R = top_k < n_vis ? top_k : n_vis;

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

// Few keys, many queries (per-token routing: every token of a segment scores the same handful of
// archived summaries).  With a lane per key and operands straight from global memory, each lane reads
// its key row and its query 16 bytes at a time: the L1 wavefronts and the latency of those small
// reads, not the arithmetic, set the time.  Here a CTA stages the keys of its batch row once in shared
// memory, feature-major ([d/4][key] as float4, so the lanes of a half-warp read consecutive 16-byte
// words), every warp stages its own queries with whole-row coalesced loads, and each half-warp then
// scores kFewChains queries against all keys, a lane per key.  Every score is still the strictly
// sequential fused multiply-add over d: bit-identical to the kernel below.
constexpr int kFewKeys = 16;
constexpr int kFewMaxD = 1024;
constexpr int64_t kFewManyQueries = 16384;                   // from here on the grid fills every SM several times
constexpr int kFewPad = 4;                                   // floats between staged query rows: the two halves of a warp read different banks

__host__ __device__ constexpr size_t few_keys_smem_bytes(int D, int queries_per_cta, int keys = kFewKeys) {
  return sizeof(float) * ((size_t)D * keys + (size_t)queries_per_cta * (D + kFewPad));
}

// Selection for the few-keys kernels: kKeys lanes (16: a half-warp, two queries per warp at once; 32: the
// whole warp) hold the scores of one query, lane s of the group that of key s.  The rank of a key among the
// visible ones (how many beat it: higher score, or the same score and a lower index) comes from kKeys
// independent shuffles instead of a round of dependent ones per route; the key of rank r is route r.  All 32
// lanes must call it together.
template <int kKeys = kFewKeys>
__device__ __forceinline__ void few_keys_select(float score, int lane, int64_t b, int64_t q, int64_t Q, int S, bool query_live,
                                                const int32_t* __restrict__ visible, int top_k, float temperature,
                                                int64_t* __restrict__ indices_out, float* __restrict__ gates_out,
                                                float* __restrict__ scores_out) {
  static_assert(kKeys == 16 || kKeys == 32, "a query's scores lie in a half-warp or in a warp");
  const int group = lane & ~(kKeys - 1);                      // first lane of this query's group
  const int s = lane & (kKeys - 1);
  if (scores_out != nullptr && query_live && s < S) scores_out[(b * Q + q) * S + s] = score;
  int n_vis = S;
  if (visible != nullptr && query_live) {
    n_vis = visible[q];
    n_vis = n_vis < 0 ? 0 : (n_vis > S ? S : n_vis);
  }
  const int R = top_k < n_vis ? top_k : n_vis;
  const bool seen = s < n_vis;
  const unsigned long long mine =
      seen ? (((unsigned long long)ordered_bits(score) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)s)) : 0ull;
  int rank = 0;
#pragma unroll
  for (int j = 0; j < kKeys; ++j) {
    const unsigned long long other = __shfl_sync(0xffffffffu, mine, group | j);
    rank += other > mine ? 1 : 0;
  }
  if (R == n_vis) rank = s;                                  // every visible key is taken: identity order
  const bool chosen = seen && rank < R;
  // softmax over the chosen scores, inside the group
  const float x = chosen ? score / temperature : -CUDART_INF_F;
  float mx = x;
#pragma unroll
  for (int o = kKeys / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  // fmaxf drops NaN; put it back so a NaN score poisons the row as softmax does
  const unsigned group_mask = kKeys == 32 ? 0xffffffffu : (0xffffu << group);
  const unsigned nan_mask = __ballot_sync(0xffffffffu, chosen && x != x) & group_mask;
  const float e = chosen ? expf(x - mx) : 0.0f;
  float sum = e;
#pragma unroll
  for (int o = kKeys / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (query_live) {
    int64_t* idx_row = indices_out + (b * Q + q) * top_k;
    float* gate_row = gates_out + (b * Q + q) * top_k;
    if (chosen) {
      idx_row[rank] = s;
      gate_row[rank] = nan_mask != 0u ? CUDART_NAN_F : e / sum;
    }
    for (int r = R + s; r < top_k; r += kKeys) {             // slots without a route
      idx_row[r] = -1;
      gate_row[r] = 0.0f;
    }
  }
}

// kFewChains queries per group of kKeys lanes (a half-warp for up to 16 keys, the warp for up to 32), kFewWarps
// warps per CTA; TQ: the queries as stored, float or bf16 (widened while they are staged, which is exact: the
// scores do not depend on it)
template <int kFewChains, int kFewWarps, typename TQ, int kKeys = kFewKeys>
__global__ void __launch_bounds__(kFewWarps * 32)
topk_route_few_keys_kernel(const TQ* __restrict__ queries, const float* __restrict__ keys,
                           const int32_t* __restrict__ visible, int64_t Q, int S, int D, int top_k,
                           float scale, float temperature, int64_t* __restrict__ indices_out,
                           float* __restrict__ gates_out, float* __restrict__ scores_out) {
  constexpr int kFewPerWarp = (32 / kKeys) * kFewChains;
  constexpr int kFewPerCta = kFewWarps * kFewPerWarp;
  extern __shared__ float4 s_few[];                           // keys [D/4][kKeys], then queries [kFewPerCta][D/4 + 1]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t b = blockIdx.y;
  const int64_t q0 = (int64_t)blockIdx.x * kFewPerCta;
  const int D4 = D >> 2;
  const int row4 = D4 + kFewPad / 4;
  float4* s_keys = s_few;
  float4* s_q = s_few + (size_t)D4 * kKeys + (size_t)warp * kFewPerWarp * row4;      // this warp's queries

  // this warp's queries are consecutive rows: one contiguous piece of global memory, eight loads per
  // lane in flight; rows past the last query are filled with zeros and dropped below
  const int64_t first = q0 + warp * kFewPerWarp;
  const int64_t rows_here = Q - first < kFewPerWarp ? (Q - first > 0 ? Q - first : 0) : kFewPerWarp;
  if constexpr (sizeof(TQ) == 4) {
    const int n_valid = (int)rows_here * D4;
    const float4* qsrc = reinterpret_cast<const float4*>(queries + (b * Q + first) * D);
    for (int e0 = lane; e0 < kFewPerWarp * D4; e0 += 32 * 8) {
      float4 t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = e0 + 32 * i;
        t[i] = e < n_valid ? __ldg(qsrc + e) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = e0 + 32 * i;
        if (e < kFewPerWarp * D4) {
          const int slot = e / D4;
          s_q[slot * row4 + (e - slot * D4)] = t[i];
        }
      }
    }
  } else {
    // bf16 rows (D % 8 == 0): 16 bytes are eight features, two float4 of the staged row
    const int D8 = D >> 3;
    const int n_valid = (int)rows_here * D8;
    const uint4* qsrc = reinterpret_cast<const uint4*>(queries + (b * Q + first) * D);
    for (int e0 = lane; e0 < kFewPerWarp * D8; e0 += 32 * 8) {
      uint4 t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = e0 + 32 * i;
        t[i] = e < n_valid ? __ldg(qsrc + e) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = e0 + 32 * i;
        if (e < kFewPerWarp * D8) {
          const int slot = e / D8;
          float4* dst = s_q + slot * row4 + 2 * (e - slot * D8);
          dst[0] = make_float4(__uint_as_float(t[i].x << 16), __uint_as_float(t[i].x & 0xffff0000u),
                               __uint_as_float(t[i].y << 16), __uint_as_float(t[i].y & 0xffff0000u));
          dst[1] = make_float4(__uint_as_float(t[i].z << 16), __uint_as_float(t[i].z & 0xffff0000u),
                               __uint_as_float(t[i].w << 16), __uint_as_float(t[i].w & 0xffff0000u));
        }
      }
    }
  }
  const float4* kb = reinterpret_cast<const float4*>(keys + b * (int64_t)S * D);
  for (int e = threadIdx.x; e < D4 * kKeys; e += kFewWarps * 32) {
    const int s = e & (kKeys - 1);
    const int d4 = e / kKeys;
    s_keys[e] = s < S ? __ldg(kb + (int64_t)s * D4 + d4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  __syncthreads();

  const int half = lane / kKeys;                              // the group of this lane (always 0 with 32 keys)
  const int s = lane & (kKeys - 1);
  const float4* ks = s_keys + s;
  const float4* qs = s_q + (size_t)half * kFewChains * row4;  // chain c of this group: query half * kFewChains + c of the warp
  float acc[kFewChains];
#pragma unroll
  for (int c = 0; c < kFewChains; ++c) acc[c] = 0.0f;
  constexpr int kFewDepth = 2;
  for (int d0 = 0; d0 < D4; d0 += kFewDepth) {
    float4 k4[kFewDepth];
    float4 q4[kFewDepth][kFewChains];
#pragma unroll
    for (int i = 0; i < kFewDepth; ++i) {
      if (d0 + i < D4) {
        k4[i] = ks[(d0 + i) * kKeys];
#pragma unroll
        for (int c = 0; c < kFewChains; ++c) q4[i][c] = qs[c * row4 + d0 + i];
      }
    }
#pragma unroll
    for (int i = 0; i < kFewDepth; ++i) {
      if (d0 + i < D4) {
#pragma unroll
        for (int c = 0; c < kFewChains; ++c) acc[c] = fmaf(q4[i][c].x, k4[i].x, acc[c]);
#pragma unroll
        for (int c = 0; c < kFewChains; ++c) acc[c] = fmaf(q4[i][c].y, k4[i].y, acc[c]);
#pragma unroll
        for (int c = 0; c < kFewChains; ++c) acc[c] = fmaf(q4[i][c].z, k4[i].z, acc[c]);
#pragma unroll
        for (int c = 0; c < kFewChains; ++c) acc[c] = fmaf(q4[i][c].w, k4[i].w, acc[c]);
      }
    }
  }
  // selection in registers, all groups of the warp at once
#pragma unroll
  for (int c = 0; c < kFewChains; ++c) {
    const int slot = warp * kFewPerWarp + half * kFewChains + c;
    const int64_t q = q0 + slot;
    few_keys_select<kKeys>(acc[c] * scale, lane, b, q, Q, S, q < Q, visible, top_k, temperature, indices_out, gates_out,
                           scores_out);
  }
}

// The same for very many queries (all tokens of a layer at once): a lane scores a block of 4 queries x 4 keys,
// so that every value read from shared memory feeds four multiply-adds instead of one and the arithmetic,
// not the shared-memory pipe, sets the time.  A warp owns 32 queries (lane (qg, kg): queries qg + 8 i, keys
// 4 kg + j) and walks the features in tiles of 64 that it stages itself, the next tile's loads in flight
// while it computes; each score is still the strictly sequential fused multiply-add over d.
constexpr int kBlkWarps = 8;
constexpr int kBlkQueries = 32;                              // per warp
constexpr int kBlkTile = 64;                                 // features per staged tile
constexpr int kBlkRow4 = kBlkTile / 4 + 1;                   // float4 per staged query row: 8 consecutive rows hit all banks

__host__ __device__ constexpr size_t blocked_smem_bytes(int D) {
  return sizeof(float4) * ((size_t)(D / 4) * kFewKeys + (size_t)kBlkWarps * kBlkQueries * kBlkRow4);
}

template <typename TQ>
__global__ void __launch_bounds__(kBlkWarps * 32, 2)
topk_route_blocked_kernel(const TQ* __restrict__ queries, const float* __restrict__ keys,
                          const int32_t* __restrict__ visible, int64_t Q, int S, int D, int top_k, float scale,
                          float temperature, int64_t* __restrict__ indices_out, float* __restrict__ gates_out,
                          float* __restrict__ scores_out) {
  extern __shared__ float4 s_blk[];                            // keys [D/4][kFewKeys], then per warp [32][kBlkRow4]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t b = blockIdx.y;
  const int D4 = D >> 2;
  float4* s_keys = s_blk;
  float4* s_q = s_blk + (size_t)D4 * kFewKeys + (size_t)warp * kBlkQueries * kBlkRow4;
  const int64_t first = ((int64_t)blockIdx.x * kBlkWarps + warp) * kBlkQueries;    // this warp's first query
  const int rows_here = Q - first < kBlkQueries ? (Q - first > 0 ? (int)(Q - first) : 0) : kBlkQueries;

  const float4* kb = reinterpret_cast<const float4*>(keys + b * (int64_t)S * D);
  // key 4 kg + j sits at position 4 j + kg of its feature row: the four lanes kg that read their j-th key
  // together read neighbouring 16-byte words
  for (int e = threadIdx.x; e < D4 * kFewKeys; e += kBlkWarps * 32) {
    const int pos = e & (kFewKeys - 1);
    const int s = 4 * (pos & 3) + (pos >> 2);
    const int d4 = e >> 4;
    s_keys[e] = s < S ? __ldg(kb + (int64_t)s * D4 + d4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }

  // a tile of the warp's queries: 32 rows x 64 features; 16-byte pieces, a row's pieces in neighbouring lanes
  constexpr int kPieces = sizeof(TQ) == 2 ? 8 : 16;            // per row and tile
  constexpr int kLoads = kBlkQueries * kPieces / 32;            // per lane and tile
  const TQ* qbase = queries + (b * Q + first) * D;
  uint4 pre[kLoads];
  auto fetch = [&](int tile) {
#pragma unroll
    for (int i = 0; i < kLoads; ++i) {
      const int e = lane + 32 * i;
      const int row = e / kPieces, piece = e % kPieces;
      pre[i] = row < rows_here ? __ldg(reinterpret_cast<const uint4*>(qbase + (int64_t)row * D + tile * kBlkTile) + piece)
                               : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int i = 0; i < kLoads; ++i) {
      const int e = lane + 32 * i;
      const int row = e / kPieces, piece = e % kPieces;
      if constexpr (sizeof(TQ) == 2) {
        float4* dst = s_q + row * kBlkRow4 + 2 * piece;
        dst[0] = make_float4(__uint_as_float(pre[i].x << 16), __uint_as_float(pre[i].x & 0xffff0000u),
                             __uint_as_float(pre[i].y << 16), __uint_as_float(pre[i].y & 0xffff0000u));
        dst[1] = make_float4(__uint_as_float(pre[i].z << 16), __uint_as_float(pre[i].z & 0xffff0000u),
                             __uint_as_float(pre[i].w << 16), __uint_as_float(pre[i].w & 0xffff0000u));
      } else {
        s_q[row * kBlkRow4 + piece] = make_float4(__uint_as_float(pre[i].x), __uint_as_float(pre[i].y),
                                                  __uint_as_float(pre[i].z), __uint_as_float(pre[i].w));
      }
    }
  };

  const int kg = lane & 3, qg = lane >> 2;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  }
  const int n_tiles = D / kBlkTile;
  fetch(0);
  __syncthreads();                                            // the keys are staged
  for (int tile = 0; tile < n_tiles; ++tile) {
    __syncwarp();                                             // everybody is done with the tile before
    stage();
    if (tile + 1 < n_tiles) fetch(tile + 1);
    __syncwarp();
    const float4* ks = s_keys + (size_t)tile * (kBlkTile / 4) * kFewKeys + kg;
    const float4* qs = s_q + qg * kBlkRow4;
#pragma unroll 4
    for (int d4 = 0; d4 < kBlkTile / 4; ++d4) {
      float4 k4[4], q4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) k4[j] = ks[d4 * kFewKeys + 4 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i) q4[i] = qs[8 * i * kBlkRow4 + d4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q4[i].x, k4[j].x, acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q4[i].y, k4[j].y, acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q4[i].z, k4[j].z, acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q4[i].w, k4[j].w, acc[i][j]);
      }
    }
  }
  // the scores of a query lie in four lanes: through the warp's staging area into the layout of the selection
  // (lane (half, s): key s of the query of that half-warp)
  __syncwarp();
  float* sc = reinterpret_cast<float*>(s_q);                   // [32 queries][17]
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) sc[(qg + 8 * i) * (kFewKeys + 1) + 4 * kg + j] = acc[i][j] * scale;
  }
  __syncwarp();
  const int half = lane >> 4, s = lane & (kFewKeys - 1);
  for (int pair = 0; pair < kBlkQueries / 2; ++pair) {
    const int slot = 2 * pair + half;
    const int64_t q = first + slot;
    few_keys_select(sc[slot * (kFewKeys + 1) + s], lane, b, q, Q, S, q < Q, visible, top_k, temperature, indices_out,
                    gates_out, scores_out);
  }
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

  select_and_gate(sc, taken, n_vis, top_k, temperature, lane, indices_out + bq * top_k, gates_out + bq * top_k);
}

}  // namespace
}  // namespace grmx

namespace grmx {
namespace {
template <int kChains, int kWarps, typename TQ, int kKeys = kFewKeys>
int launch_few_keys(const TQ* queries, const float* keys, const int32_t* visible, int64_t B, int64_t Q, int64_t S,
                    int64_t D, int top_k, float scale, float temperature, int64_t* indices_out, float* gates_out,
                    float* scores_out, cudaStream_t stream) {
  constexpr int per_cta = (32 / kKeys) * kChains * kWarps;
  const size_t need = few_keys_smem_bytes(static_cast<int>(D), per_cta, kKeys);
  {
    // the opt-in is per device and grows with the largest request seen there
    static std::mutex mutex;
    static size_t configured[64] = {0};
    int device = 0;
    cudaGetDevice(&device);
    std::lock_guard<std::mutex> lock(mutex);
    if (device < 0 || device >= 64 || need > configured[device]) {
      const cudaError_t opted = cudaFuncSetAttribute(topk_route_few_keys_kernel<kChains, kWarps, TQ, kKeys>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(need));
      GRMX_REQUIRE(opted == cudaSuccess, "grmx_topk_route: shared-memory opt-in failed: %s", cudaGetErrorString(opted));
      if (device >= 0 && device < 64) configured[device] = need;
    }
  }
  const dim3 grid(static_cast<unsigned>((Q + per_cta - 1) / per_cta), static_cast<unsigned>(B));
  topk_route_few_keys_kernel<kChains, kWarps, TQ, kKeys><<<grid, kWarps * 32, need, stream>>>(
      queries, keys, visible, Q, static_cast<int>(S), static_cast<int>(D), top_k, scale, temperature, indices_out,
      gates_out, scores_out);
  return check_launch("topk_route_few_keys");
}

template <typename TQ>
int launch_blocked(const TQ* queries, const float* keys, const int32_t* visible, int64_t B, int64_t Q, int64_t S,
                   int64_t D, int top_k, float scale, float temperature, int64_t* indices_out, float* gates_out,
                   float* scores_out, cudaStream_t stream) {
  const size_t need = blocked_smem_bytes(static_cast<int>(D));
  {
    static std::mutex mutex;
    static size_t configured[64] = {0};
    int device = 0;
    cudaGetDevice(&device);
    std::lock_guard<std::mutex> lock(mutex);
    if (device < 0 || device >= 64 || need > configured[device]) {
      const cudaError_t opted = cudaFuncSetAttribute(topk_route_blocked_kernel<TQ>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(need));
      GRMX_REQUIRE(opted == cudaSuccess, "grmx_topk_route: shared-memory opt-in failed: %s", cudaGetErrorString(opted));
      if (device >= 0 && device < 64) configured[device] = need;
    }
  }
  constexpr int per_cta = kBlkWarps * kBlkQueries;
  const dim3 grid(static_cast<unsigned>((Q + per_cta - 1) / per_cta), static_cast<unsigned>(B));
  topk_route_blocked_kernel<TQ><<<grid, kBlkWarps * 32, need, stream>>>(queries, keys, visible, Q, static_cast<int>(S),
                                                                        static_cast<int>(D), top_k, scale, temperature,
                                                                        indices_out, gates_out, scores_out);
  return check_launch("topk_route_blocked");
}
// GRMX_ROUTE_BLOCKED=off keeps very many queries on the lane-per-key kernel
bool blocked_form_applies(int64_t B, int64_t Q, int64_t D) {
  static const bool disabled = [] {
    const char* env = getenv("GRMX_ROUTE_BLOCKED");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  return !disabled && B * Q >= kFewManyQueries && D % kBlkTile == 0;
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
  const bool aligned = ((reinterpret_cast<uintptr_t>(queries) | reinterpret_cast<uintptr_t>(keys)) & 15u) == 0;
  if (S >= 1 && S <= kFewKeys && Q >= 64 && D >= 4 && D % 4 == 0 && D <= kFewMaxD && aligned && B <= 65535) {
    // measured at 8 x 512 queries of 512 features: one query per half-warp and 16 warps per CTA
    // (15.9 us against 29 us with four queries per half-warp and 4 warps, 43 us for the kernel below)
    // many CTAs per SM: two queries per half-warp share each key load (116 against 125 us at 65536 queries)
    if (blocked_form_applies(B, Q, D)) {
      return launch_blocked<float>(queries, keys, visible, B, Q, S, D, top_k, scale, temperature, indices_out, gates_out,
                                   scores_out, static_cast<cudaStream_t>(stream));
    }
    if (B * Q >= kFewManyQueries) {
      return launch_few_keys<2, 8, float>(queries, keys, visible, B, Q, S, D, top_k, scale, temperature, indices_out,
                                          gates_out, scores_out, static_cast<cudaStream_t>(stream));
    }
    return launch_few_keys<1, 16, float>(queries, keys, visible, B, Q, S, D, top_k, scale, temperature, indices_out, gates_out,
                                  scores_out, static_cast<cudaStream_t>(stream));
  }
  // GRMX_ROUTE_WARP_KEYS=off keeps 17..32 keys on the kernel without staging
  static const bool warp_keys_off = [] {
    const char* env = getenv("GRMX_ROUTE_WARP_KEYS");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  if (!warp_keys_off && S > kFewKeys && S <= 32 && Q >= 16 && D >= 4 && D % 4 == 0 && D <= kFewMaxD && aligned &&
      B <= 65535) {
    // 17..32 keys (segment-level routing over a full archive): the same staging with the whole warp on one
    // query, a lane per key; the kernel below reads every key row 16 bytes per lane at a stride of a row, 32
    // L1 wavefronts per load (measured at 128 rows x 32 queries x 32 keys of 64 features: 20 us)
    return launch_few_keys<1, 16, float, 32>(queries, keys, visible, B, Q, S, D, top_k, scale, temperature, indices_out,
                                             gates_out, scores_out, static_cast<cudaStream_t>(stream));
  }
  const size_t smem = (size_t)kWarpsPerCta * S * (sizeof(float) + 1) + 16;
  topk_route_kernel<<<static_cast<unsigned>(blocks), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      queries, keys, visible, BQ, Q, static_cast<int>(S), static_cast<int>(D), top_k, scale,
      temperature, nullptr, indices_out, gates_out, scores_out);
  return check_launch("topk_route");
}

extern "C" int grmx_topk_route_bf16q(const void* queries_bf16, const float* keys, const int32_t* visible, int64_t B,
                                     int64_t Q, int64_t S, int64_t D, int top_k, float scale, float temperature,
                                     int64_t* indices_out, float* gates_out, float* scores_out, void* stream) {
  using namespace grmx;
  const char* who = "grmx_topk_route_bf16q";
  GRMX_REQUIRE(B >= 0 && Q >= 0 && S >= 0 && D >= 0, "%s: negative size", who);
  GRMX_REQUIRE(top_k >= 0 && top_k <= kMaxTopK, "%s: top_k %d outside [0, %d]", who, top_k, kMaxTopK);
  if (B * Q == 0 || top_k == 0) return GRMX_OK;
  GRMX_REQUIRE(indices_out && gates_out, "%s: NULL output pointer", who);
  GRMX_REQUIRE(queries_bf16 && keys, "%s: NULL input pointer", who);
  const bool aligned = ((reinterpret_cast<uintptr_t>(queries_bf16) | reinterpret_cast<uintptr_t>(keys)) & 15u) == 0;
  if (!(S >= 1 && S <= kFewKeys && Q >= 64 && D >= 8 && D % 8 == 0 && D <= kFewMaxD && aligned && B <= 65535)) {
    return fail(GRMX_ERR_UNSUPPORTED,
                "%s: covers 1..%d keys, at least 64 queries per batch row, D %% 8 == 0, D <= %d, 16-byte aligned "
                "inputs; widen the queries to float32 and call grmx_topk_route otherwise", who, kFewKeys, kFewMaxD);
  }
  if (blocked_form_applies(B, Q, D)) {
    return launch_blocked<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(queries_bf16), keys, visible, B, Q, S, D, top_k,
                                         scale, temperature, indices_out, gates_out, scores_out,
                                         static_cast<cudaStream_t>(stream));
  }
  if (B * Q >= kFewManyQueries) {
    return launch_few_keys<2, 8, __nv_bfloat16>(static_cast<const __nv_bfloat16*>(queries_bf16), keys, visible, B, Q, S,
                                                D, top_k, scale, temperature, indices_out, gates_out, scores_out,
                                                static_cast<cudaStream_t>(stream));
  }
  return launch_few_keys<1, 16, __nv_bfloat16>(static_cast<const __nv_bfloat16*>(queries_bf16), keys, visible, B, Q, S,
                                               D, top_k, scale, temperature, indices_out, gates_out, scores_out,
                                               static_cast<cudaStream_t>(stream));
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
