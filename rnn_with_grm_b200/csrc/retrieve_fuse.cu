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
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

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


// ---- slot-major form: one CTA per batch row ----
// With few queries per row that choose among few archived matrices (segment-level routing: Q queries,
// R of S slots each, Q * R a multiple of S), the query-major kernel above reads every matrix once per
// query that chose it, from L2 at best.  Here a CTA walks the chosen slots of its row: a producer warp
// brings each matrix into a ring in shared memory, one bulk copy per matrix row (rows padded by 16 bytes so
// that a lane per matrix row reads without bank conflicts); consumer warps apply it to all queries that
// chose it -- a lane owns a matrix row, the query values are broadcast reads, no cross-lane reduction --
// and add gate * (M q) to the sums of their slot set; the sets are added in a fixed order, then the
// residual and the LayerNorm follow per query.  The sum over a query's routes therefore runs in an order
// fixed by the slots, not by the routes: results agree with the query-major kernel to fp32 rounding.
constexpr int kRowsConsumers = 8;                        // consumer warps
constexpr int kRowsThreads = (kRowsConsumers + 1) * 32;  // + the producer warp
constexpr int kRowsBatch = 8;                            // queries applied to a matrix chunk held in registers
constexpr int kRowsMaxStages = 32;

struct RowsPlan {
  int n_blocks;      // 32-row blocks of a matrix: 1, 2, 4 or 8
  int n_sets;        // sets of n_blocks warps; set s takes the chosen slots s, s + n_sets, ...
  int n_stages;      // units of 32 matrix rows in the ring, the same number for every consumer warp
  size_t smem;
};

// NB queries applied to 32 columns of one matrix row held in m, where m[j] is the 16-byte piece (j + rot) & 7
// of those columns: acc_row[q * Hp] += gate * (m . q[32 columns])
template <int K, int NB>
__device__ __forceinline__ void rows_apply(const float4 (&m)[8], const float* q_cols, int rot, const int* list_q,
                                           const float* list_g, int i0, int left, float* acc_row, int Hp) {
  float dot[NB];
  const float4* qv[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    dot[u] = 0.0f;
    qv[u] = reinterpret_cast<const float4*>(q_cols + list_q[u < left ? i0 + u : i0] * K);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float4 x[NB];
#pragma unroll
    for (int u = 0; u < NB; ++u) x[u] = qv[u][(j + rot) & 7];
#pragma unroll
    for (int u = 0; u < NB; ++u) dot[u] = fmaf(m[j].x, x[u].x, dot[u]);
#pragma unroll
    for (int u = 0; u < NB; ++u) dot[u] = fmaf(m[j].y, x[u].y, dot[u]);
#pragma unroll
    for (int u = 0; u < NB; ++u) dot[u] = fmaf(m[j].z, x[u].z, dot[u]);
#pragma unroll
    for (int u = 0; u < NB; ++u) dot[u] = fmaf(m[j].w, x[u].w, dot[u]);
  }
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    if (u < left) {
      float* a = acc_row + list_q[i0 + u] * Hp;
      *a = fmaf(list_g[i0 + u], dot[u], *a);
    }
  }
}

// The same for K a multiple of 64, with four times fewer shared-memory reads per multiply-add: lane
// (kq, rg) = (lane / 8, lane % 8) holds rows 4 rg .. 4 rg + 3 of the unit over a quarter of a span of columns
// (128 columns when K is a multiple of 128, else 64), 16 columns (four 16-byte pieces) at a time, so a query
// value read from shared memory feeds four rows.  The pieces of a lane's columns are visited in an order
// rotated by rg (eight lanes that read together hit eight different bank groups, four with the narrow span;
// the query is read in the same order).  The partial sums of the four lanes kq of a row group are added by
// shuffles and lane kq adds row 4 rg + kq to the sums.
template <int K, int NB, int PIECES>
__device__ __forceinline__ void rows_apply_tiled(const float4 (&m)[4][4], const float* q_cols, int first_piece, int rg, int kq,
                                                 const int* list_q, const float* list_g, int i0, int left, float* acc_rows,
                                                 int Hp, bool row_live) {
  float dot[4][NB];
  const float4* qv[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    qv[u] = reinterpret_cast<const float4*>(q_cols + list_q[u < left ? i0 + u : i0] * K);
#pragma unroll
    for (int i = 0; i < 4; ++i) dot[i][u] = 0.0f;
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int piece = (first_piece + p + rg) & (PIECES - 1);
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const float4 x = qv[u][piece];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dot[i][u] = fmaf(m[i][p].x, x.x, dot[i][u]);
        dot[i][u] = fmaf(m[i][p].y, x.y, dot[i][u]);
        dot[i][u] = fmaf(m[i][p].z, x.z, dot[i][u]);
        dot[i][u] = fmaf(m[i][p].w, x.w, dot[i][u]);
      }
    }
  }
  // lanes kq = 0..3 of a row group differ in lane bits 3 and 4
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float t = dot[i][u];
      t += __shfl_xor_sync(0xffffffffu, t, 8);
      t += __shfl_xor_sync(0xffffffffu, t, 16);
      if (i == kq) mine = t;
    }
    if (u < left && row_live) {
      float* a = acc_rows + list_q[i0 + u] * Hp;
      *a = fmaf(list_g[i0 + u], mine, *a);
    }
  }
}

template <int KC>                      // 32-float chunks per matrix row: K = 32 * KC
__global__ void __launch_bounds__(kRowsThreads)
retrieve_fuse_rows_kernel(const float* __restrict__ archive, const int64_t* __restrict__ indices,
                          const float* __restrict__ gates, const float* __restrict__ queries,
                          const float* __restrict__ online, const float* __restrict__ ln_weight,
                          const float* __restrict__ ln_bias, float ln_eps, float* __restrict__ out,
                          int S, int Q, int R, int H, int mode, RowsPlan plan, uint32_t* __restrict__ error_word) {
  using namespace tc;
  constexpr int K = 32 * KC;
  extern __shared__ float4 s_rows_mem[];
  const int Hp = 32 * plan.n_blocks;
  constexpr int kUnitFloats = 32 * K;                           // a unit of the ring: 32 rows of a matrix, as they lie in memory
  float* s_ring = reinterpret_cast<float*>(s_rows_mem);         // [n_stages][32][K]
  float* s_q = s_ring + plan.n_stages * kUnitFloats;            // [Q, K]
  float* s_acc = s_q + Q * K;                                   // [n_sets][Q][Hp]
  float* s_gate = s_acc + plan.n_sets * Q * Hp;                 // [Q * R]
  float* s_list_g = s_gate + Q * R;                             // [Q * R]: gate of every live entry, grouped by slot
  int* s_list_q = reinterpret_cast<int*>(s_list_g + Q * R);     // [Q * R]: its query
  int* s_idx = s_list_q + Q * R;                                // [Q * R], -1 = no route
  int* s_start = s_idx + Q * R;                                 // [S + 1]
  int* s_chosen = s_start + S + 1;                              // [S + 1]: the slots somebody chose; [S] = how many
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(s_chosen + S + 1);   // an even number of words lies before it
  uint64_t* bar_empty = bar_full + kRowsMaxStages;
  int* s_issued = reinterpret_cast<int*>(bar_empty + kRowsMaxStages);   // [kRowsMaxStages]: parity of the last fill, -1 none
  volatile int* s_abort = s_issued + kRowsMaxStages;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int64_t b = blockIdx.x;
  const int entries = Q * R;
  const bool residual = mode == GRMX_FUSE_RESIDUAL_LN;
  if (tid == 0) {
    for (int i = 0; i < kRowsMaxStages; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], 1);
      s_issued[i] = -1;
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i <= S; i += kRowsThreads) s_start[i] = 0;
  __syncthreads();
  for (int e = tid; e < entries; e += kRowsThreads) {
    int64_t seg = indices[b * entries + e];
    if (seg >= S || seg < -1) {
      if (error_word != nullptr) atomicOr(error_word, kErrGatherIndex);
      seg = -1;
    }
    s_idx[e] = static_cast<int>(seg);
    s_gate[e] = gates[b * entries + e];
    if (seg >= 0) atomicAdd(&s_start[seg + 1], 1);              // how many entries chose the slot
  }
  {
    const float4* src = reinterpret_cast<const float4*>(queries + b * Q * K);
    float4* dst = reinterpret_cast<float4*>(s_q);
    for (int i = tid; i < Q * K / 4; i += kRowsThreads) dst[i] = src[i];
  }
  // the sums start from zero; set 0 from the online state when that is to be added
  {
    float4* acc4 = reinterpret_cast<float4*>(s_acc);
    const int first = residual ? Q * Hp / 4 : 0;
    for (int i = first + tid; i < plan.n_sets * Q * Hp / 4; i += kRowsThreads) acc4[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (residual) {
      for (int q = warp; q < Q; q += kRowsThreads / 32) {
        for (int hh = lane; hh < Hp; hh += 32) s_acc[q * Hp + hh] = hh < H ? online[(b * Q + q) * H + hh] : 0.0f;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    int chosen = 0;
    for (int slot = 0; slot < S; ++slot) {
      if (s_start[slot + 1] > 0) s_chosen[chosen++] = slot;
      s_start[slot + 1] += s_start[slot];
    }
    s_chosen[S] = chosen;
  }
  __syncthreads();
  // live entries grouped by slot, in entry order within a slot (deterministic): a warp per slot, 32 entries a
  // step.  Only the consumers need the lists; the producer knows the chosen slots and starts its copies.
  for (int slot = warp; warp < kRowsConsumers && slot < S; slot += kRowsConsumers) {
    int at = s_start[slot];
    const int stop = s_start[slot + 1];
    for (int e0 = 0; e0 < entries && at < stop; e0 += 32) {
      const int e = e0 + lane;
      const bool match = e < entries && s_idx[e] == slot;
      const unsigned votes = __ballot_sync(0xffffffffu, match);
      if (match) {
        const int pos = at + __popc(votes & ((1u << lane) - 1u));
        s_list_q[pos] = e / R;
        s_list_g[pos] = s_gate[e];
      }
      at += __popc(votes);
    }
  }
  if (warp < kRowsConsumers) asm volatile("bar.sync 1, %0;" ::"n"(kRowsConsumers * 32) : "memory");
  const int n_chosen = s_chosen[S];
  const int per_warp = plan.n_stages / kRowsConsumers;          // stages of a consumer warp's own ring

  // Consumer warp w = set * n_blocks + rb takes rows 32 rb .. 32 rb + 31 of the chosen slots set, set + n_sets, ...
  // A unit of the ring is that block of rows of one matrix, contiguous in memory: one bulk copy.  Warp w owns
  // the stages w, w + 8, ... and walks them with its own unit counter, so it sees every completion of their
  // barriers (a waiter that skipped one would take the parity of an older phase for the one it waits for).
  if (warp == kRowsConsumers) {
    // ===== producer: lane w feeds consumer warp w, so one instruction issues up to eight copies (issuing a
    // bulk copy keeps the issuing warp busy for about 0.3 us, measured; one copy per instruction made the
    // producer the bottleneck) =====
    const float* arch_b = archive + b * S * static_cast<int64_t>(H) * K;
    const int rb = lane % plan.n_blocks, set = lane / plan.n_blocks;
    const int n_units = lane < kRowsConsumers && set < n_chosen ? (n_chosen - set + plan.n_sets - 1) / plan.n_sets : 0;
    const int most = (n_chosen + plan.n_sets - 1) / plan.n_sets;  // set 0 has the most units
    for (int v = 0; v < most; ++v) {
      const bool mine = v < n_units;
      const int stage = lane + kRowsConsumers * (v % per_warp);
      const uint32_t fill_parity = static_cast<uint32_t>(v / per_warp) & 1u;
      bool ready = !mine || v < per_warp;                       // else: the unit before in this stage has been read
      bool all_ready = false;
      for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (!ready) ready = mbar_try_wait(&bar_empty[stage], fill_parity ^ 1u) != 0;
        all_ready = __all_sync(0xffffffffu, ready);
        if (all_ready || ((it & 63u) == 63u && *s_abort)) break;
      }
      if (!all_ready) {
        *s_abort = 1;
        break;
      }
      if (mine) {
        const float* mat = arch_b + static_cast<int64_t>(s_chosen[set + v * plan.n_sets]) * H * K;
        const int rows = min(32, H - 32 * rb);
        const uint32_t bytes = static_cast<uint32_t>(rows) * K * 4u;
        mbar_expect_tx(&bar_full[stage], bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(s_ring + stage * kUnitFloats)),
                     "l"(mat + static_cast<int64_t>(32 * rb) * K), "r"(bytes), "r"(smem_u32(&bar_full[stage]))
                     : "memory");
        s_issued[stage] = static_cast<int>(fill_parity);
      }
      __syncwarp();
    }
    if (*s_abort && lane == 0) {   // let the copies in flight land before the shared memory is released
      for (int stage = 0; stage < plan.n_stages; ++stage) {
        if (s_issued[stage] >= 0) mbar_wait_quiet(&bar_full[stage], static_cast<uint32_t>(s_issued[stage]));
      }
    }
  } else {
    // ===== consumers =====
    const int rb = warp % plan.n_blocks, set = warp / plan.n_blocks;   // warps beyond the last set have no work
    const int h = 32 * rb + lane;
    const int lane_read = h < H ? lane : H - 1 - 32 * rb;       // rows past H are computed and dropped
    // Rows lie K floats apart, a multiple of 32 banks: lane l therefore reads the 16-byte pieces of a
    // 32-column chunk in the order l, l + 1, ... (mod 8), which spreads eight neighbouring lanes over all
    // banks, and reads the query in the same order.
    const int rot = lane_read & 7;
    float* acc_row = s_acc + set * Q * Hp + 32 * rb + lane;
    int v = 0;
    for (int ci = set < plan.n_sets ? set : n_chosen; ci < n_chosen; ci += plan.n_sets, ++v) {
      const int stage = warp + kRowsConsumers * (v % per_warp);
      if (!mbar_wait(&bar_full[stage], static_cast<uint32_t>(v / per_warp) & 1u, s_abort)) break;
      const int slot = s_chosen[ci];
      const int begin = s_start[slot], end = s_start[slot + 1];
      if constexpr (K % 64 == 0) {
        // ---- four rows x a quarter span per lane (see rows_apply_tiled) ----
        constexpr int kSpan = K % 128 == 0 ? 128 : 64;          // columns per span
        constexpr int kPieces = kSpan / 16;                     // 16-byte pieces of a lane's quarter: 8 or 4
        const int rg = lane & 7, kq = lane >> 3;
        const int rows_here = min(32, H - 32 * rb);
        const float* unit = s_ring + stage * kUnitFloats;
        const bool row_live = 4 * rg + kq < rows_here;          // the row this lane adds to the sums
        float* acc_rows = s_acc + set * Q * Hp + 32 * rb + 4 * rg + kq;
#pragma unroll 1
        for (int span = 0; span < K / kSpan; ++span) {
#pragma unroll 1
          for (int half = 0; half < kPieces / 4; ++half) {
            float4 m[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = min(4 * rg + i, rows_here - 1);     // rows past the end are computed and dropped
              const float4* row = reinterpret_cast<const float4*>(unit + r * K + kSpan * span + (kSpan / 4) * kq);
#pragma unroll
              for (int p4 = 0; p4 < 4; ++p4) m[i][p4] = row[(4 * half + p4 + rg) & (kPieces - 1)];
            }
            if (span == K / kSpan - 1 && half == kPieces / 4 - 1) {   // the unit is in registers: its stage can be refilled
              __syncwarp();
              if (lane == 0) {
                mbar_arrive(&bar_empty[stage]);
              }
            }
            const float* q_cols = s_q + kSpan * span + (kSpan / 4) * kq;
            for (int i0 = begin; i0 < end;) {
              const int left = end - i0;                        // uniform across the warp
              if (left > 4) {
                rows_apply_tiled<K, kRowsBatch, kPieces>(m, q_cols, 4 * half, rg, kq, s_list_q, s_list_g, i0, left, acc_rows, Hp, row_live);
                i0 += kRowsBatch;
              } else {
                rows_apply_tiled<K, 4, kPieces>(m, q_cols, 4 * half, rg, kq, s_list_q, s_list_g, i0, left, acc_rows, Hp, row_live);
                i0 += 4;
              }
            }
          }
        }
      } else {
      const float4* row = reinterpret_cast<const float4*>(s_ring + stage * kUnitFloats + lane_read * K);
#pragma unroll 1
      for (int c = 0; c < KC; ++c) {
        float4 m[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) m[j] = row[8 * c + ((j + rot) & 7)];
        if (c == KC - 1) {   // the unit is in registers: its stage can be refilled
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&bar_empty[stage]);
          }
        }
        // kRowsBatch queries at a time (four when no more are left), all of their dot products advancing
        // together: without branches inside, the chains of different queries interleave.  Entries past
        // the end of the list repeat the first one and are dropped.
        for (int i0 = begin; i0 < end;) {
          const int left = end - i0;                            // uniform across the warp
          if (left > 4) {
            rows_apply<K, kRowsBatch>(m, s_q + 32 * c, rot, s_list_q, s_list_g, i0, left, acc_row, Hp);
            i0 += kRowsBatch;
          } else {
            rows_apply<K, 4>(m, s_q + 32 * c, rot, s_list_q, s_list_g, i0, left, acc_row, Hp);
            i0 += 4;
          }
        }
      }
      }
    }
  }
  __syncthreads();
  if (*s_abort) {
    if (tid == 0 && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
    return;
  }

  // per query: the sets added in order (set 0 started from the online state), then the LayerNorm, one warp
  // per query
  for (int q = warp; q < Q; q += kRowsThreads / 32) {
    const int64_t bq = b * Q + q;
    float* x = s_acc + q * Hp;
    if (residual) {
      bool live = false;
      for (int r = 0; r < R; ++r) live |= s_idx[q * R + r] >= 0;
      if (!live) {                       // nothing archived for this query: the online state passes through
        for (int hh = lane; hh < H; hh += 32) out[bq * H + hh] = x[hh];
        continue;
      }
    }
    float part = 0.0f;
    for (int hh = lane; hh < H; hh += 32) {
      float v = x[hh];
      for (int set = 1; set < plan.n_sets; ++set) v += s_acc[(set * Q + q) * Hp + hh];
      x[hh] = v;
      part += v;
    }
    if (!residual) {
      for (int hh = lane; hh < H; hh += 32) out[bq * H + hh] = x[hh];
      continue;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float mean = part / static_cast<float>(H);
    part = 0.0f;
    for (int hh = lane; hh < H; hh += 32) {
      const float d = x[hh] - mean;
      part = fmaf(d, d, part);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const float rstd = rsqrtf(part / static_cast<float>(H) + ln_eps);
    for (int hh = lane; hh < H; hh += 32) {
      float y = (x[hh] - mean) * rstd;
      if (ln_weight != nullptr) y *= ln_weight[hh];
      if (ln_bias != nullptr) y += ln_bias[hh];
      out[bq * H + hh] = y;
    }
  }
}

// How a shape is laid out in shared memory; n_stages == 0: not covered.
RowsPlan rows_plan(int64_t S, int64_t Q, int64_t R, int64_t H, int64_t K) {
  RowsPlan plan = {0, 0, 0, 0};
  const int64_t n_blocks = (H + 31) / 32;
  if (n_blocks != 1 && n_blocks != 2 && n_blocks != 4 && n_blocks != 8) return plan;
  plan.n_blocks = static_cast<int>(n_blocks);
  plan.n_sets = kRowsConsumers / plan.n_blocks;
  const int64_t fixed = 4 * (Q * K + plan.n_sets * Q * 32 * n_blocks + 4 * Q * R + 2 * (S + 1)) +
                        (8 * 2 + 4) * kRowsMaxStages + 16;
  const int64_t unit = 4 * 32 * K;                              // 32 rows of a matrix
  const int64_t budget = 200 * 1024;
  int64_t stages = (budget - fixed) / unit;
  if (stages > kRowsMaxStages) stages = kRowsMaxStages;
  stages -= stages % kRowsConsumers;                            // the same number for every consumer warp
  if (stages < kRowsConsumers) return plan;
  plan.n_stages = static_cast<int>(stages);
  plan.smem = static_cast<size_t>(fixed + stages * unit);
  return plan;
}

// Shapes the slot-major kernel covers (K = 32, 64, ..., 256; H in 1..256 with 1, 2, 4 or 8 blocks of 32
// rows; a unit of 32 rows per consumer warp and everything else of a row within 200 KiB of shared memory).
bool rows_form_covers(const float* archive, const float* queries, int64_t B, int64_t S, int64_t Q, int64_t R,
                      int64_t H, int64_t K, int mode) {
  if (mode == GRMX_FUSE_RETRIEVED || B < 1 || B > 0x7fffffffLL || R < 1 || S < 1 || Q < 1 || H < 1) return false;
  if (K % 32 != 0 || K > 256 || S > 4096 || Q * R > 8192 || S * Q * R > (1 << 18)) return false;
  if (!tc::device_is_sm100()) return false;
  if ((reinterpret_cast<uintptr_t>(archive) | reinterpret_cast<uintptr_t>(queries)) & 15u) return false;
  return rows_plan(S, Q, R, H, K).n_stages >= kRowsConsumers;
}

int launch_rows_form(const float* archive, const int64_t* indices, const float* gates, const float* queries,
                     const float* online, const float* ln_weight, const float* ln_bias, float ln_eps, float* out,
                     int64_t B, int64_t S, int64_t Q, int64_t R, int64_t H, int64_t K, int mode, cudaStream_t stream) {
  const RowsPlan plan = rows_plan(S, Q, R, H, K);
  uint32_t* err = device_error_word_ptr();
#define GRMX_ROWS_LAUNCH(KC)                                                                                        \
  do {                                                                                                              \
    if (plan.smem > 48 * 1024) {                                                                                    \
      const cudaError_t attr = cudaFuncSetAttribute(retrieve_fuse_rows_kernel<KC>,                                  \
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 1024); \
      if (attr != cudaSuccess) return fail(GRMX_ERR_LAUNCH, "retrieve_fuse (slot-major): %s", cudaGetErrorString(attr)); \
    }                                                                                                               \
    retrieve_fuse_rows_kernel<KC><<<static_cast<unsigned>(B), kRowsThreads, plan.smem, stream>>>(                   \
        archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps, out, (int)S, (int)Q, (int)R,      \
        (int)H, mode, plan, err);                                                                                         \
  } while (0)
  switch (K / 32) {
    case 1: GRMX_ROWS_LAUNCH(1); break;
    case 2: GRMX_ROWS_LAUNCH(2); break;
    case 3: GRMX_ROWS_LAUNCH(3); break;
    case 4: GRMX_ROWS_LAUNCH(4); break;
    case 5: GRMX_ROWS_LAUNCH(5); break;
    case 6: GRMX_ROWS_LAUNCH(6); break;
    case 7: GRMX_ROWS_LAUNCH(7); break;
    default: GRMX_ROWS_LAUNCH(8); break;
  }
#undef GRMX_ROWS_LAUNCH
  return check_launch("retrieve_fuse_rows");
}

// The slot-major form pays when a row's queries share matrices (Q * R entries over S slots) and there are
// enough rows to fill the GPU; GRMX_RETRIEVE_ROWS=off keeps every call on the query-major kernel.
bool rows_form_preferred(int64_t B, int64_t S, int64_t Q, int64_t R) {
  static const bool disabled = [] {
    const char* env = getenv("GRMX_RETRIEVE_ROWS");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  return !disabled && B >= 64 && Q * R >= 2 * S;
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
  if (rows_form_preferred(B, S, Q, R) && rows_form_covers(archive, queries, B, S, Q, R, H, K, mode)) {
    return launch_rows_form(archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps,
                            static_cast<float*>(out), B, S, Q, R, H, K, mode, static_cast<cudaStream_t>(stream));
  }
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

extern "C" int grmx_retrieve_fuse_rows(const float* archive, const int64_t* indices, const float* gates,
                                       const float* queries, const float* online, const float* ln_weight,
                                       const float* ln_bias, float ln_eps, void* out, int64_t B, int64_t S,
                                       int64_t Q, int64_t R, int64_t H, int64_t K, int mode, void* stream) {
  using namespace grmx;
  const char* who = "grmx_retrieve_fuse_rows";
  GRMX_REQUIRE(B >= 0 && S >= 0 && Q >= 0 && R >= 0 && H >= 0 && K >= 0, "%s: negative size", who);
  GRMX_REQUIRE(mode == GRMX_FUSE_CONTRIB || mode == GRMX_FUSE_RESIDUAL_LN, "%s: bad mode %d", who, mode);
  if (B * Q * H == 0) return GRMX_OK;
  GRMX_REQUIRE(out != nullptr && indices != nullptr && gates != nullptr && queries != nullptr && archive != nullptr,
               "%s: NULL tensor", who);
  GRMX_REQUIRE(mode != GRMX_FUSE_RESIDUAL_LN || online, "%s: NULL online state", who);
  if (!rows_form_covers(archive, queries, B, S, Q, R, H, K, mode)) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: needs K a multiple of 32 up to 256, H up to 256 in 1, 2, 4 or 8 blocks of 32 "
                "rows, 16-byte aligned tensors and eight blocks of 32 matrix rows plus a row's queries and sums within "
                "200 KiB of shared memory", who);
  }
  return launch_rows_form(archive, indices, gates, queries, online, ln_weight, ln_bias, ln_eps,
                          static_cast<float*>(out), B, S, Q, R, H, K, mode, static_cast<cudaStream_t>(stream));
}
