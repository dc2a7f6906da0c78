/*
 * Plain-C restatement of GRM's segment-memory path -- TEST INFRASTRUCTURE ONLY.
 *
 * Built by oracle/build_oracle.py into oracle/_build/libgrm_oracle.so and used
 * as (a) the bit-exact checker for routing scores / top-k / gather and (b) the
 * timed CPU "port" baseline.  Nothing in the product package links or loads it.
 * Parity status: pinned -- tests/test_oracle.py compares every function with
 * fixtures generated from the reference's Python implementation.
 *
 * Citations are paths inside the Sggggt/RNN_with_GRM project.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Token-serial scan in fp32, operation order of grm/csrc/grm_cuda.cpp:67-83:
 *   update = (v k^T) * inv_scale;  M = M*decay + update*beta;  h = M q       */
void grm_chunk_update_seq_f32(const float* keys, const float* values, const float* queries,
                              const float* memory_in, float* hidden, float* memory_out, int64_t B,
                              int64_t T, int64_t K, int64_t H, float decay) {
  const float inv_scale = (float)(1.0 / sqrt((double)K));
  const float beta = (float)(1.0 - (double)decay);
  const int64_t rows = B * H;
#pragma omp parallel for schedule(static)
  for (int64_t bh = 0; bh < rows; ++bh) {
    const int64_t b = bh / H;
    const int64_t h = bh % H;
    float* m = memory_out + bh * K;
    memcpy(m, memory_in + bh * K, sizeof(float) * (size_t)K);
    for (int64_t t = 0; t < T; ++t) {
      const float* k = keys + (b * T + t) * K;
      const float* q = queries + (b * T + t) * K;
      const float v = values[(b * T + t) * H + h];
      float acc = 0.0f;
      for (int64_t j = 0; j < K; ++j) {
        const float update = (v * k[j]) * inv_scale;
        m[j] = m[j] * decay + update * beta;
        acc += m[j] * q[j];
      }
      hidden[(b * T + t) * H + h] = acc;
    }
  }
}

/* hidden[n,r,h] = sum_k M[n,r,h,k] q[n,k]   (grm/core/cuda_ops.py:257-262) */
void grm_apply_query_f32(const float* memories, const float* queries, float* hidden, int64_t N,
                         int64_t R, int64_t H, int64_t K) {
  const int64_t rows = N * R * H;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    const int64_t n = row / (R * H);
    const float* m = memories + row * K;
    const float* q = queries + n * K;
    float acc = 0.0f;
    for (int64_t j = 0; j < K; ++j) acc += m[j] * q[j];
    hidden[row] = acc;
  }
}

/* out[b,j,:] = mem[b, idx[b,j], :]   (grm/core/cuda_ops.py:265-284); -1 -> zeros.
 * Returns the number of indices outside [-1, S). */
int64_t grm_batched_gather(const void* memories, const int64_t* indices, void* out, int64_t B,
                           int64_t S, int64_t J, int64_t row_bytes) {
  int64_t bad = 0;
  for (int64_t b = 0; b < B; ++b) {
    for (int64_t j = 0; j < J; ++j) {
      const int64_t seg = indices[b * J + j];
      char* dst = (char*)out + (b * J + j) * row_bytes;
      if (seg >= 0 && seg < S) {
        memcpy(dst, (const char*)memories + (b * S + seg) * row_bytes, (size_t)row_bytes);
      } else {
        memset(dst, 0, (size_t)row_bytes);
        if (seg != -1) ++bad;
      }
    }
  }
  return bad;
}

/* score[b,q,s] = scale * (sequential fp32 fused multiply-add over d).  The
 * summation order is the engine's contract; the reference uses torch.matmul
 * (grm/core/paper_grm.py:574) whose order is unspecified. */
void grm_route_scores(const float* queries, const float* keys, float* scores, int64_t B, int64_t Q,
                      int64_t S, int64_t D, float scale) {
#pragma omp parallel for schedule(static)
  for (int64_t bq = 0; bq < B * Q; ++bq) {
    const int64_t b = bq / Q;
    const float* q = queries + bq * D;
    for (int64_t s = 0; s < S; ++s) {
      const float* k = keys + (b * S + s) * D;
      float acc = 0.0f;
      for (int64_t d = 0; d < D; ++d) acc = fmaf(q[d], k[d], acc);
      scores[bq * S + s] = acc * scale;
    }
  }
}

/* Order used for selection: NaN above every number, zeros of either sign equal. */
static int score_greater(float a, int64_t ia, float b, int64_t ib) {
  const int an = isnan(a), bn = isnan(b);
  if (an != bn) return an;
  if (!an && a != b) return a > b;
  return ia < ib;
}

/* Selection and gates (grm/core/gating_unit.py:81-90, grm/core/paper_grm.py:576-588):
 * R = min(top_k, visible); identity order when R == visible; otherwise the R
 * best scores, descending, equal scores to the lower index; gates =
 * softmax(selected / temperature); unused slots: index -1, gate 0. */
void grm_topk_select(const float* scores, const int32_t* visible, int64_t B, int64_t Q, int64_t S,
                     int top_k, float temperature, int64_t* indices_out, float* gates_out) {
  for (int64_t bq = 0; bq < B * Q; ++bq) {
    const int64_t q = bq % Q;
    const float* sc = scores + bq * S;
    int64_t* idx = indices_out + bq * top_k;
    float* gate = gates_out + bq * top_k;
    int64_t n_vis = visible ? visible[q] : S;
    if (n_vis < 0) n_vis = 0;
    if (n_vis > S) n_vis = S;
    const int64_t R = top_k < n_vis ? top_k : n_vis;
    float sel[64];
    for (int r = 0; r < top_k; ++r) { idx[r] = -1; gate[r] = 0.0f; }
    if (R == 0) continue;
    if (R == n_vis) {
      for (int64_t r = 0; r < R; ++r) { idx[r] = r; sel[r] = sc[r]; }
    } else {
      char* taken = (char*)calloc((size_t)n_vis, 1);
      for (int64_t r = 0; r < R; ++r) {
        int64_t best = -1;
        for (int64_t s = 0; s < n_vis; ++s) {
          if (taken[s]) continue;
          if (best < 0 || score_greater(sc[s], s, sc[best], best)) best = s;
        }
        taken[best] = 1;
        idx[r] = best;
        sel[r] = sc[best];
      }
      free(taken);
    }
    float mx = -INFINITY;
    int any_nan = 0;
    for (int64_t r = 0; r < R; ++r) {
      sel[r] = sel[r] / temperature;
      if (isnan(sel[r])) any_nan = 1;
      if (sel[r] > mx) mx = sel[r];
    }
    float sum = 0.0f;
    for (int64_t r = 0; r < R; ++r) { sel[r] = expf(sel[r] - mx); sum += sel[r]; }
    for (int64_t r = 0; r < R; ++r) gate[r] = any_nan ? NAN : sel[r] / sum;
  }
}

/* gather -> apply-query -> gate-weighted sum -> LayerNorm(online + contrib)
 * (grm/core/paper_grm.py:229-234,301-307,604-611; grm/core/aggregator.py:104-119,144).
 * A query with no live slot copies `online` (paper_grm.py:620-621). */
void grm_retrieve_fuse_f32(const float* archive, const int64_t* indices, const float* gates,
                           const float* queries, const float* online, const float* ln_weight,
                           const float* ln_bias, float eps, float* out, int64_t B, int64_t S,
                           int64_t Q, int64_t R, int64_t H, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t bq = 0; bq < B * Q; ++bq) {
    const int64_t b = bq / Q;
    float* x = out + bq * H;
    int live = 0;
    for (int64_t h = 0; h < H; ++h) x[h] = online[bq * H + h];
    for (int64_t r = 0; r < R; ++r) {
      const int64_t seg = indices[bq * R + r];
      if (seg < 0 || seg >= S) continue;
      live = 1;
      const float g = gates[bq * R + r];
      const float* m = archive + (b * S + seg) * H * K;
      for (int64_t h = 0; h < H; ++h) {
        float acc = 0.0f;
        for (int64_t j = 0; j < K; ++j) acc += m[h * K + j] * queries[bq * K + j];
        x[h] += g * acc;
      }
    }
    if (!live) continue;
    double mean = 0.0, var = 0.0;
    for (int64_t h = 0; h < H; ++h) mean += x[h];
    mean /= (double)H;
    for (int64_t h = 0; h < H; ++h) var += (x[h] - mean) * (x[h] - mean);
    var /= (double)H;
    const double rstd = 1.0 / sqrt(var + (double)eps);
    for (int64_t h = 0; h < H; ++h) {
      double y = (x[h] - mean) * rstd;
      if (ln_weight) y *= ln_weight[h];
      if (ln_bias) y += ln_bias[h];
      x[h] = (float)y;
    }
  }
}
