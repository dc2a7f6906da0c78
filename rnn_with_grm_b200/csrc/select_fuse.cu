// Selection half of the fused retrieval when the candidates have already been applied to the query.
//
// With per-token routing every token of a segment chooses among the same few archived matrices, so
// the caller applies the query to all of them with one batched GEMM (states[b,q,s,:] = M[b,s] q[b,q])
// and what is left of RetrievedStateFusion (grm/core/aggregator.py:104-105, 116-118) is, per token:
// pick R of the S candidate states, weight them by the gates, add the online state, LayerNorm.
// One warp per token; the row stays in registers between the sum and the normalisation.
#include <type_traits>

#include "common.cuh"

namespace grmx {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kMaxPerLane = 32;   // register path covers H <= 1024
constexpr int kMaxRoutes = 32;

// VEC consecutive elements of a row: one 16-byte load when VEC spans 16 bytes.  The loaded words are
// kept as they come (for bf16, half the registers of the floats) until they are used.
__device__ __forceinline__ uint4 load_raw16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

template <typename T, int VEC>
__device__ __forceinline__ void unpack_piece(const uint4& v, float (&out)[VEC]) {
  static_assert(VEC * sizeof(T) == 16, "a 16-byte piece");
  if constexpr (sizeof(T) == 4) {
    out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
    out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {            // bf16 -> fp32 is a shift
      out[2 * j] = __uint_as_float(w[j] << 16);
      out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void load_piece(const T* p, float (&out)[VEC]) {
  if constexpr (VEC == 1) {
    if constexpr (sizeof(T) == 4) out[0] = __ldg(reinterpret_cast<const float*>(p));
    else out[0] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  } else {
    unpack_piece<T, VEC>(load_raw16(p), out);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_piece(T* p, const float (&in)[VEC]) {
  if constexpr (VEC == 1) {
    if constexpr (sizeof(T) == 4) *reinterpret_cast<float*>(p) = in[0];
    else *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(in[0]);
  } else if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(in[2 * j], in[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Lane l owns the pieces l, l + 32, ... of the row, VEC elements each, kPieces of them at most
// (kPieces * 32 * VEC >= H: short rows take fewer registers and more warps fit an SM).
template <typename T, int VEC, int kPieces>
__global__ void __launch_bounds__(kWarpsPerCta * 32, (VEC > 1 && kPieces * VEC <= 16) ? 4 : 1)
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

  // the online row is requested now and kept as loaded (packed) until the routes have been summed
  using Held = typename std::conditional<(VEC > 1), uint4, float>::type;
  Held held[kPieces];
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    if constexpr (VEC > 1) {
      held[i] = (fuse && h < H) ? load_raw16(online + bq * H + h) : make_uint4(0u, 0u, 0u, 0u);
    } else {
      float one[1] = {0.0f};
      if (fuse && h < H) load_piece<T, 1>(online + bq * H + h, one);
      held[i] = one[0];
    }
  }
  float contrib[kPieces][VEC];
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) contrib[i][j] = 0.0f;
  }
  // kRoutes routes at a time (as many as the registers hold): their rows are all requested before
  // the first one is used.  The sum still runs in route order.
  constexpr int kRoutes = (VEC > 1 ? kPieces <= 4 : kPieces <= 16) ? 4 : 2;
  for (int r0 = 0; r0 < R; r0 += kRoutes) {
    const T* row[kRoutes];
    float gate[kRoutes];
#pragma unroll
    for (int u = 0; u < kRoutes; ++u) {
      // every lane takes part in the shuffles, whatever part of the row it owns
      const int src = r0 + u < R ? r0 + u : 0;
      const int64_t idx = __shfl_sync(0xffffffffu, my_idx, src);
      gate[u] = __shfl_sync(0xffffffffu, my_gate, src);
      row[u] = (r0 + u < R && idx >= 0) ? cand + idx * H : nullptr;   // the same for all lanes
    }
    if constexpr (VEC > 1) {
      uint4 raw[kRoutes][kPieces];
#pragma unroll
      for (int u = 0; u < kRoutes; ++u) {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          const int h = (lane + 32 * i) * VEC;
          raw[u][i] = (row[u] != nullptr && h < H) ? load_raw16(row[u] + h) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < kRoutes; ++u) {
        if (row[u] == nullptr) continue;                      // an empty route adds nothing, not even 0 * x
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          float m[VEC];
          unpack_piece<T, VEC>(raw[u][i], m);
#pragma unroll
          for (int j = 0; j < VEC; ++j) contrib[i][j] = fmaf(gate[u], m[j], contrib[i][j]);
        }
      }
    } else {
      float m[kRoutes][kPieces];
#pragma unroll
      for (int u = 0; u < kRoutes; ++u) {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
          const int h = lane + 32 * i;
          float one[1] = {0.0f};
          if (row[u] != nullptr && h < H) load_piece<T, 1>(row[u] + h, one);
          m[u][i] = one[0];
        }
      }
#pragma unroll
      for (int u = 0; u < kRoutes; ++u) {
        if (row[u] == nullptr) continue;
#pragma unroll
        for (int i = 0; i < kPieces; ++i) contrib[i][0] = fmaf(gate[u], m[u][i], contrib[i][0]);
      }
    }
  }
  float x[kPieces][VEC];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    if constexpr (VEC > 1) unpack_piece<T, VEC>(held[i], x[i]);
    else x[i][0] = held[i];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      x[i][j] += contrib[i][j];       // online + contribution, as the reference adds them
      sum += x[i][j];
    }
  }
  if (!fuse || !live) {
    // the contribution alone, or (nothing archived for this token) the online state untouched
#pragma unroll
    for (int i = 0; i < kPieces; ++i) {
      const int h = (lane + 32 * i) * VEC;
      if (h < H) store_piece<T, VEC>(out + bq * H + h, x[i]);
    }
    return;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / (float)H;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    if (h < H) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float d = x[i][j] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / (float)H + ln_eps);
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    if (h < H) {
      // weight and bias of the piece in 16-byte loads (one 4-byte load per element costs the cache a
      // line per lane and instruction: a thousand wavefronts per row of 512)
      float wv[VEC], bv[VEC];
      if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int j4 = 0; j4 < VEC / 4; ++j4) {
          const float4 w4 = ln_weight != nullptr ? __ldg(reinterpret_cast<const float4*>(ln_weight + h) + j4)
                                                 : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
          const float4 b4 = ln_bias != nullptr ? __ldg(reinterpret_cast<const float4*>(ln_bias + h) + j4)
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          wv[4 * j4] = w4.x; wv[4 * j4 + 1] = w4.y; wv[4 * j4 + 2] = w4.z; wv[4 * j4 + 3] = w4.w;
          bv[4 * j4] = b4.x; bv[4 * j4 + 1] = b4.y; bv[4 * j4 + 2] = b4.z; bv[4 * j4 + 3] = b4.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          wv[j] = ln_weight != nullptr ? __ldg(ln_weight + h + j) : 1.0f;
          bv[j] = ln_bias != nullptr ? __ldg(ln_bias + h + j) : 0.0f;
        }
      }
      float y[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        y[j] = (x[i][j] - mean) * rstd;
        if (ln_weight != nullptr) y[j] *= wv[j];
        if (ln_bias != nullptr) y[j] += bv[j];
      }
      store_piece<T, VEC>(out + bq * H + h, y);
    }
  }
}

template <typename T, int VEC, int kPieces>
void launch_select_fuse_pieces(const void* states, const int64_t* indices, const float* gates, const void* online,
                               const float* ln_weight, const float* ln_bias, float ln_eps, void* out, int64_t BQ,
                               int S, int R, int H, int mode, cudaStream_t s, uint32_t* err) {
  const int64_t blocks = (BQ + kWarpsPerCta - 1) / kWarpsPerCta;
  select_fuse_kernel<T, VEC, kPieces><<<static_cast<unsigned>(blocks), kWarpsPerCta * 32, 0, s>>>(
      static_cast<const T*>(states), indices, gates, static_cast<const T*>(online), ln_weight, ln_bias, ln_eps,
      static_cast<T*>(out), BQ, S, R, H, mode, err);
}

template <typename T, int VEC>
void launch_select_fuse(const void* states, const int64_t* indices, const float* gates, const void* online,
                        const float* ln_weight, const float* ln_bias, float ln_eps, void* out, int64_t BQ, int S,
                        int R, int H, int mode, cudaStream_t s, uint32_t* err) {
  constexpr int kMost = kMaxPerLane / VEC;
  const int needed = (H + 32 * VEC - 1) / (32 * VEC);
#define GRMX_SELECT(P)                                                                                           \
  launch_select_fuse_pieces<T, VEC, (P) <= kMost ? (P) : kMost>(states, indices, gates, online, ln_weight, ln_bias, \
                                                                ln_eps, out, BQ, S, R, H, mode, s, err)
  if (needed <= 1) GRMX_SELECT(1);
  else if (needed <= 2) GRMX_SELECT(2);
  else if (needed <= 4) GRMX_SELECT(4);
  else if (needed <= 8) GRMX_SELECT(8);
  else GRMX_SELECT(kMost);
#undef GRMX_SELECT
}


// LayerNorm(a + b) over rows of H values, one pass, a warp per row: the residual block between layers
// (grm/core/multilayer_grm.py:93,96).  The same arithmetic as the residual rule above with b as the only
// candidate and a unit gate (sum in fp32, one rounding; mean and variance in the same order), without the
// route bookkeeping and its dependent loads: both rows are requested at once.
template <typename T, int VEC, int kPieces>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
add_layer_norm_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ ln_weight,
                      const float* __restrict__ ln_bias, float ln_eps, T* __restrict__ out, int64_t rows, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;   // whole warps leave together; no CTA barrier below
  uint4 ra[kPieces], rb[kPieces];
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    ra[i] = h < H ? load_raw16(a + row * H + h) : make_uint4(0u, 0u, 0u, 0u);
    rb[i] = h < H ? load_raw16(b + row * H + h) : make_uint4(0u, 0u, 0u, 0u);
  }
  float x[kPieces][VEC];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    float other[VEC];
    unpack_piece<T, VEC>(ra[i], x[i]);
    unpack_piece<T, VEC>(rb[i], other);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      x[i][j] += other[j];
      sum += x[i][j];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / (float)H;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    if (h < H) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float d = x[i][j] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / (float)H + ln_eps);
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int h = (lane + 32 * i) * VEC;
    if (h < H) {
      float y[VEC];
#pragma unroll
      for (int j4 = 0; j4 < VEC / 4; ++j4) {
        const float4 w4 = ln_weight != nullptr ? __ldg(reinterpret_cast<const float4*>(ln_weight + h) + j4)
                                               : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        const float4 b4 = ln_bias != nullptr ? __ldg(reinterpret_cast<const float4*>(ln_bias + h) + j4)
                                             : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
        const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = (x[i][4 * j4 + j] - mean) * rstd;
          if (ln_weight != nullptr) v *= wv[j];
          if (ln_bias != nullptr) v += bv[j];
          y[4 * j4 + j] = v;
        }
      }
      store_piece<T, VEC>(out + row * H + h, y);
    }
  }
}

template <typename T, int VEC>
void launch_add_layer_norm(const void* a, const void* b, const float* w, const float* bias, float eps, void* out,
                           int64_t rows, int H, cudaStream_t s) {
  const unsigned blocks = static_cast<unsigned>((rows + kWarpsPerCta - 1) / kWarpsPerCta);
  const int needed = (H + 32 * VEC - 1) / (32 * VEC);
#define GRMX_ALN(P)                                                                                                  \
  add_layer_norm_kernel<T, VEC, P><<<blocks, kWarpsPerCta * 32, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), \
                                                                          w, bias, eps, static_cast<T*>(out), rows, H)
  if (needed <= 1) GRMX_ALN(1);
  else if (needed <= 2) GRMX_ALN(2);
  else if (needed <= 4) GRMX_ALN(4);
  else GRMX_ALN(kMaxPerLane / VEC);
#undef GRMX_ALN
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
  // 16-byte pieces when every row starts on a 16-byte boundary
  const uintptr_t bases = reinterpret_cast<uintptr_t>(states) | reinterpret_cast<uintptr_t>(online) |
                          reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(ln_weight) |
                          reinterpret_cast<uintptr_t>(ln_bias);
  const int per16 = dtype == GRMX_F32 ? 4 : 8;
  const bool vec = H % per16 == 0 && (bases & 15u) == 0;
  if (dtype == GRMX_F32) {
    if (vec) launch_select_fuse<float, 4>(states, indices, gates, online, ln_weight, ln_bias, ln_eps, out, BQ, (int)S, (int)R, (int)H, mode, s, err);
    else launch_select_fuse<float, 1>(states, indices, gates, online, ln_weight, ln_bias, ln_eps, out, BQ, (int)S, (int)R, (int)H, mode, s, err);
  } else {
    if (vec) launch_select_fuse<__nv_bfloat16, 8>(states, indices, gates, online, ln_weight, ln_bias, ln_eps, out, BQ, (int)S, (int)R, (int)H, mode, s, err);
    else launch_select_fuse<__nv_bfloat16, 1>(states, indices, gates, online, ln_weight, ln_bias, ln_eps, out, BQ, (int)S, (int)R, (int)H, mode, s, err);
  }
  return check_launch("select_fuse");
}

extern "C" int grmx_add_layer_norm(const void* a, const void* b, const float* ln_weight, const float* ln_bias,
                                   float ln_eps, void* out, int64_t rows, int64_t H, int dtype, void* stream) {
  using namespace grmx;
  const char* who = "grmx_add_layer_norm";
  GRMX_REQUIRE(rows >= 0 && H >= 0, "%s: negative size", who);
  GRMX_REQUIRE(dtype == GRMX_F32 || dtype == GRMX_BF16, "%s: dtype must be f32 or bf16", who);
  if (rows * H == 0) return GRMX_OK;
  GRMX_REQUIRE(a != nullptr && b != nullptr && out != nullptr, "%s: NULL tensor", who);
  const int per16 = dtype == GRMX_F32 ? 4 : 8;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out) |
                          reinterpret_cast<uintptr_t>(ln_weight) | reinterpret_cast<uintptr_t>(ln_bias);
  if (H % per16 != 0 || (bases & 15u) != 0 || H > 32 * kMaxPerLane) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: needs rows of whole 16-byte pieces, 16-byte aligned tensors and H <= %d", who,
                32 * kMaxPerLane);
  }
  GRMX_REQUIRE((rows + kWarpsPerCta - 1) / kWarpsPerCta <= 0x7fffffffLL, "%s: grid too large", who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == GRMX_F32) launch_add_layer_norm<float, 4>(a, b, ln_weight, ln_bias, ln_eps, out, rows, (int)H, s);
  else launch_add_layer_norm<__nv_bfloat16, 8>(a, b, ln_weight, ln_bias, ln_eps, out, rows, (int)H, s);
  return check_launch("add_layer_norm");
}
