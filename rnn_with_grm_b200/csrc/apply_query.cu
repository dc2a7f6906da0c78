// hidden[n,r,h] = sum_k memories[n,r,h,k] * queries[n,k] and its gradients.
//
// The forward is a stream over `memories` (0.5 flop per byte), so it is laid
// out for HBM: a group of G lanes owns one matrix row and reads it with
// 16-byte loads, four rows in flight per group, q staged once per CTA in
// shared memory.  Math: grm/core/cuda_ops.py:257-262.
#include <algorithm>

#include "common.cuh"

namespace grmx {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 256;

template <typename T, int VEC>
struct VecLoad;
template <>
struct VecLoad<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&out)[4]) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <>
struct VecLoad<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float (&out)[1]) { out[0] = __ldg(p); }
};
template <>
struct VecLoad<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <>
struct VecLoad<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&out)[1]) {
    out[0] = __bfloat162float(*p);
  }
};
template <>
struct VecLoad<__half, 8> {
  static __device__ __forceinline__ void load(const __half* p, float (&out)[8]) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
};
template <>
struct VecLoad<__half, 1> {
  static __device__ __forceinline__ void load(const __half* p, float (&out)[1]) {
    out[0] = __half2float(*p);
  }
};

// G lanes per row (power of two <= 32), chosen on the host so that one pass of
// the group covers min(K, 32*VEC) elements.
template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads)
apply_query_fwd_kernel(const T* __restrict__ memories, const T* __restrict__ queries,
                       T* __restrict__ hidden, int64_t rows_per_n, int K, int G,
                       int64_t ctas_per_n) {
  extern __shared__ float s_q[];
  const int64_t n = blockIdx.x / ctas_per_n;
  const int64_t row_base = (blockIdx.x % ctas_per_n) * kRowsPerCta;
  for (int k = threadIdx.x; k < K; k += kThreads) s_q[k] = to_float<T>(queries[n * K + k]);
  __syncthreads();

  const int lane_in_group = threadIdx.x % G;
  const int group = threadIdx.x / G;
  const int groups = kThreads / G;
  const int64_t row_end = min(row_base + (int64_t)kRowsPerCta, rows_per_n);
  const T* mem_n = memories + n * rows_per_n * K;
  T* hid_n = hidden + n * rows_per_n;

  constexpr int UNROLL = 4;
  // The trip count is uniform over the CTA so that the shuffles below always
  // see a full warp; rows past the end are masked instead.
  const int64_t span = (int64_t)groups * UNROLL;
  const int64_t iters = (row_end - row_base + span - 1) / span;
  for (int64_t it = 0; it < iters; ++it) {
    const int64_t row = row_base + group + it * span;
    float acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u] = 0.0f;
    for (int k0 = lane_in_group * VEC; k0 < K; k0 += G * VEC) {
      float m[UNROLL][VEC];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t r = row + (int64_t)u * groups;
        if (r < row_end) {
          VecLoad<T, VEC>::load(mem_n + r * K + k0, m[u]);
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) m[u][j] = 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[u] = fmaf(m[u][j], s_q[k0 + j], acc[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float a = acc[u];
      for (int o = G >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      const int64_t r = row + (int64_t)u * groups;
      if (lane_in_group == 0 && r < row_end) hid_n[r] = from_float<T>(a);
    }
  }
}

// One CTA per n.  Thread (kx, ry) walks rows ry, ry+RG, ... of column kx.
template <typename T>
__global__ void __launch_bounds__(kThreads)
apply_query_bwd_kernel(const T* __restrict__ grad_hidden, const T* __restrict__ memories,
                       const T* __restrict__ queries, T* __restrict__ grad_memories,
                       T* __restrict__ grad_queries, int64_t rows_per_n, int K, int KT) {
  extern __shared__ float s_part[];  // [RG][KT]
  const int64_t n = blockIdx.x;
  const int kx = threadIdx.x % KT;
  const int ry = threadIdx.x / KT;
  const int RG = kThreads / KT;
  const T* dh = grad_hidden + n * rows_per_n;
  const T* mem = memories + n * rows_per_n * K;
  T* dmem = grad_memories + n * rows_per_n * K;

  for (int k0 = 0; k0 < K; k0 += KT) {
    const int k = k0 + kx;
    float acc = 0.0f;
    if (k < K) {
      const float q = to_float<T>(queries[n * K + k]);
      for (int64_t row = ry; row < rows_per_n; row += RG) {
        const float g = to_float<T>(dh[row]);
        dmem[row * K + k] = from_float<T>(g * q);
        acc = fmaf(g, to_float<T>(mem[row * K + k]), acc);
      }
    }
    s_part[ry * KT + kx] = acc;
    __syncthreads();
    if (ry == 0 && k < K) {
      float total = 0.0f;
      for (int r = 0; r < RG; ++r) total += s_part[r * KT + kx];
      grad_queries[n * K + k] = from_float<T>(total);
    }
    __syncthreads();
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int VEC>
int launch_fwd(const void* memories, const void* queries, void* hidden, int64_t N, int64_t R,
               int64_t H, int64_t K, cudaStream_t stream) {
  const int64_t rows_per_n = R * H;
  const int64_t ctas_per_n = (rows_per_n + kRowsPerCta - 1) / kRowsPerCta;
  const int64_t blocks = N * ctas_per_n;
  if (blocks > 0x7fffffffLL) return fail(GRMX_ERR_UNSUPPORTED, "apply_query: grid too large");
  int G = 1;
  while (G < 32 && G * VEC < K) G <<= 1;
  apply_query_fwd_kernel<T, VEC><<<static_cast<unsigned>(blocks), kThreads, K * sizeof(float), stream>>>(
      static_cast<const T*>(memories), static_cast<const T*>(queries), static_cast<T*>(hidden),
      rows_per_n, static_cast<int>(K), G, ctas_per_n);
  return check_launch("apply_query_fwd");
}

template <typename T>
int launch_bwd(const void* grad_hidden, const void* memories, const void* queries,
               void* grad_memories, void* grad_queries, int64_t N, int64_t R, int64_t H, int64_t K,
               cudaStream_t stream) {
  int KT = 1;
  while (KT < kThreads && KT < K) KT <<= 1;
  const size_t smem = sizeof(float) * kThreads;
  apply_query_bwd_kernel<T><<<static_cast<unsigned>(N), kThreads, smem, stream>>>(
      static_cast<const T*>(grad_hidden), static_cast<const T*>(memories),
      static_cast<const T*>(queries), static_cast<T*>(grad_memories), static_cast<T*>(grad_queries),
      R * H, static_cast<int>(K), KT);
  return check_launch("apply_query_bwd");
}

}  // namespace
}  // namespace grmx

extern "C" {

int grmx_apply_query_fwd(const void* memories, const void* queries, void* hidden, int64_t N,
                         int64_t R, int64_t H, int64_t K, int dtype, void* stream) {
  using namespace grmx;
  GRMX_REQUIRE(N >= 0 && R >= 0 && H >= 0 && K >= 0, "grmx_apply_query_fwd: negative size");
  GRMX_REQUIRE(dtype_valid(dtype), "grmx_apply_query_fwd: bad dtype code %d", dtype);
  if (N * R * H == 0) return GRMX_OK;
  GRMX_REQUIRE(memories && queries && hidden, "grmx_apply_query_fwd: NULL tensor pointer");
  GRMX_REQUIRE(K > 0 && K <= 8192, "grmx_apply_query_fwd: key dim %lld outside (0, 8192]", (long long)K);
  GRMX_REQUIRE(N <= 0x7fffffffLL, "grmx_apply_query_fwd: N too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec_ok = aligned16(memories);
  if (dtype == GRMX_F32) {
    if (vec_ok && K % 4 == 0) return launch_fwd<float, 4>(memories, queries, hidden, N, R, H, K, s);
    return launch_fwd<float, 1>(memories, queries, hidden, N, R, H, K, s);
  }
  if (dtype == GRMX_BF16) {
    if (vec_ok && K % 8 == 0) return launch_fwd<__nv_bfloat16, 8>(memories, queries, hidden, N, R, H, K, s);
    return launch_fwd<__nv_bfloat16, 1>(memories, queries, hidden, N, R, H, K, s);
  }
  if (vec_ok && K % 8 == 0) return launch_fwd<__half, 8>(memories, queries, hidden, N, R, H, K, s);
  return launch_fwd<__half, 1>(memories, queries, hidden, N, R, H, K, s);
}

int grmx_apply_query_bwd(const void* grad_hidden, const void* memories, const void* queries,
                         void* grad_memories, void* grad_queries, int64_t N, int64_t R,
                         int64_t H, int64_t K, int dtype, void* stream) {
  using namespace grmx;
  GRMX_REQUIRE(N >= 0 && R >= 0 && H >= 0 && K >= 0, "grmx_apply_query_bwd: negative size");
  GRMX_REQUIRE(dtype_valid(dtype), "grmx_apply_query_bwd: bad dtype code %d", dtype);
  if (N * K == 0) return GRMX_OK;
  GRMX_REQUIRE(queries && grad_queries, "grmx_apply_query_bwd: NULL tensor pointer");
  if (R * H > 0) {
    GRMX_REQUIRE(grad_hidden && memories && grad_memories, "grmx_apply_query_bwd: NULL tensor pointer");
  }
  GRMX_REQUIRE(N <= 0x7fffffffLL, "grmx_apply_query_bwd: N too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == GRMX_F32) {
    return launch_bwd<float>(grad_hidden, memories, queries, grad_memories, grad_queries, N, R, H, K, s);
  }
  if (dtype == GRMX_BF16) {
    return launch_bwd<__nv_bfloat16>(grad_hidden, memories, queries, grad_memories, grad_queries, N, R, H, K, s);
  }
  return launch_bwd<__half>(grad_hidden, memories, queries, grad_memories, grad_queries, N, R, H, K, s);
}

}  // extern "C"
