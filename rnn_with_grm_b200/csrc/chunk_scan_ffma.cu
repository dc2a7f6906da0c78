// fp32 CUDA-core kernel of the linear-memory scan (exact mode).
//
// One CTA owns 32 rows of the state of one batch row for the whole call.
// Eight lanes share a state row: each holds KS of its key columns in
// registers, so a row's dot product with q needs three shuffles.  Tokens are
// staged through shared memory sixteen at a time (q and k converted to fp32
// once per CTA), which costs two barriers per sixteen tokens.
//
// Follows the sequential definition of the update
// (grm/csrc/grm_cuda.cpp:67-83): M <- decay*M + coeff * v k^T, h = M q.
#include "scan.cuh"

namespace grmx {
namespace {

constexpr int kRowsPerCta = 32;
constexpr int kLanesPerRow = 8;
constexpr int kThreads = kRowsPerCta * kLanesPerRow;
constexpr int kTokenBlock = 16;

template <typename IoT, typename StT, int KS>
__global__ void __launch_bounds__(kThreads) linear_scan_ffma_kernel(ScanParams p) {
  constexpr int VEC = KS >= 4 ? 4 : KS;
  constexpr int NV = KS / VEC;
  constexpr int KPAD = kLanesPerRow * KS;

  __shared__ __align__(16) float s_k[kTokenBlock][KPAD];
  __shared__ __align__(16) float s_q[kTokenBlock][KPAD];
  __shared__ float s_v[kTokenBlock][kRowsPerCta];
  __shared__ float s_o[kTokenBlock][kRowsPerCta];

  const int tid = threadIdx.x;
  const int slice = tid & (kLanesPerRow - 1);
  const int row_local = tid >> 3;
  const int64_t tiles = (p.H + kRowsPerCta - 1) / kRowsPerCta;
  const int64_t b = blockIdx.x / tiles;
  const int64_t row0 = (blockIdx.x % tiles) * kRowsPerCta;
  const int64_t row = row0 + row_local;
  const bool row_ok = row < p.H;
  const int K = static_cast<int>(p.K);

  const IoT* keys = static_cast<const IoT*>(p.keys) + b * p.T * p.K;
  const IoT* queries = static_cast<const IoT*>(p.queries) + b * p.T * p.K;
  const IoT* values = static_cast<const IoT*>(p.values) + b * p.T * p.H;
  IoT* hidden = static_cast<IoT*>(p.hidden_out) + b * p.T * p.H;
  const StT* m_in = static_cast<const StT*>(p.memory_in) + b * p.H * p.K;

  float m[KS];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int k = VEC * (slice + kLanesPerRow * i) + j;
      m[i * VEC + j] = (row_ok && k < K)
                           ? to_float<StT>(m_in[row * p.m_row_stride + k * p.m_col_stride])
                           : 0.0f;
    }
  }

  const float decay = p.decay;
  const float coeff = p.update_coeff;
  const int64_t T = p.T;

  for (int64_t step0 = 0; step0 < T; step0 += kTokenBlock) {
    const int n_tok = static_cast<int>(T - step0 < kTokenBlock ? T - step0 : kTokenBlock);

    for (int idx = tid; idx < kTokenBlock * KPAD; idx += kThreads) {
      const int tt = idx / KPAD;
      const int k = idx - tt * KPAD;
      float kv = 0.0f, qv = 0.0f;
      if (tt < n_tok && k < K) {
        const int64_t t = p.reverse ? (T - 1 - (step0 + tt)) : (step0 + tt);
        kv = to_float<IoT>(keys[t * p.K + k]);
        qv = to_float<IoT>(queries[t * p.K + k]);
      }
      s_k[tt][k] = kv;
      s_q[tt][k] = qv;
    }
    for (int idx = tid; idx < kTokenBlock * kRowsPerCta; idx += kThreads) {
      const int tt = idx / kRowsPerCta;
      const int r = idx - tt * kRowsPerCta;
      float vv = 0.0f;
      if (tt < n_tok && row0 + r < p.H) {
        const int64_t t = p.reverse ? (T - 1 - (step0 + tt)) : (step0 + tt);
        vv = to_float<IoT>(values[t * p.H + row0 + r]);
      }
      s_v[tt][r] = vv;
    }
    __syncthreads();

    for (int tt = 0; tt < n_tok; ++tt) {
      const float a = (p.first_step_no_decay && step0 + tt == 0) ? 1.0f : decay;
      const float vc = coeff * s_v[tt][row_local];
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k0 = VEC * (slice + kLanesPerRow * i);
        float kk[VEC], qq[VEC];
        if constexpr (VEC == 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&s_k[tt][k0]);
          const float4 q4 = *reinterpret_cast<const float4*>(&s_q[tt][k0]);
          kk[0] = k4.x; kk[1] = k4.y; kk[2] = k4.z; kk[3] = k4.w;
          qq[0] = q4.x; qq[1] = q4.y; qq[2] = q4.z; qq[3] = q4.w;
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            kk[j] = s_k[tt][k0 + j];
            qq[j] = s_q[tt][k0 + j];
          }
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const float next = fmaf(a, m[i * VEC + j], vc * kk[j]);
          m[i * VEC + j] = next;
          acc = fmaf(next, qq[j], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (slice == 0) s_o[tt][row_local] = acc * p.hidden_scale;
    }
    __syncthreads();

    for (int idx = tid; idx < kTokenBlock * kRowsPerCta; idx += kThreads) {
      const int tt = idx / kRowsPerCta;
      const int r = idx - tt * kRowsPerCta;
      if (tt < n_tok && row0 + r < p.H) {
        const int64_t t = p.reverse ? (T - 1 - (step0 + tt)) : (step0 + tt);
        hidden[t * p.H + row0 + r] = from_float<IoT>(s_o[tt][r]);
      }
    }
    // No barrier here: the staging buffers were last read before the barrier
    // above, and s_o is next written only after the next staging barrier.
  }

  if (p.memory_out != nullptr && row_ok) {
    StT* m_out = static_cast<StT*>(p.memory_out) + b * p.H * p.K + row * p.K;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const int k = VEC * (slice + kLanesPerRow * i) + j;
        if (k < K) m_out[k] = from_float<StT>(m[i * VEC + j] * p.memory_out_scale);
      }
    }
  }
}

template <typename IoT, typename StT>
int launch_for_types(const ScanParams& p, cudaStream_t stream) {
  const int64_t tiles = (p.H + kRowsPerCta - 1) / kRowsPerCta;
  const int64_t blocks = p.B * tiles;
  if (blocks <= 0) return GRMX_OK;
  if (blocks > 0x7fffffffLL) return fail(GRMX_ERR_UNSUPPORTED, "linear scan: grid too large");
  const dim3 grid(static_cast<unsigned>(blocks));
  const int K = static_cast<int>(p.K);
#define GRMX_SCAN_CASE(KS_)                                                           \
  if (K <= kLanesPerRow * KS_) {                                                      \
    linear_scan_ffma_kernel<IoT, StT, KS_><<<grid, kThreads, 0, stream>>>(p);         \
    return check_launch("linear_scan_ffma");                                          \
  }
  GRMX_SCAN_CASE(1)
  GRMX_SCAN_CASE(2)
  GRMX_SCAN_CASE(4)
  GRMX_SCAN_CASE(8)
  GRMX_SCAN_CASE(16)
  GRMX_SCAN_CASE(32)
#undef GRMX_SCAN_CASE
  return fail(GRMX_ERR_UNSUPPORTED, "linear scan: key dim %d exceeds 256", K);
}

}  // namespace

int launch_scan_ffma(const ScanParams& p, int io_dtype, int state_dtype, cudaStream_t stream) {
  if (io_dtype == GRMX_F32 && state_dtype == GRMX_F32) {
    return launch_for_types<float, float>(p, stream);
  }
  if (io_dtype == GRMX_BF16 && state_dtype == GRMX_F32) {
    return launch_for_types<__nv_bfloat16, float>(p, stream);
  }
  if (io_dtype == GRMX_BF16 && state_dtype == GRMX_BF16) {
    return launch_for_types<__nv_bfloat16, __nv_bfloat16>(p, stream);
  }
  if (io_dtype == GRMX_F16 && state_dtype == GRMX_F32) {
    return launch_for_types<__half, float>(p, stream);
  }
  if (io_dtype == GRMX_F16 && state_dtype == GRMX_F16) {
    return launch_for_types<__half, __half>(p, stream);
  }
  return fail(GRMX_ERR_UNSUPPORTED,
              "linear scan: state dtype must be fp32 or equal to the io dtype (io=%d state=%d)",
              io_dtype, state_dtype);
}

}  // namespace grmx
