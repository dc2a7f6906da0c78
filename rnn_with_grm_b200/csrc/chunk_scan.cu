// C-ABI entry points of the linear-memory scan: argument checks, kernel-family
// selection, and the backward pass expressed as three scans.
#include <algorithm>
#include <cmath>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

int validate_scan(const ScanParams& p, int io_dtype, int state_dtype, int path, const char* who) {
  GRMX_REQUIRE(p.B >= 0 && p.T >= 0 && p.K > 0 && p.H > 0,
               "%s: bad sizes B=%lld T=%lld K=%lld H=%lld", who, (long long)p.B, (long long)p.T,
               (long long)p.K, (long long)p.H);
  GRMX_REQUIRE(dtype_valid(io_dtype) && dtype_valid(state_dtype), "%s: bad dtype code", who);
  GRMX_REQUIRE(state_dtype == GRMX_F32 || state_dtype == io_dtype,
               "%s: state dtype must be fp32 or equal to the io dtype", who);
  GRMX_REQUIRE(path == GRMX_PATH_AUTO || path == GRMX_PATH_FFMA || path == GRMX_PATH_TCGEN05,
               "%s: bad path code %d", who, path);
  if (p.B == 0) return GRMX_OK;
  GRMX_REQUIRE(p.memory_in != nullptr, "%s: memory_in is NULL", who);
  if (p.T > 0) {
    GRMX_REQUIRE(p.keys && p.values && p.queries && p.hidden_out, "%s: NULL tensor pointer", who);
  }
  return GRMX_OK;
}

// memory_out = scale * memory_in for the T == 0 call.
template <typename StT>
__global__ void copy_state_kernel(const StT* __restrict__ m_in, StT* __restrict__ m_out, int64_t B,
                                  int64_t H, int64_t K, int64_t rs, int64_t cs, float scale) {
  const int64_t total = B * H * K;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t k = i % K;
    const int64_t h = (i / K) % H;
    const int64_t b = i / (K * H);
    m_out[i] = from_float<StT>(to_float<StT>(m_in[b * H * K + h * rs + k * cs]) * scale);
  }
}

int copy_state(const ScanParams& p, int state_dtype, cudaStream_t stream) {
  if (p.memory_out == nullptr) return GRMX_OK;
  const int64_t total = p.B * p.H * p.K;
  if (total == 0) return GRMX_OK;
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 4096));
  const float scale = p.memory_out_scale;
  if (state_dtype == GRMX_F32) {
    copy_state_kernel<float><<<blocks, threads, 0, stream>>>(
        static_cast<const float*>(p.memory_in), static_cast<float*>(p.memory_out), p.B, p.H, p.K,
        p.m_row_stride, p.m_col_stride, scale);
  } else if (state_dtype == GRMX_BF16) {
    copy_state_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p.memory_in), static_cast<__nv_bfloat16*>(p.memory_out),
        p.B, p.H, p.K, p.m_row_stride, p.m_col_stride, scale);
  } else {
    copy_state_kernel<__half><<<blocks, threads, 0, stream>>>(
        static_cast<const __half*>(p.memory_in), static_cast<__half*>(p.memory_out), p.B, p.H, p.K,
        p.m_row_stride, p.m_col_stride, scale);
  }
  return check_launch("copy_state");
}

int run_scan(const ScanParams& p, int io_dtype, int state_dtype, int path, cudaStream_t stream,
             const char* who, void* scratch = nullptr, int64_t scratch_bytes = 0) {
  int rc = validate_scan(p, io_dtype, state_dtype, path, who);
  if (rc != GRMX_OK) return rc;
  if (p.B == 0) return GRMX_OK;
  if (p.T == 0) return copy_state(p, state_dtype, stream);

  const char* why = "";
  const bool tc_ok = scan_tcgen05_supported(p, io_dtype, state_dtype, &why);
  if (path == GRMX_PATH_TCGEN05 && !tc_ok) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: tcgen05 path unavailable: %s", who, why);
  }
  if (tc_ok && path != GRMX_PATH_FFMA) {
    if (scratch != nullptr && scan_tcgen05_split_scratch_bytes(p) > 0) {
      return launch_scan_tcgen05_split(p, scratch, scratch_bytes, stream);
    }
    return launch_scan_tcgen05(p, stream);
  }
  return launch_scan_ffma(p, io_dtype, state_dtype, stream);
}

}  // namespace
}  // namespace grmx

extern "C" {

int grmx_linear_scan(const void* keys, const void* values, const void* queries,
                     const void* memory_in, int64_t m_row_stride, int64_t m_col_stride,
                     void* hidden_out, void* memory_out, int64_t B, int64_t T, int64_t K,
                     int64_t H, float decay, float update_coeff, float hidden_scale,
                     float memory_out_scale, int reverse, int first_step_no_decay,
                     int io_dtype, int state_dtype, int path, void* stream) {
  grmx::ScanParams p;
  p.keys = keys; p.values = values; p.queries = queries; p.memory_in = memory_in;
  p.hidden_out = hidden_out; p.memory_out = memory_out;
  p.B = B; p.T = T; p.K = K; p.H = H;
  p.m_row_stride = m_row_stride; p.m_col_stride = m_col_stride;
  p.decay = decay; p.update_coeff = update_coeff; p.hidden_scale = hidden_scale;
  p.memory_out_scale = memory_out_scale;
  p.reverse = reverse ? 1 : 0; p.first_step_no_decay = first_step_no_decay ? 1 : 0;
  return grmx::run_scan(p, io_dtype, state_dtype, path, static_cast<cudaStream_t>(stream),
                        "grmx_linear_scan");
}

int grmx_chunk_scan_fwd(const void* keys, const void* values, const void* queries,
                        const void* memory_in, void* hidden_out, void* memory_out,
                        int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                        int io_dtype, int state_dtype, int path, void* stream) {
  if (K <= 0) return grmx::fail(GRMX_ERR_ARG, "grmx_chunk_scan_fwd: K must be positive");
  if (B > 0 && memory_out == nullptr) {
    return grmx::fail(GRMX_ERR_ARG, "grmx_chunk_scan_fwd: memory_out is NULL");
  }
  const float beta = 1.0f - decay;
  const float inv_scale = 1.0f / sqrtf(static_cast<float>(K));
  grmx::ScanParams p;
  p.keys = keys; p.values = values; p.queries = queries; p.memory_in = memory_in;
  p.hidden_out = hidden_out; p.memory_out = memory_out;
  p.B = B; p.T = T; p.K = K; p.H = H;
  p.m_row_stride = K; p.m_col_stride = 1;
  p.decay = decay; p.update_coeff = beta * inv_scale; p.hidden_scale = 1.0f;
  p.memory_out_scale = 1.0f; p.reverse = 0; p.first_step_no_decay = 0;
  return grmx::run_scan(p, io_dtype, state_dtype, path, static_cast<cudaStream_t>(stream),
                        "grmx_chunk_scan_fwd");
}

int grmx_chunk_scan_fwd_segments(const void* keys, const void* values, const void* queries,
                                 const void* memory_in, void* hidden_out, void* memory_out, float* archive,
                                 int64_t capacity, int64_t first_slot, int64_t segment_tokens, int64_t B,
                                 int64_t T, int64_t K, int64_t H, float decay, int io_dtype, int state_dtype,
                                 void* stream) {
  const char* who = "grmx_chunk_scan_fwd_segments";
  if (K <= 0) return grmx::fail(GRMX_ERR_ARG, "%s: K must be positive", who);
  if (B > 0 && (memory_out == nullptr || archive == nullptr)) {
    return grmx::fail(GRMX_ERR_ARG, "%s: memory_out or archive is NULL", who);
  }
  if (segment_tokens <= 0 || segment_tokens % 128 != 0 || T % segment_tokens != 0) {
    return grmx::fail(GRMX_ERR_UNSUPPORTED, "%s: segments must be whole multiples of 128 tokens and divide T", who);
  }
  const int64_t segments = T / segment_tokens;
  if (first_slot < 0 || capacity < 0 || first_slot + segments > capacity) {
    return grmx::fail(GRMX_ERR_ARG, "%s: slots [%lld, %lld) do not fit an archive of %lld", who, (long long)first_slot,
                      (long long)(first_slot + segments), (long long)capacity);
  }
  if ((reinterpret_cast<uintptr_t>(archive) & 15u) != 0) {
    return grmx::fail(GRMX_ERR_ARG, "%s: archive must be 16-byte aligned", who);
  }
  grmx::ScanParams p;
  p.keys = keys; p.values = values; p.queries = queries; p.memory_in = memory_in;
  p.hidden_out = hidden_out; p.memory_out = memory_out;
  p.B = B; p.T = T; p.K = K; p.H = H;
  p.m_row_stride = K; p.m_col_stride = 1;
  p.decay = decay; p.update_coeff = (1.0f - decay) * (1.0f / sqrtf(static_cast<float>(K)));
  p.hidden_scale = 1.0f; p.memory_out_scale = 1.0f; p.reverse = 0; p.first_step_no_decay = 0;
  p.snapshots = archive + first_slot * H * K;
  p.snap_batch_stride = capacity * H * K;
  p.snap_stride = H * K;
  p.snap_chunks = static_cast<int>(segment_tokens / 128);
  const int rc = grmx::validate_scan(p, io_dtype, state_dtype, GRMX_PATH_TCGEN05, who);
  if (rc != GRMX_OK) return rc;
  if (B == 0 || T == 0) return GRMX_OK;
  const char* why = "";
  if (!grmx::scan_tcgen05_supported(p, io_dtype, state_dtype, &why) || !grmx::scan_tcgen05_pipe_supported(p)) {
    return grmx::fail(GRMX_ERR_UNSUPPORTED, "%s: needs the tensor-core scan: %s", who, why);
  }
  return grmx::launch_scan_tcgen05(p, static_cast<cudaStream_t>(stream));
}

int64_t grmx_chunk_scan_scratch_bytes(int64_t B, int64_t T, int64_t K, int64_t H, int io_dtype,
                                      int state_dtype) {
  if (B <= 0 || T <= 0 || K <= 0 || H <= 0) return 0;
  if (io_dtype != GRMX_BF16 || state_dtype != GRMX_F32) return 0;
  grmx::ScanParams p = {};
  p.B = B; p.T = T; p.K = K; p.H = H;
  return grmx::scan_tcgen05_split_scratch_bytes(p);
}

int grmx_chunk_scan_fwd_ws(const void* keys, const void* values, const void* queries,
                           const void* memory_in, void* hidden_out, void* memory_out,
                           int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                           int io_dtype, int state_dtype, int path, void* scratch,
                           int64_t scratch_bytes, void* stream) {
  if (K <= 0) return grmx::fail(GRMX_ERR_ARG, "grmx_chunk_scan_fwd_ws: K must be positive");
  if (B > 0 && memory_out == nullptr) {
    return grmx::fail(GRMX_ERR_ARG, "grmx_chunk_scan_fwd_ws: memory_out is NULL");
  }
  if (scratch_bytes < 0) return grmx::fail(GRMX_ERR_ARG, "grmx_chunk_scan_fwd_ws: negative scratch size");
  grmx::ScanParams p;
  p.keys = keys; p.values = values; p.queries = queries; p.memory_in = memory_in;
  p.hidden_out = hidden_out; p.memory_out = memory_out;
  p.B = B; p.T = T; p.K = K; p.H = H;
  p.m_row_stride = K; p.m_col_stride = 1;
  p.decay = decay; p.update_coeff = (1.0f - decay) * (1.0f / sqrtf(static_cast<float>(K)));
  p.hidden_scale = 1.0f; p.memory_out_scale = 1.0f; p.reverse = 0; p.first_step_no_decay = 0;
  return grmx::run_scan(p, io_dtype, state_dtype, path, static_cast<cudaStream_t>(stream),
                        "grmx_chunk_scan_fwd_ws", scratch, scratch_bytes);
}

int grmx_chunk_scan_bwd(const void* grad_hidden, const void* grad_memory_out,
                        const void* keys, const void* values, const void* queries,
                        const void* memory_in, void* grad_keys, void* grad_values,
                        void* grad_queries, void* grad_memory, int64_t B, int64_t T,
                        int64_t K, int64_t H, float decay, int io_dtype, int state_dtype,
                        int path, void* stream) {
  using grmx::ScanParams;
  const char* who = "grmx_chunk_scan_bwd";
  if (K <= 0 || H <= 0) return grmx::fail(GRMX_ERR_ARG, "%s: K and H must be positive", who);
  if (B > 0 && (grad_memory_out == nullptr || memory_in == nullptr || grad_memory == nullptr)) {
    return grmx::fail(GRMX_ERR_ARG, "%s: NULL state pointer", who);
  }
  if (B > 0 && T > 0 &&
      !(grad_hidden && keys && values && queries && grad_keys && grad_values && grad_queries)) {
    return grmx::fail(GRMX_ERR_ARG, "%s: NULL tensor pointer", who);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float coeff = (1.0f - decay) / sqrtf(static_cast<float>(K));

  // With A_t = decay*A_{t+1} + dh_t q_t^T and A_{T-1} = dM_out + dh q^T
  // (the total gradient reaching M_t):
  //   dq_t = M_t^T dh_t          forward scan on the transposed state
  //   dv_t = coeff * A_t   k_t   reverse scan, state A
  //   dk_t = coeff * A_t^T v_t   reverse scan, state A^T
  //   dM_0 = decay * A_0
  ScanParams dq;
  dq.keys = values; dq.values = keys; dq.queries = grad_hidden; dq.memory_in = memory_in;
  dq.hidden_out = grad_queries; dq.memory_out = nullptr;
  dq.B = B; dq.T = T; dq.K = H; dq.H = K;
  dq.m_row_stride = 1; dq.m_col_stride = K;
  dq.decay = decay; dq.update_coeff = coeff; dq.hidden_scale = 1.0f; dq.memory_out_scale = 1.0f;
  dq.reverse = 0; dq.first_step_no_decay = 0;

  ScanParams dv;
  dv.keys = queries; dv.values = grad_hidden; dv.queries = keys; dv.memory_in = grad_memory_out;
  dv.hidden_out = grad_values; dv.memory_out = grad_memory;
  dv.B = B; dv.T = T; dv.K = K; dv.H = H;
  dv.m_row_stride = K; dv.m_col_stride = 1;
  dv.decay = decay; dv.update_coeff = 1.0f; dv.hidden_scale = coeff; dv.memory_out_scale = decay;
  dv.reverse = 1; dv.first_step_no_decay = 1;

  ScanParams dk;
  dk.keys = grad_hidden; dk.values = queries; dk.queries = values; dk.memory_in = grad_memory_out;
  dk.hidden_out = grad_keys; dk.memory_out = nullptr;
  dk.B = B; dk.T = T; dk.K = H; dk.H = K;
  dk.m_row_stride = 1; dk.m_col_stride = K;
  dk.decay = decay; dk.update_coeff = 1.0f; dk.hidden_scale = coeff; dk.memory_out_scale = 1.0f;
  dk.reverse = 1; dk.first_step_no_decay = 1;

  if (T == 0) {
    // hidden is empty and memory_out == memory_in, so dM_0 = dM_out.
    dv.memory_out_scale = 1.0f;
    return grmx::run_scan(dv, io_dtype, state_dtype, path, s, who);
  }
  int rc = grmx::run_scan(dq, io_dtype, state_dtype, path, s, who);
  if (rc != GRMX_OK) return rc;
  rc = grmx::run_scan(dv, io_dtype, state_dtype, path, s, who);
  if (rc != GRMX_OK) return rc;
  return grmx::run_scan(dk, io_dtype, state_dtype, path, s, who);
}

int grmx_selftest_bounded_wait(uint32_t wait_limit, void* stream) {
  if (wait_limit == 0 || wait_limit > (1u << 24)) {
    return grmx::fail(GRMX_ERR_ARG, "grmx_selftest_bounded_wait: wait_limit must be in [1, 2^24]");
  }
  if (!grmx::tc::device_is_sm100()) {
    return grmx::fail(GRMX_ERR_UNSUPPORTED, "grmx_selftest_bounded_wait: needs an sm_100 device");
  }
  return grmx::tc::launch_bounded_wait_selftest(wait_limit, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
