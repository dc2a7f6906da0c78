// PyTorch face of the engine: registers torch.ops.grm_cuda.* with the schemas
// of the reference extension (grm/csrc/bindings.cpp:5-11) for the CUDA
// dispatch key, plus torch.ops.grmx.* for the calls the reference has no op
// for.  Every kernel is reached through the C ABI of grmx.h; this file only
// checks shapes, allocates outputs from the caching allocator and passes the
// current stream.  There is no CPU registration: a CPU tensor fails loudly in
// the dispatcher.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <atomic>
#include <tuple>

#include "grmx.h"

namespace {

std::atomic<int> g_scan_path{GRMX_PATH_AUTO};

int dtype_code(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kFloat: return GRMX_F32;
    case at::kBFloat16: return GRMX_BF16;
    case at::kHalf: return GRMX_F16;
    default: TORCH_CHECK(false, "grm_cuda: ", what, " has unsupported dtype ", t, " (float32, bfloat16, float16)");
  }
  return -1;
}

void check_status(int rc) { TORCH_CHECK(rc == GRMX_OK, "grm_cuda: ", grmx_last_error()); }

void* current_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

void require_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "grm_cuda: ", name, " must be a CUDA tensor (this engine has no CPU path)");
}

// shape contract of the reference: grm/csrc/grm_cuda.cpp:13-27
void check_chunk_inputs(const at::Tensor& keys, const at::Tensor& values, const at::Tensor& queries,
                        const at::Tensor& memory) {
  TORCH_CHECK(keys.dim() == 3, "keys must have shape [B, T, K]");
  TORCH_CHECK(values.dim() == 3, "values must have shape [B, T, H]");
  TORCH_CHECK(queries.dim() == 3, "queries must have shape [B, T, K]");
  TORCH_CHECK(memory.dim() == 3, "memory must have shape [B, H, K]");
  TORCH_CHECK(keys.sizes().slice(0, 2) == values.sizes().slice(0, 2), "keys and values batch/time dims must match");
  TORCH_CHECK(keys.sizes() == queries.sizes(), "keys and queries must have the same shape");
  TORCH_CHECK(values.size(0) == memory.size(0), "memory batch dim must match values batch dim");
  TORCH_CHECK(values.size(2) == memory.size(1), "memory hidden dim must match values hidden dim");
  TORCH_CHECK(keys.size(2) == memory.size(2), "memory key dim must match keys key dim");
  require_cuda(keys, "keys");
  require_cuda(values, "values");
  require_cuda(queries, "queries");
  require_cuda(memory, "memory");
  TORCH_CHECK(keys.scalar_type() == values.scalar_type() && keys.scalar_type() == queries.scalar_type(),
              "grm_cuda: keys, values and queries must share one dtype");
  TORCH_CHECK(memory.scalar_type() == at::kFloat || memory.scalar_type() == keys.scalar_type(),
              "grm_cuda: memory must be float32 or have the dtype of keys");
}

// grm/csrc/grm_cuda.cpp:29-42
void check_apply_query_inputs(const at::Tensor& memories, const at::Tensor& queries) {
  TORCH_CHECK(memories.dim() == 4 || memories.dim() == 5, "memories must have shape [B, R, H, K] or [B, Q, R, H, K]");
  if (memories.dim() == 4) {
    TORCH_CHECK(queries.dim() == 2, "queries must have shape [B, K] when memories rank is 4");
    TORCH_CHECK(memories.size(0) == queries.size(0), "batch dim mismatch between memories and queries");
    TORCH_CHECK(memories.size(3) == queries.size(1), "key dim mismatch between memories and queries");
  } else {
    TORCH_CHECK(queries.dim() == 3, "queries must have shape [B, Q, K] when memories rank is 5");
    TORCH_CHECK(memories.size(0) == queries.size(0), "batch dim mismatch between memories and queries");
    TORCH_CHECK(memories.size(1) == queries.size(1), "query dim mismatch between memories and queries");
    TORCH_CHECK(memories.size(4) == queries.size(2), "key dim mismatch between memories and queries");
  }
  require_cuda(memories, "memories");
  require_cuda(queries, "queries");
  TORCH_CHECK(memories.scalar_type() == queries.scalar_type(), "grm_cuda: memories and queries must share one dtype");
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> chunk_update_forward_cuda(
    const at::Tensor& keys, const at::Tensor& values, const at::Tensor& queries,
    const at::Tensor& memory, double memory_decay) {
  check_chunk_inputs(keys, values, queries, memory);
  c10::cuda::CUDAGuard guard(keys.device());
  auto k = keys.contiguous();
  auto v = values.contiguous();
  auto q = queries.contiguous();
  auto m = memory.contiguous();
  const int64_t B = k.size(0), T = k.size(1), K = k.size(2), H = v.size(2);
  auto aux = at::empty({0}, m.options());
  if (T == 0) {
    return {at::zeros({B, 0, H}, v.options()), m, aux};
  }
  auto hidden = at::empty({B, T, H}, v.options());
  auto memory_out = at::empty_like(m);
  const int io = dtype_code(k.scalar_type(), "keys");
  const int st = dtype_code(m.scalar_type(), "memory");
  // few rows, many tokens: give the kernel a workspace so it can cut the rows along T
  // Few rows and many tokens: the scan is cut along T.  Up to four pieces the library does that in one
  // launch without a workspace; the two-kernel form over a workspace pays when the call allows more
  // pieces than that, i.e. when the workspace holds five or more piece states per row.
  int64_t scratch_bytes = g_scan_path.load() == GRMX_PATH_FFMA ? 0 : grmx_chunk_scan_scratch_bytes(B, T, K, H, io, st);
  if (scratch_bytes < 5 * B * H * K * static_cast<int64_t>(sizeof(float))) scratch_bytes = 0;
  at::Tensor scratch;
  if (scratch_bytes > 0) scratch = at::empty({scratch_bytes}, k.options().dtype(at::kByte));
  check_status(grmx_chunk_scan_fwd_ws(k.data_ptr(), v.data_ptr(), q.data_ptr(), m.data_ptr(),
                                      hidden.data_ptr(), memory_out.data_ptr(), B, T, K, H,
                                      static_cast<float>(memory_decay), io, st, g_scan_path.load(),
                                      scratch_bytes > 0 ? scratch.data_ptr() : nullptr, scratch_bytes,
                                      current_stream()));
  return {hidden, memory_out, aux};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> chunk_update_backward_cuda(
    const at::Tensor& grad_hidden, const at::Tensor& grad_memory_out, const at::Tensor& keys,
    const at::Tensor& values, const at::Tensor& queries, const at::Tensor& memory,
    const at::Tensor& aux, double memory_decay) {
  (void)aux;
  check_chunk_inputs(keys, values, queries, memory);
  require_cuda(grad_hidden, "grad_hidden");
  require_cuda(grad_memory_out, "grad_memory_out");
  TORCH_CHECK(grad_hidden.sizes() == values.sizes(), "grad_hidden must have the shape of values");
  TORCH_CHECK(grad_memory_out.sizes() == memory.sizes(), "grad_memory_out must have the shape of memory");
  c10::cuda::CUDAGuard guard(keys.device());
  auto k = keys.contiguous();
  auto v = values.contiguous();
  auto q = queries.contiguous();
  auto m = memory.contiguous();
  auto gh = grad_hidden.to(v.scalar_type()).contiguous();
  auto gm = grad_memory_out.to(m.scalar_type()).contiguous();
  const int64_t B = k.size(0), T = k.size(1), K = k.size(2), H = v.size(2);
  auto grad_k = at::empty_like(k);
  auto grad_v = at::empty_like(v);
  auto grad_q = at::empty_like(q);
  auto grad_m = at::empty_like(m);
  check_status(grmx_chunk_scan_bwd(gh.data_ptr(), gm.data_ptr(), k.data_ptr(), v.data_ptr(), q.data_ptr(),
                                   m.data_ptr(), grad_k.data_ptr(), grad_v.data_ptr(), grad_q.data_ptr(),
                                   grad_m.data_ptr(), B, T, K, H, static_cast<float>(memory_decay),
                                   dtype_code(k.scalar_type(), "keys"), dtype_code(m.scalar_type(), "memory"),
                                   g_scan_path.load(), current_stream()));
  return {grad_k, grad_v, grad_q, grad_m};
}

at::Tensor apply_query_forward_cuda(const at::Tensor& memories, const at::Tensor& queries) {
  check_apply_query_inputs(memories, queries);
  c10::cuda::CUDAGuard guard(memories.device());
  auto mem = memories.contiguous();
  auto q = queries.contiguous();
  const bool rank5 = mem.dim() == 5;
  const int64_t N = rank5 ? mem.size(0) * mem.size(1) : mem.size(0);
  const int64_t R = mem.size(rank5 ? 2 : 1), H = mem.size(rank5 ? 3 : 2), K = mem.size(rank5 ? 4 : 3);
  at::Tensor hidden = rank5 ? at::empty({mem.size(0), mem.size(1), R, H}, mem.options())
                            : at::empty({mem.size(0), R, H}, mem.options());
  if (K == 0) hidden.zero_();
  check_status(grmx_apply_query_fwd(mem.data_ptr(), q.data_ptr(), hidden.data_ptr(), N, R, H, K,
                                    dtype_code(mem.scalar_type(), "memories"), current_stream()));
  return hidden;
}

std::tuple<at::Tensor, at::Tensor> apply_query_backward_cuda(const at::Tensor& grad_hidden,
                                                             const at::Tensor& memories,
                                                             const at::Tensor& queries) {
  check_apply_query_inputs(memories, queries);
  require_cuda(grad_hidden, "grad_hidden");
  c10::cuda::CUDAGuard guard(memories.device());
  auto mem = memories.contiguous();
  auto q = queries.contiguous();
  auto gh = grad_hidden.to(mem.scalar_type()).contiguous();
  const bool rank5 = mem.dim() == 5;
  const int64_t N = rank5 ? mem.size(0) * mem.size(1) : mem.size(0);
  const int64_t R = mem.size(rank5 ? 2 : 1), H = mem.size(rank5 ? 3 : 2), K = mem.size(rank5 ? 4 : 3);
  TORCH_CHECK(gh.numel() == N * R * H, "grad_hidden has the wrong number of elements");
  auto grad_mem = at::empty_like(mem);
  auto grad_q = at::empty_like(q);
  check_status(grmx_apply_query_bwd(gh.data_ptr(), mem.data_ptr(), q.data_ptr(), grad_mem.data_ptr(),
                                    grad_q.data_ptr(), N, R, H, K, dtype_code(mem.scalar_type(), "memories"),
                                    current_stream()));
  return {grad_mem, grad_q};
}

// grm/csrc/grm_cuda.cpp:156-161
at::Tensor batched_memory_gather_cuda(const at::Tensor& memories_per_batch, const at::Tensor& topk_indices) {
  TORCH_CHECK(memories_per_batch.dim() == 4, "memories_per_batch must have shape [B, S, H, K]");
  TORCH_CHECK(topk_indices.dim() == 2 || topk_indices.dim() == 3, "topk_indices must have shape [B, R] or [B, Q, R]");
  TORCH_CHECK(memories_per_batch.size(0) == topk_indices.size(0),
              "batch dim mismatch between memories_per_batch and topk_indices");
  require_cuda(memories_per_batch, "memories_per_batch");
  require_cuda(topk_indices, "topk_indices");
  c10::cuda::CUDAGuard guard(memories_per_batch.device());
  auto mem = memories_per_batch.contiguous();
  auto idx = topk_indices.toType(at::kLong).contiguous();
  const int64_t B = mem.size(0), S = mem.size(1), H = mem.size(2), K = mem.size(3);
  dtype_code(mem.scalar_type(), "memories_per_batch");
  std::vector<int64_t> shape(idx.sizes().begin(), idx.sizes().end());
  shape.push_back(H);
  shape.push_back(K);
  auto out = at::empty(shape, mem.options());
  const int64_t J = B > 0 ? idx.numel() / B : 0;
  check_status(grmx_batched_gather(mem.data_ptr(), idx.data_ptr<int64_t>(), out.data_ptr(), B, S, J, H * K,
                                   static_cast<int>(mem.element_size()), current_stream()));
  return out;
}

// ---- calls with no counterpart op in the reference (namespace grmx) ----

std::tuple<at::Tensor, at::Tensor> linear_scan_cuda(const at::Tensor& keys, const at::Tensor& values,
                                                    const at::Tensor& queries, const at::Tensor& memory,
                                                    double decay, double update_coeff, double hidden_scale,
                                                    double memory_out_scale, bool reverse,
                                                    bool first_step_no_decay, int64_t path) {
  check_chunk_inputs(keys, values, queries, memory);
  c10::cuda::CUDAGuard guard(keys.device());
  auto k = keys.contiguous();
  auto v = values.contiguous();
  auto q = queries.contiguous();
  auto m = memory.contiguous();
  const int64_t B = k.size(0), T = k.size(1), K = k.size(2), H = v.size(2);
  auto hidden = at::empty({B, T, H}, v.options());
  auto memory_out = at::empty_like(m);
  check_status(grmx_linear_scan(k.data_ptr(), v.data_ptr(), q.data_ptr(), m.data_ptr(), K, 1,
                                hidden.data_ptr(), memory_out.data_ptr(), B, T, K, H,
                                static_cast<float>(decay), static_cast<float>(update_coeff),
                                static_cast<float>(hidden_scale), static_cast<float>(memory_out_scale),
                                reverse ? 1 : 0, first_step_no_decay ? 1 : 0,
                                dtype_code(k.scalar_type(), "keys"), dtype_code(m.scalar_type(), "memory"),
                                static_cast<int>(path), current_stream()));
  return {hidden, memory_out};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> topk_route_cuda(const at::Tensor& queries,
                                                               const at::Tensor& keys,
                                                               const c10::optional<at::Tensor>& visible,
                                                               int64_t top_k, double scale,
                                                               double temperature, bool return_scores) {
  TORCH_CHECK(queries.dim() == 3, "queries must have shape [B, Q, D]");
  TORCH_CHECK(keys.dim() == 3, "keys must have shape [B, S, D]");
  TORCH_CHECK(queries.size(0) == keys.size(0), "batch dim mismatch between queries and keys");
  TORCH_CHECK(queries.size(2) == keys.size(2), "feature dim mismatch between queries and keys");
  require_cuda(queries, "queries");
  require_cuda(keys, "keys");
  c10::cuda::CUDAGuard guard(queries.device());
  auto k = keys.to(at::kFloat).contiguous();
  const int64_t B = queries.size(0), Q = queries.size(1), D = queries.size(2), S = k.size(1);
  // bf16 queries of the per-token shapes are read as they are (grmx_topk_route_bf16q); everything else
  // is widened to fp32 first
  at::Tensor q = queries.contiguous();
  const bool lowp = q.scalar_type() == at::kBFloat16 && S >= 1 && S <= 16 && Q >= 64 && D >= 8 && D % 8 == 0 &&
                    D <= 1024 && B <= 65535 && (reinterpret_cast<uintptr_t>(q.data_ptr()) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(k.data_ptr()) & 15u) == 0;
  if (!lowp) q = q.to(at::kFloat);
  at::Tensor vis;
  const int32_t* vis_ptr = nullptr;
  if (visible.has_value() && visible->defined()) {
    require_cuda(*visible, "visible");
    TORCH_CHECK(visible->numel() == Q, "visible must hold one count per query");
    vis = visible->to(at::kInt).contiguous();
    vis_ptr = vis.data_ptr<int32_t>();
  }
  auto idx = at::empty({B, Q, top_k}, k.options().dtype(at::kLong));
  auto gates = at::empty({B, Q, top_k}, k.options());
  at::Tensor scores = return_scores ? at::empty({B, Q, S}, k.options()) : at::empty({0}, k.options());
  if (lowp) {
    check_status(grmx_topk_route_bf16q(q.data_ptr(), k.data_ptr<float>(), vis_ptr, B, Q, S, D,
                                       static_cast<int>(top_k), static_cast<float>(scale),
                                       static_cast<float>(temperature), idx.data_ptr<int64_t>(),
                                       gates.data_ptr<float>(), return_scores ? scores.data_ptr<float>() : nullptr,
                                       current_stream()));
    return {gates, idx, scores};
  }
  check_status(grmx_topk_route(q.data_ptr<float>(), k.data_ptr<float>(), vis_ptr, B, Q, S, D,
                               static_cast<int>(top_k), static_cast<float>(scale),
                               static_cast<float>(temperature), idx.data_ptr<int64_t>(),
                               gates.data_ptr<float>(), return_scores ? scores.data_ptr<float>() : nullptr,
                               current_stream()));
  return {gates, idx, scores};
}

// selection and gates on scores the caller holds (after masking with -inf, say): [B,Q,S] -> gates, indices [B,Q,top_k]
std::tuple<at::Tensor, at::Tensor> topk_select_cuda(const at::Tensor& scores, const c10::optional<at::Tensor>& visible,
                                                    int64_t top_k, double temperature) {
  TORCH_CHECK(scores.dim() == 3, "scores must have shape [B, Q, S]");
  require_cuda(scores, "scores");
  c10::cuda::CUDAGuard guard(scores.device());
  auto sc = scores.to(at::kFloat).contiguous();
  const int64_t B = sc.size(0), Q = sc.size(1), S = sc.size(2);
  at::Tensor vis;
  const int32_t* vis_ptr = nullptr;
  if (visible.has_value() && visible->defined()) {
    require_cuda(*visible, "visible");
    TORCH_CHECK(visible->numel() == Q, "visible must hold one count per query");
    vis = visible->to(at::kInt).contiguous();
    vis_ptr = vis.data_ptr<int32_t>();
  }
  auto idx = at::empty({B, Q, top_k}, sc.options().dtype(at::kLong));
  auto gates = at::empty({B, Q, top_k}, sc.options());
  check_status(grmx_topk_select(sc.data_ptr<float>(), vis_ptr, B, Q, S, static_cast<int>(top_k),
                                static_cast<float>(temperature), idx.data_ptr<int64_t>(), gates.data_ptr<float>(),
                                current_stream()));
  return {gates, idx};
}

// states [B,Q,S,H] (fp32 or bf16), indices [B,Q,R], gates [B,Q,R] -> [B,Q,H] in the dtype of states
at::Tensor select_fuse_cuda(const at::Tensor& states, const at::Tensor& indices, const at::Tensor& gates,
                            const c10::optional<at::Tensor>& online, const c10::optional<at::Tensor>& ln_weight,
                            const c10::optional<at::Tensor>& ln_bias, double ln_eps, int64_t mode) {
  TORCH_CHECK(states.dim() == 4, "states must have shape [B, Q, S, H]");
  TORCH_CHECK(indices.dim() == 3 && gates.dim() == 3, "indices and gates must have shape [B, Q, R]");
  TORCH_CHECK(indices.sizes() == gates.sizes(), "indices and gates differ in shape");
  TORCH_CHECK(states.size(0) == indices.size(0) && states.size(1) == indices.size(1), "batch/query dim mismatch");
  require_cuda(states, "states");
  require_cuda(indices, "indices");
  require_cuda(gates, "gates");
  TORCH_CHECK(states.scalar_type() == at::kFloat || states.scalar_type() == at::kBFloat16,
              "states must be float32 or bfloat16");
  c10::cuda::CUDAGuard guard(states.device());
  auto st = states.contiguous();
  auto idx = indices.toType(at::kLong).contiguous();
  auto g = gates.to(at::kFloat).contiguous();
  const int64_t B = st.size(0), Q = st.size(1), S = st.size(2), H = st.size(3), R = idx.size(2);
  at::Tensor o_keep, w_keep, b_keep;
  const void* o_ptr = nullptr;
  if (online.has_value() && online->defined()) {
    require_cuda(*online, "online");
    o_keep = online->to(st.scalar_type()).contiguous();
    TORCH_CHECK(o_keep.sizes() == at::IntArrayRef({B, Q, H}), "online has the wrong shape");
    o_ptr = o_keep.data_ptr();
  }
  auto opt = [&](const c10::optional<at::Tensor>& t, const char* name, at::Tensor& keep) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    require_cuda(*t, name);
    keep = t->to(at::kFloat).contiguous();
    TORCH_CHECK(keep.numel() == H, name, " has the wrong shape");
    return keep.data_ptr<float>();
  };
  const float* w_ptr = opt(ln_weight, "ln_weight", w_keep);
  const float* b_ptr = opt(ln_bias, "ln_bias", b_keep);
  at::Tensor out = at::empty({B, Q, H}, st.options());
  check_status(grmx_select_fuse(st.data_ptr(), idx.data_ptr<int64_t>(), g.data_ptr<float>(), o_ptr, w_ptr, b_ptr,
                                static_cast<float>(ln_eps), out.data_ptr(), B, Q, S, R, H,
                                st.scalar_type() == at::kFloat ? GRMX_F32 : GRMX_BF16, static_cast<int>(mode),
                                current_stream()));
  return out;
}

// LayerNorm(a + b) over the last dimension (fp32 or bf16 rows of whole 16-byte pieces, H <= 1024)
at::Tensor add_layer_norm_cuda(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& ln_weight,
                               const c10::optional<at::Tensor>& ln_bias, double ln_eps) {
  TORCH_CHECK(a.sizes() == b.sizes() && a.dim() >= 1, "a and b must have the same shape");
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kFloat || a.scalar_type() == at::kBFloat16),
              "a and b must both be float32 or bfloat16");
  require_cuda(a, "a");
  require_cuda(b, "b");
  c10::cuda::CUDAGuard guard(a.device());
  auto ca = a.contiguous(), cb = b.contiguous();
  const int64_t H = ca.size(-1);
  const int64_t rows = H > 0 ? ca.numel() / H : 0;
  at::Tensor w_keep, b_keep;
  auto opt = [&](const c10::optional<at::Tensor>& t, const char* name, at::Tensor& keep) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    require_cuda(*t, name);
    keep = t->to(at::kFloat).contiguous();
    TORCH_CHECK(keep.numel() == H, name, " has the wrong shape");
    return keep.data_ptr<float>();
  };
  const float* w_ptr = opt(ln_weight, "ln_weight", w_keep);
  const float* b_ptr = opt(ln_bias, "ln_bias", b_keep);
  at::Tensor out = at::empty_like(ca);
  check_status(grmx_add_layer_norm(ca.data_ptr(), cb.data_ptr(), w_ptr, b_ptr, static_cast<float>(ln_eps), out.data_ptr(),
                                   rows, H, ca.scalar_type() == at::kFloat ? GRMX_F32 : GRMX_BF16, current_stream()));
  return out;
}

std::tuple<at::Tensor, at::Tensor> chunk_scan_segments_cuda(const at::Tensor& keys, const at::Tensor& values,
                                                            const at::Tensor& queries, const at::Tensor& memory,
                                                            double memory_decay, at::Tensor archive, int64_t first_slot,
                                                            int64_t segment_tokens) {
  check_chunk_inputs(keys, values, queries, memory);
  TORCH_CHECK(archive.is_cuda() && archive.dim() == 4 && archive.scalar_type() == at::kFloat && archive.is_contiguous(),
              "archive must be a contiguous float32 CUDA tensor [B, capacity, H, K]");
  c10::cuda::CUDAGuard guard(keys.device());
  auto k = keys.contiguous();
  auto v = values.contiguous();
  auto q = queries.contiguous();
  auto m = memory.contiguous();
  const int64_t B = k.size(0), T = k.size(1), K = k.size(2), H = v.size(2);
  TORCH_CHECK(archive.size(0) == B && archive.size(2) == H && archive.size(3) == K, "archive does not match the scan");
  auto hidden = at::empty({B, T, H}, v.options());
  auto memory_out = at::empty_like(m);
  check_status(grmx_chunk_scan_fwd_segments(k.data_ptr(), v.data_ptr(), q.data_ptr(), m.data_ptr(), hidden.data_ptr(),
                                            memory_out.data_ptr(), archive.data_ptr<float>(), archive.size(1),
                                            first_slot, segment_tokens, B, T, K, H, static_cast<float>(memory_decay),
                                            dtype_code(k.scalar_type(), "keys"), dtype_code(m.scalar_type(), "memory"),
                                            current_stream()));
  return {hidden, memory_out};
}

at::Tensor l2_normalize_cuda(const at::Tensor& x, double eps, bool to_bfloat16) {
  TORCH_CHECK(x.is_cuda(), "l2_normalize needs a CUDA tensor");
  TORCH_CHECK(x.dim() >= 1, "l2_normalize needs at least one dimension");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "l2_normalize takes float32 or bfloat16");
  c10::cuda::CUDAGuard guard(x.device());
  auto in = x.contiguous();
  const bool cast = to_bfloat16 && in.scalar_type() == at::kFloat;
  auto out = at::empty_like(in, cast ? in.options().dtype(at::kBFloat16) : in.options());
  const int64_t K = in.size(-1);
  const int64_t N = K == 0 ? 0 : in.numel() / K;
  check_status(grmx_normalize_rows(in.data_ptr(), out.data_ptr(), N, K, static_cast<float>(eps),
                                   in.scalar_type() == at::kFloat ? GRMX_F32 : GRMX_BF16,
                                   out.scalar_type() == at::kFloat ? GRMX_F32 : GRMX_BF16, current_stream()));
  return out;
}

// x bf16 [..., D], weights bf16 [128, D] (two stacked 64-row matrices), bias fp32 [128]? -> two bf16 [..., 64]
std::tuple<at::Tensor, at::Tensor> project_normalize_cuda(const at::Tensor& x, const at::Tensor& weights,
                                                          const c10::optional<at::Tensor>& bias, double eps) {
  TORCH_CHECK(x.is_cuda() && weights.is_cuda(), "project_normalize needs CUDA tensors");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && weights.scalar_type() == at::kBFloat16, "x and weights must be bfloat16");
  TORCH_CHECK(x.dim() >= 2 && weights.dim() == 2 && weights.size(1) == x.size(-1) && weights.size(0) % 2 == 0,
              "weights must be [2K, D] for x [..., D]");
  c10::cuda::CUDAGuard guard(x.device());
  auto in = x.contiguous();
  auto w = weights.contiguous();
  const int64_t D = in.size(-1), K = w.size(0) / 2;
  const int64_t rows = in.numel() / D;
  at::Tensor b_keep;
  const float* b_ptr = nullptr;
  if (bias.has_value() && bias->defined()) {
    b_keep = bias->to(at::kFloat).contiguous();
    TORCH_CHECK(b_keep.numel() == 2 * K, "bias must hold 2K values");
    b_ptr = b_keep.data_ptr<float>();
  }
  std::vector<int64_t> shape(in.sizes().begin(), in.sizes().end());
  shape.back() = K;
  auto a = at::empty(shape, in.options());
  auto b = at::empty(shape, in.options());
  check_status(grmx_project_normalize(in.data_ptr(), w.data_ptr(), b_ptr, a.data_ptr(), b.data_ptr(), rows, D, K,
                                      static_cast<float>(eps), current_stream()));
  return {a, b};
}

void archive_push_cuda(const at::Tensor& memory, at::Tensor archive, c10::optional<at::Tensor> shadow, int64_t slot) {
  TORCH_CHECK(archive.dim() == 4 && memory.dim() == 3, "memory [B, H, K] goes into archive [B, S, H, K]");
  TORCH_CHECK(memory.is_cuda() && archive.is_cuda(), "archive_push needs CUDA tensors");
  TORCH_CHECK(memory.scalar_type() == at::kFloat && archive.scalar_type() == at::kFloat, "memory and archive are float32");
  TORCH_CHECK(archive.is_contiguous(), "archive must be contiguous: it is written in place");
  const int64_t B = archive.size(0), S = archive.size(1), H = archive.size(2), K = archive.size(3);
  TORCH_CHECK(memory.size(0) == B && memory.size(1) == H && memory.size(2) == K, "memory does not match the archive");
  void* shadow_ptr = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    TORCH_CHECK(shadow->scalar_type() == at::kBFloat16 && shadow->is_contiguous() && shadow->sizes() == archive.sizes() &&
                    shadow->is_cuda(), "the bf16 ring must be a contiguous bfloat16 CUDA tensor shaped like the archive");
    shadow_ptr = shadow->data_ptr();
  }
  c10::cuda::CUDAGuard guard(archive.device());
  auto mem = memory.contiguous();
  check_status(grmx_archive_push(mem.data_ptr<float>(), archive.data_ptr<float>(), shadow_ptr, B, S, slot, H * K,
                                 current_stream()));
}

at::Tensor retrieve_fuse_cuda(const at::Tensor& archive, const at::Tensor& indices,
                              const c10::optional<at::Tensor>& gates, const at::Tensor& queries,
                              const c10::optional<at::Tensor>& online,
                              const c10::optional<at::Tensor>& ln_weight,
                              const c10::optional<at::Tensor>& ln_bias, double ln_eps, int64_t mode) {
  TORCH_CHECK(archive.dim() == 4, "archive must have shape [B, S, H, K]");
  TORCH_CHECK(indices.dim() == 3, "indices must have shape [B, Q, R]");
  TORCH_CHECK(queries.dim() == 3, "queries must have shape [B, Q, K]");
  TORCH_CHECK(archive.size(0) == indices.size(0) && archive.size(0) == queries.size(0), "batch dim mismatch");
  TORCH_CHECK(indices.size(1) == queries.size(1), "query dim mismatch between indices and queries");
  TORCH_CHECK(archive.size(3) == queries.size(2), "key dim mismatch between archive and queries");
  require_cuda(archive, "archive");
  require_cuda(indices, "indices");
  require_cuda(queries, "queries");
  TORCH_CHECK(archive.scalar_type() == at::kFloat, "archive must be float32");
  c10::cuda::CUDAGuard guard(archive.device());
  auto arch = archive.contiguous();
  auto idx = indices.toType(at::kLong).contiguous();
  auto q = queries.to(at::kFloat).contiguous();
  const int64_t B = arch.size(0), S = arch.size(1), H = arch.size(2), K = arch.size(3);
  const int64_t Q = idx.size(1), R = idx.size(2);
  auto opt = [&](const c10::optional<at::Tensor>& t, std::vector<int64_t> shape, const char* name,
                 at::Tensor& keep) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    require_cuda(*t, name);
    keep = t->to(at::kFloat).contiguous();
    TORCH_CHECK(keep.sizes() == at::IntArrayRef(shape), name, " has the wrong shape");
    return keep.data_ptr<float>();
  };
  at::Tensor g_keep, o_keep, w_keep, b_keep;
  const float* g_ptr = opt(gates, {B, Q, R}, "gates", g_keep);
  const float* o_ptr = opt(online, {B, Q, H}, "online", o_keep);
  const float* w_ptr = opt(ln_weight, {H}, "ln_weight", w_keep);
  const float* b_ptr = opt(ln_bias, {H}, "ln_bias", b_keep);
  at::Tensor out = mode == GRMX_FUSE_RETRIEVED ? at::empty({B, Q, R, H}, arch.options())
                                               : at::empty({B, Q, H}, arch.options());
  check_status(grmx_retrieve_fuse(arch.data_ptr<float>(), idx.data_ptr<int64_t>(), g_ptr,
                                  q.data_ptr<float>(), o_ptr, w_ptr, b_ptr, static_cast<float>(ln_eps),
                                  out.data_ptr(), B, S, Q, R, H, K, static_cast<int>(mode),
                                  current_stream()));
  return out;
}

// bf16 archive ring [B,S,H,K], bf16 queries [B,Q,K], bf16 online [B,Q,H] -> bf16 [B,Q,H] (tensor-core retrieval)
at::Tensor retrieve_fuse_tc_cuda(const at::Tensor& archive, const at::Tensor& indices, const at::Tensor& gates,
                                 const at::Tensor& queries, const c10::optional<at::Tensor>& online,
                                 const c10::optional<at::Tensor>& ln_weight, const c10::optional<at::Tensor>& ln_bias,
                                 double ln_eps, int64_t mode) {
  TORCH_CHECK(archive.dim() == 4, "archive must have shape [B, S, H, K]");
  TORCH_CHECK(indices.dim() == 3 && gates.dim() == 3 && indices.sizes() == gates.sizes(),
              "indices and gates must have shape [B, Q, R]");
  TORCH_CHECK(queries.dim() == 3, "queries must have shape [B, Q, K]");
  TORCH_CHECK(archive.size(0) == indices.size(0) && archive.size(0) == queries.size(0), "batch dim mismatch");
  TORCH_CHECK(indices.size(1) == queries.size(1), "query dim mismatch between indices and queries");
  TORCH_CHECK(archive.size(3) == queries.size(2), "key dim mismatch between archive and queries");
  require_cuda(archive, "archive");
  require_cuda(indices, "indices");
  require_cuda(gates, "gates");
  require_cuda(queries, "queries");
  TORCH_CHECK(archive.scalar_type() == at::kBFloat16 && queries.scalar_type() == at::kBFloat16,
              "archive and queries must be bfloat16");
  c10::cuda::CUDAGuard guard(archive.device());
  auto arch = archive.contiguous();
  auto idx = indices.toType(at::kLong).contiguous();
  auto g = gates.to(at::kFloat).contiguous();
  auto q = queries.contiguous();
  const int64_t B = arch.size(0), S = arch.size(1), H = arch.size(2), K = arch.size(3);
  const int64_t Q = idx.size(1), R = idx.size(2);
  at::Tensor o_keep, w_keep, b_keep;
  const void* o_ptr = nullptr;
  if (online.has_value() && online->defined()) {
    require_cuda(*online, "online");
    o_keep = online->to(at::kBFloat16).contiguous();
    TORCH_CHECK(o_keep.sizes() == at::IntArrayRef({B, Q, H}), "online has the wrong shape");
    o_ptr = o_keep.data_ptr();
  }
  auto opt = [&](const c10::optional<at::Tensor>& t, const char* name, at::Tensor& keep) -> const float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    require_cuda(*t, name);
    keep = t->to(at::kFloat).contiguous();
    TORCH_CHECK(keep.numel() == H, name, " has the wrong shape");
    return keep.data_ptr<float>();
  };
  const float* w_ptr = opt(ln_weight, "ln_weight", w_keep);
  const float* b_ptr = opt(ln_bias, "ln_bias", b_keep);
  at::Tensor out = at::empty({B, Q, H}, arch.options());
  check_status(grmx_retrieve_fuse_tc(arch.data_ptr(), idx.data_ptr<int64_t>(), g.data_ptr<float>(), q.data_ptr(), o_ptr,
                                     w_ptr, b_ptr, static_cast<float>(ln_eps), out.data_ptr(), B, S, Q, R, H, K,
                                     static_cast<int>(mode), current_stream()));
  return out;
}

}  // namespace

TORCH_LIBRARY(grm_cuda, m) {
  m.def("chunk_update_forward(Tensor keys, Tensor values, Tensor queries, Tensor memory, float memory_decay) -> (Tensor hidden, Tensor memory_out, Tensor aux)");
  m.def("chunk_update_backward(Tensor grad_hidden, Tensor grad_memory_out, Tensor keys, Tensor values, Tensor queries, Tensor memory, Tensor aux, float memory_decay) -> (Tensor grad_keys, Tensor grad_values, Tensor grad_queries, Tensor grad_memory)");
  m.def("apply_query_forward(Tensor memories, Tensor queries) -> Tensor");
  m.def("apply_query_backward(Tensor grad_hidden, Tensor memories, Tensor queries) -> (Tensor grad_memories, Tensor grad_queries)");
  m.def("batched_memory_gather(Tensor memories_per_batch, Tensor topk_indices) -> Tensor");
}

TORCH_LIBRARY_IMPL(grm_cuda, CUDA, m) {
  m.impl("chunk_update_forward", chunk_update_forward_cuda);
  m.impl("chunk_update_backward", chunk_update_backward_cuda);
  m.impl("apply_query_forward", apply_query_forward_cuda);
  m.impl("apply_query_backward", apply_query_backward_cuda);
  m.impl("batched_memory_gather", batched_memory_gather_cuda);
}

TORCH_LIBRARY(grmx, m) {
  m.def("linear_scan(Tensor keys, Tensor values, Tensor queries, Tensor memory, float decay, float update_coeff, float hidden_scale, float memory_out_scale, bool reverse, bool first_step_no_decay, int path) -> (Tensor hidden, Tensor memory_out)");
  m.def("topk_route(Tensor queries, Tensor keys, Tensor? visible, int top_k, float scale, float temperature, bool return_scores) -> (Tensor gates, Tensor indices, Tensor scores)");
  m.def("topk_select(Tensor scores, Tensor? visible, int top_k, float temperature) -> (Tensor gates, Tensor indices)");
  m.def("retrieve_fuse(Tensor archive, Tensor indices, Tensor? gates, Tensor queries, Tensor? online, Tensor? ln_weight, Tensor? ln_bias, float ln_eps, int mode) -> Tensor");
  m.def("retrieve_fuse_tc(Tensor archive, Tensor indices, Tensor gates, Tensor queries, Tensor? online, Tensor? ln_weight, Tensor? ln_bias, float ln_eps, int mode) -> Tensor");
  m.def("chunk_scan_segments(Tensor keys, Tensor values, Tensor queries, Tensor memory, float decay, Tensor(a!) archive, int first_slot, int segment_tokens) -> (Tensor hidden, Tensor memory_out)");
  m.def("l2_normalize(Tensor x, float eps, bool to_bfloat16) -> Tensor");
  m.def("project_normalize(Tensor x, Tensor weights, Tensor? bias, float eps) -> (Tensor a, Tensor b)");
  m.def("archive_push(Tensor memory, Tensor(a!) archive, Tensor(b!)? shadow, int slot) -> ()");
  m.def("add_layer_norm(Tensor a, Tensor b, Tensor? ln_weight, Tensor? ln_bias, float ln_eps) -> Tensor");
  m.def("select_fuse(Tensor states, Tensor indices, Tensor gates, Tensor? online, Tensor? ln_weight, Tensor? ln_bias, float ln_eps, int mode) -> Tensor");
}

TORCH_LIBRARY_IMPL(grmx, CUDA, m) {
  m.impl("linear_scan", linear_scan_cuda);
  m.impl("topk_route", topk_route_cuda);
  m.impl("topk_select", topk_select_cuda);
  m.impl("retrieve_fuse", retrieve_fuse_cuda);
  m.impl("retrieve_fuse_tc", retrieve_fuse_tc_cuda);
  m.impl("select_fuse", select_fuse_cuda);
  m.impl("add_layer_norm", add_layer_norm_cuda);
  m.impl("archive_push", archive_push_cuda);
  m.impl("project_normalize", project_normalize_cuda);
  m.impl("l2_normalize", l2_normalize_cuda);
  m.impl("chunk_scan_segments", chunk_scan_segments_cuda);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "GRM segment-memory engine for B200 (sm_100a): torch.ops.grm_cuda.* over the grmx C ABI";
  m.attr("__grm_cuda_with_kernels__") = pybind11::bool_(true);
  m.def("grmx_version", []() { return grmx_version(); });
  m.def("launch_count", []() { return grmx_launch_count(); });
  m.def("set_scan_path", [](int path) {
    TORCH_CHECK(path == GRMX_PATH_AUTO || path == GRMX_PATH_FFMA || path == GRMX_PATH_TCGEN05,
                "scan path must be 0 (auto), 1 (ffma) or 2 (tcgen05)");
    g_scan_path.store(path);
  });
  m.def("get_scan_path", []() { return g_scan_path.load(); });
  // The device error word of the current device: kernels report a bounded wait that gave up or an
  // out-of-range routing index there instead of trapping.  Reading it waits for the current stream.
  m.def("device_error_word", []() {
    uint32_t word = 0;
    check_status(grmx_device_error_word(&word, current_stream()));
    return word;
  });
  m.def("device_error_reset", []() { check_status(grmx_device_error_reset(current_stream())); });
}
