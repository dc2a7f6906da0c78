/*
 * grmx.h -- C ABI of the B200 (sm_100a) engine for GRM's segment-memory path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on
 * the CUDA stream it is given and returns immediately: no allocation, no host
 * synchronisation, no exception crosses this boundary.  A return value of 0
 * means "enqueued"; any other value is an argument or launch error whose text
 * is available from grmx_last_error() on the calling thread.
 *
 * Tensors are dense and row-major unless a stride argument says otherwise.
 * Shapes use the reference's names: B = op batch (batch x heads when heads
 * are independent), T = tokens in the call, K = memory key dim (d_k),
 * H = hidden / value dim (d_v), S = archived segments, R = routes (top-k),
 * Q = queries per batch row.  The recurrent state is M[B, H, K], K fastest
 * (reference: grm/csrc/grm_cuda.cpp:18-26).
 *
 * The file:line citations name the reference interface each call replaces
 * (paths relative to the Sggggt/RNN_with_GRM project root).
 */
#ifndef GRMX_H_
#define GRMX_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of tensors crossing the ABI */
#define GRMX_F32 0
#define GRMX_BF16 1
#define GRMX_F16 2

/* status codes */
#define GRMX_OK 0
#define GRMX_ERR_ARG 1         /* bad shape / null pointer / bad enum           */
#define GRMX_ERR_UNSUPPORTED 2 /* valid request this build has no kernel for    */
#define GRMX_ERR_LAUNCH 3      /* CUDA reported an error at launch              */
#define GRMX_ERR_DEVICE 4      /* wrong device (not sm_100) for the chosen path */

/* kernel family for the chunk scan */
#define GRMX_PATH_AUTO 0    /* tcgen05 path when shape/dtype allow it, else FFMA */
#define GRMX_PATH_FFMA 1    /* fp32 CUDA-core scan: exact mode, any shape        */
#define GRMX_PATH_TCGEN05 2 /* bf16 tensor-core chunked scan, fp32 state         */

/* fusion rule applied by grmx_retrieve_fuse */
#define GRMX_FUSE_RETRIEVED 0 /* out[B,Q,R,H]  = M[idx] q                           */
#define GRMX_FUSE_CONTRIB 1   /* out[B,Q,H]    = sum_r gate_r M[idx_r] q            */
#define GRMX_FUSE_RESIDUAL_LN 2 /* out[B,Q,H]  = LayerNorm(h + sum_r gate_r M[idx_r] q) */

typedef struct grmx_device_info {
  int32_t device;
  int32_t cc_major;
  int32_t cc_minor;
  int32_t sm_count;
  int32_t max_smem_per_block; /* opt-in bytes */
  int32_t has_tcgen05;        /* 1 when cc is 10.x */
  int64_t total_mem;
} grmx_device_info;

/* library version: major*10000 + minor*100 + patch */
int grmx_version(void);

/* Text of the last error raised on the calling thread ("" when none). */
const char* grmx_last_error(void);

/* Fills *out for CUDA device `device`.  Host-only query (cudaGetDeviceProperties). */
int grmx_query_device(int device, grmx_device_info* out);

/* Number of kernel launches this library has enqueued in this process
 * (all threads).  Used by the benchmark to count launches in a timed region. */
int64_t grmx_launch_count(void);

/*
 * Chunked linear-memory update + query application.
 *
 *   M_t = decay * M_{t-1} + (1-decay)/sqrt(K) * v_t k_t^T      (M_{-1} = memory_in)
 *   hidden_t = M_t q_t                                          (update is inclusive)
 *   memory_out = M_{T-1}
 *
 * keys, queries [B,T,K]; values, hidden_out [B,T,H] in io_dtype; memory_in,
 * memory_out [B,H,K] in state_dtype (GRMX_F32, or equal to io_dtype).
 * T == 0 copies memory_in to memory_out and writes no hidden.
 * path selects the kernel family (GRMX_PATH_*).
 * With few batch rows and many tokens the tensor-core path cuts every row along T into up to
 * four pieces that run on different SMs; each piece derives the state it starts from by running
 * the state recurrence alone over the tokens before it (one launch, no workspace; set
 * GRMX_SCAN_CUT=off in the environment to keep rows whole).
 *
 * Replaces grm_cuda::chunk_update_forward (grm/csrc/bindings.cpp:6,
 * grm/csrc/chunk_update.cu:523-586; math grm/core/cuda_ops.py:218-254,
 * sequential form grm/csrc/grm_cuda.cpp:46-90).
 */
int grmx_chunk_scan_fwd(const void* keys, const void* values, const void* queries,
                        const void* memory_in, void* hidden_out, void* memory_out,
                        int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                        int io_dtype, int state_dtype, int path, void* stream);

/*
 * grmx_chunk_scan_fwd over a sequence of T / segment_tokens whole segments in ONE launch, leaving the
 * state at the end of segment j in archive[b, first_slot + j, :, :] (archive float32 [B, capacity, H, K],
 * dense, 16-byte aligned) besides hidden_out and the final memory_out.  The result is that of one
 * grmx_chunk_scan_fwd call per segment with the state carried from call to call: the reference's segment
 * loop (grm/core/paper_grm.py:702-728, memory_initialization_mode "checkpoint") runs the scan and the
 * archive append once per segment; the retrieval of a segment reads only earlier slots, so it can follow
 * for all segments at once.  Tensor-core scan only (bf16 tokens, fp32 state, K and H multiples of 64),
 * segment_tokens a multiple of 128 that divides T, first_slot + T / segment_tokens <= capacity;
 * GRMX_ERR_UNSUPPORTED otherwise (run the segments one by one).
 */
int grmx_chunk_scan_fwd_segments(const void* keys, const void* values, const void* queries,
                                 const void* memory_in, void* hidden_out, void* memory_out, float* archive,
                                 int64_t capacity, int64_t first_slot, int64_t segment_tokens, int64_t B,
                                 int64_t T, int64_t K, int64_t H, float decay, int io_dtype, int state_dtype,
                                 void* stream);

/*
 * grmx_chunk_scan_fwd with a caller-provided workspace: the two-kernel form of the cut along T.
 * A first kernel computes every piece's own contribution to the state into `scratch` (device
 * memory, 16-byte aligned, contents irrelevant on entry, not preserved), the scan kernel rebuilds
 * each piece's start state from them.  More pieces than the one-launch form allows (no piece
 * repeats the work of another), at the price of a second launch: the better choice for very
 * long rows.
 * grmx_chunk_scan_scratch_bytes returns the size that cut needs for the given call on the
 * current device, or 0 when the call would not be cut.  With scratch == NULL or a buffer that
 * is too small the call behaves exactly like grmx_chunk_scan_fwd.  Results are the same up to
 * floating-point summation order.  Same reference interface as grmx_chunk_scan_fwd.
 */
int64_t grmx_chunk_scan_scratch_bytes(int64_t B, int64_t T, int64_t K, int64_t H, int io_dtype,
                                      int state_dtype);
int grmx_chunk_scan_fwd_ws(const void* keys, const void* values, const void* queries,
                           const void* memory_in, void* hidden_out, void* memory_out,
                           int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                           int io_dtype, int state_dtype, int path, void* scratch,
                           int64_t scratch_bytes, void* stream);

/*
 * The same scan for callers that cannot allocate device memory where they call it (a server
 * that has given all of HBM to its own pool, a real-time callback, a sandboxed plugin that
 * only owns its input and output buffers).  bf16 tokens, fp32 state, d_k and d_v multiples of 64,
 * layouts as in grmx_chunk_scan_fwd.  The workspace is an array inside the library image,
 * grmx_static_scratch_capacity() bytes (4 MiB) of device memory held by every GPU that loads
 * the library until the process exits; only heads of 64 x 64 are ever cut over it (wider heads
 * run the one-launch form and do not touch the array).  A call that would need more than the
 * array holds is refused with GRMX_ERR_UNSUPPORTED, and nothing is ever allocated or freed.
 * The first call on each device looks the array's address up (cudaGetSymbolAddress, with that
 * device current), so make that first call outside any stream capture; the remembered address
 * does not survive cudaDeviceReset or the teardown of the device's primary context.  All calls
 * share the one array: nothing in it has to be cleared between calls (each call overwrites what
 * it later reads), but two calls that run on the GPU at the same time -- different streams, or
 * different host threads -- race on it.
 * grmx_chunk_scan_scratch_bytes_on is grmx_chunk_scan_scratch_bytes for a device of sm_count
 * multiprocessors instead of the current one (a pure host computation), and
 * grmx_static_scratch_admits(need) is the admission test itself: GRMX_OK when `need` bytes fit the
 * array, GRMX_ERR_UNSUPPORTED with the refusal text otherwise.  Together they tell a caller ahead
 * of time, without a GPU, whether a shape will be accepted.
 * No counterpart in the reference.
 */
int64_t grmx_static_scratch_capacity(void);
int64_t grmx_chunk_scan_scratch_bytes_on(int64_t B, int64_t T, int64_t K, int64_t H, int sm_count);
int grmx_static_scratch_admits(int64_t need_bytes);
int grmx_chunk_scan_fwd_static(const void* keys, const void* values, const void* queries,
                               const void* memory_in, void* hidden_out, void* memory_out,
                               int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                               void* stream);

/*
 * Gradients of grmx_chunk_scan_fwd: given grad_hidden [B,T,H] (io_dtype) and
 * grad_memory_out [B,H,K] (state_dtype) writes grad_keys, grad_queries
 * [B,T,K], grad_values [B,T,H] (io_dtype) and grad_memory [B,H,K]
 * (state_dtype).  Runs three scans of the forward kernel family with the
 * operands permuted; needs no scratch memory and no saved per-token states.
 *
 * Replaces grm_cuda::chunk_update_backward (grm/csrc/bindings.cpp:7,
 * grm/csrc/chunk_update.cu:588-716, grm/csrc/grm_cuda.cpp:92-126).
 */
int grmx_chunk_scan_bwd(const void* grad_hidden, const void* grad_memory_out,
                        const void* keys, const void* values, const void* queries,
                        const void* memory_in, void* grad_keys, void* grad_values,
                        void* grad_queries, void* grad_memory, int64_t B, int64_t T,
                        int64_t K, int64_t H, float decay, int io_dtype, int state_dtype,
                        int path, void* stream);

/*
 * The general recurrence both calls above are built from:
 *
 *   M_t = a_t * M_{t-1} + update_coeff * v_t k_t^T,   hidden_t = hidden_scale * M_t q_t
 *   a_t = decay, except a_first = 1 when first_step_no_decay != 0
 *   memory_out = memory_out_scale * M_last
 *
 * Tokens are visited in increasing order, or decreasing when reverse != 0.
 * memory_in is read with element strides (m_row_stride along H, m_col_stride
 * along K; batch stride H*K), so a transposed state can be consumed in place.
 * memory_out may be NULL.  No counterpart in the reference: its backward
 * kernel (grm/csrc/chunk_update.cu:137-278) is a separate code path.
 */
int grmx_linear_scan(const void* keys, const void* values, const void* queries,
                     const void* memory_in, int64_t m_row_stride, int64_t m_col_stride,
                     void* hidden_out, void* memory_out, int64_t B, int64_t T, int64_t K,
                     int64_t H, float decay, float update_coeff, float hidden_scale,
                     float memory_out_scale, int reverse, int first_step_no_decay,
                     int io_dtype, int state_dtype, int path, void* stream);

/*
 * hidden[n,r,h] = sum_k memories[n,r,h,k] * queries[n,k]
 * memories [N,R,H,K], queries [N,K], hidden [N,R,H], one dtype.  N = B for
 * the rank-4 form and B*Q for the rank-5 form of the reference op.
 *
 * Replaces grm_cuda::apply_query_forward (grm/csrc/bindings.cpp:8,
 * grm/csrc/apply_query.cu:14-75,185-254; math grm/core/cuda_ops.py:257-262).
 */
int grmx_apply_query_fwd(const void* memories, const void* queries, void* hidden,
                         int64_t N, int64_t R, int64_t H, int64_t K, int dtype,
                         void* stream);

/*
 * grad_memories[n,r,h,k] = grad_hidden[n,r,h] * queries[n,k]
 * grad_queries[n,k]      = sum_{r,h} grad_hidden[n,r,h] * memories[n,r,h,k]
 *
 * Replaces grm_cuda::apply_query_backward (grm/csrc/bindings.cpp:9,
 * grm/csrc/apply_query.cu:77-169,256-330).
 */
int grmx_apply_query_bwd(const void* grad_hidden, const void* memories, const void* queries,
                         void* grad_memories, void* grad_queries, int64_t N, int64_t R,
                         int64_t H, int64_t K, int dtype, void* stream);

/*
 * out[b,j,:] = memories[b, indices[b,j], :]   for j in [0, J)
 * memories [B,S,row_elems], indices int64 [B,J], out [B,J,row_elems];
 * J = R (rank-2 indices) or Q*R (rank-3); row_elems = H*K; elem_size in
 * bytes (2 or 4).  Index -1 (the empty-slot marker of grmx_topk_route)
 * yields a zero-filled row; any other index outside [0,S) does too and also
 * sets the device error word (grmx_device_error_word) instead of faulting.
 *
 * Replaces grm_cuda::batched_memory_gather (grm/csrc/bindings.cpp:10,
 * grm/csrc/batched_gather.cu:14-181; math grm/core/cuda_ops.py:265-284).
 */
int grmx_batched_gather(const void* memories, const int64_t* indices, void* out, int64_t B,
                        int64_t S, int64_t J, int64_t row_elems, int elem_size,
                        void* stream);

/*
 * Sparse top-k routing of Q queries per batch row over S segment keys.
 *
 *   score[b,q,s] = scale * sum_d queries[b,q,d] * keys[b,s,d]   (fp32 fused
 *                  multiply-add, d ascending: the summation order is part of
 *                  the contract so that indices are reproducible bit for bit)
 *   visible[q] (int32, may be NULL = S): query q sees keys s < visible[q]
 *   R_q = min(top_k, visible[q]).  When R_q == visible[q] the routes are the
 *   identity order 0..R_q-1 (no sort); otherwise the R_q highest scores in
 *   descending order, equal scores resolved to the lower index; NaN ranks
 *   above every number, -inf below.
 *   gates = softmax(selected scores / temperature) over the R_q routes.
 * indices_out int64 [B,Q,top_k] and gates_out fp32 [B,Q,top_k]; slots
 * r >= R_q hold index -1 and gate 0.  scores_out fp32 [B,Q,S] may be NULL.
 * Limits: top_k <= 32, S <= 2048.
 *
 * Replaces the PyTorch routing of TopKMemoryRetriever.forward
 * (grm/core/gating_unit.py:54-91) and _route_chunk
 * (grm/core/paper_grm.py:566-589); the projections stay with the caller.
 */
int grmx_topk_route(const float* queries, const float* keys, const int32_t* visible,
                    int64_t B, int64_t Q, int64_t S, int64_t D, int top_k, float scale,
                    float temperature, int64_t* indices_out, float* gates_out,
                    float* scores_out, void* stream);

/*
 * grmx_topk_route with the queries stored as bf16 (keys stay fp32): per-token routing reads the layer
 * input as it is, without an fp32 copy of it.  The queries are widened while they are staged, which is
 * exact, so scores, indices and gates are those of grmx_topk_route on the widened queries, bit for bit.
 * Covers the per-token shapes only: 1 <= S <= 16 keys, Q >= 64 queries per batch row, D % 8 == 0,
 * D <= 1024, B <= 65535, 16-byte aligned inputs; GRMX_ERR_UNSUPPORTED otherwise (widen and call
 * grmx_topk_route).  Same reference code as grmx_topk_route.
 */
int grmx_topk_route_bf16q(const void* queries_bf16, const float* keys, const int32_t* visible,
                          int64_t B, int64_t Q, int64_t S, int64_t D, int top_k, float scale,
                          float temperature, int64_t* indices_out, float* gates_out,
                          float* scores_out, void* stream);

/*
 * Selection and gates only, on scores the caller already holds (for example
 * after applying an attention mask with -inf): same rules as grmx_topk_route
 * from "visible" onwards.  scores fp32 [B,Q,S].
 */
int grmx_topk_select(const float* scores, const int32_t* visible, int64_t B, int64_t Q,
                     int64_t S, int top_k, float temperature, int64_t* indices_out,
                     float* gates_out, void* stream);

/*
 * Retrieval without materialising the gathered matrices:
 *
 *   retrieved[b,q,r,:] = archive[b, indices[b,q,r]] @ queries[b,q,:]
 *   contrib[b,q,:]     = sum_r gates[b,q,r] * retrieved[b,q,r,:]
 *   fused[b,q,:]       = LayerNorm(online[b,q,:] + contrib[b,q,:]) * ln_weight + ln_bias
 *
 * archive fp32 [B,S,H,K]; indices int64 [B,Q,R] (-1 = empty slot, skipped);
 * gates fp32 [B,Q,R]; queries fp32 [B,Q,K]; online fp32 [B,Q,H].  `mode`
 * (GRMX_FUSE_*) selects which of the three tensors is written to `out`.
 * A query whose slots are all empty gets out = online (no LayerNorm) in
 * GRMX_FUSE_RESIDUAL_LN mode, zeros otherwise -- the reference skips fusion
 * when no segment is archived (grm/core/paper_grm.py:620-621).
 * ln_weight / ln_bias may be NULL (identity affine).
 *
 * Replaces the chain cuda_batched_memory_gather -> cuda_apply_query ->
 * RetrievedStateFusion (grm/core/paper_grm.py:229-234,301-307,604-611;
 * grm/core/aggregator.py:104-105,116-145).
 */
int grmx_retrieve_fuse(const float* archive, const int64_t* indices, const float* gates,
                       const float* queries, const float* online, const float* ln_weight,
                       const float* ln_bias, float ln_eps, void* out, int64_t B, int64_t S,
                       int64_t Q, int64_t R, int64_t H, int64_t K, int mode, void* stream);

/*
 * The slot-major form of grmx_retrieve_fuse (modes GRMX_FUSE_CONTRIB and GRMX_FUSE_RESIDUAL_LN): one
 * CTA per batch row reads every chosen matrix once and applies it to all queries of the row that chose
 * it, where the query-major form reads a matrix once per query.  Same tensors and semantics; the sum
 * over a query's routes runs in slot order instead of route order, so results agree with
 * grmx_retrieve_fuse to fp32 rounding, not bit for bit.  Covers K a multiple of 32 up to 256, H up to 256
 * with 1, 2, 4 or 8 blocks of 32 rows, and rows whose queries and sums fit in shared memory beside eight
 * blocks of 32 matrix rows (200 KiB in all); GRMX_ERR_UNSUPPORTED otherwise.
 * grmx_retrieve_fuse takes this form by itself when B >= 64 and Q * R >= 2 * S (a row's queries share
 * matrices and there are rows enough to fill the GPU); GRMX_RETRIEVE_ROWS=off in the environment keeps
 * it on the query-major kernel.
 *
 * Replaces the same chain as grmx_retrieve_fuse for segment-level routing
 * (grm/core/paper_grm.py:566-611): every segment query of a row chooses among the same archived
 * matrices of that row (grm/csrc/batched_gather.cu:38-41 indexes within a batch row).
 */
int grmx_retrieve_fuse_rows(const float* archive, const int64_t* indices, const float* gates,
                            const float* queries, const float* online, const float* ln_weight,
                            const float* ln_bias, float ln_eps, void* out, int64_t B, int64_t S,
                            int64_t Q, int64_t R, int64_t H, int64_t K, int mode, void* stream);

/*
 * grmx_retrieve_fuse for per-token routing on the tensor cores: every token of a batch row chooses R of
 * the row's S archived matrices, all in bf16 (archive_bf16 [B,S,H,K], queries_bf16 [B,Q,K], online_bf16 and
 * out_bf16 [B,Q,H]; indices int64 and gates float32 [B,Q,R] as in grmx_retrieve_fuse).  For a tile of 128
 * tokens the kernel accumulates one product per chosen slot, (gate-scaled queries) x (the slot's matrix),
 * in a TMEM accumulator, so neither the gathered matrices nor per-candidate states ever exist in memory;
 * then residual + LayerNorm (GRMX_FUSE_RESIDUAL_LN; a token without a live route keeps its online state)
 * or the plain gate-weighted contribution (GRMX_FUSE_CONTRIB).  Sums in fp32; the gates enter the product
 * rounded to bf16.  Covers K == 64, H a multiple of 64 up to 512, 1 <= S <= 32, 1 <= R <= 8, 16-byte
 * aligned tensors; GRMX_ERR_UNSUPPORTED otherwise (use grmx_retrieve_fuse).
 *
 * Replaces the same chain as grmx_retrieve_fuse where the reference runs it per token
 * (grm/core/paper_grm.py:613-645: rank-5 gather, rank-5 apply-query grm/csrc/apply_query.cu:14-75,
 * RetrievedStateFusion on B*C rows).
 */
int grmx_retrieve_fuse_tc(const void* archive_bf16, const int64_t* indices, const float* gates,
                          const void* queries_bf16, const void* online_bf16, const float* ln_weight,
                          const float* ln_bias, float ln_eps, void* out_bf16, int64_t B, int64_t S, int64_t Q,
                          int64_t R, int64_t H, int64_t K, int mode, void* stream);

/*
 * The selection half of grmx_retrieve_fuse for callers that have already applied the query to every
 * candidate: states [B,Q,S,H] (states[b,q,s,:] = M[b,s] q[b,q], e.g. one batched GEMM per batch row when
 * all Q tokens of a segment choose among the same S archived matrices), indices int64 [B,Q,R] into S
 * (-1 = empty route), gates float32 [B,Q,R].
 *   GRMX_FUSE_CONTRIB:      out[b,q,:] = sum_r gates[r] * states[b,q,indices[r],:]
 *   GRMX_FUSE_RESIDUAL_LN:  out[b,q,:] = LayerNorm(online[b,q,:] + that sum), ln_weight/ln_bias float32 [H]
 *                           or NULL; a token without any live route returns online[b,q,:] unchanged
 * states, online and out share `dtype` (GRMX_F32 or GRMX_BF16); sums and the normalisation are fp32.
 * H <= 1024, R <= 32.  Follows grm/core/aggregator.py:104-105,116-118 (RetrievedStateFusion, "residual");
 * the reference has no native counterpart.
 */
int grmx_select_fuse(const void* states, const int64_t* indices, const float* gates, const void* online,
                     const float* ln_weight, const float* ln_bias, float ln_eps, void* out, int64_t B,
                     int64_t Q, int64_t S, int64_t R, int64_t H, int dtype, int mode, void* stream);

/*
 * out = LayerNorm(a + b) * ln_weight + ln_bias over rows of H values (dtype GRMX_F32 or GRMX_BF16 for a, b and
 * out; sum, mean and variance in fp32; ln_weight / ln_bias fp32 or NULL), one pass, both rows requested at
 * once.  The same arithmetic as grmx_select_fuse in GRMX_FUSE_RESIDUAL_LN mode with b as the only candidate
 * and a unit gate.  Rows of whole 16-byte pieces, 16-byte aligned tensors, H <= 1024; GRMX_ERR_UNSUPPORTED
 * otherwise.
 *
 * Replaces the residual block between the layers of the stack, self.layer_norm(outputs + x)
 * (grm/core/multilayer_grm.py:93,96), which the reference runs as an add followed by nn.LayerNorm.
 */
int grmx_add_layer_norm(const void* a, const void* b, const float* ln_weight, const float* ln_bias,
                        float ln_eps, void* out, int64_t rows, int64_t H, int dtype, void* stream);

/*
 * out[n,:] = x[n,:] / max(||x[n,:]||_2, eps) for N rows of K elements, in one pass (fp32 sum of squares).
 * (in_dtype, out_dtype) is (F32,F32), (BF16,BF16) or (F32,BF16): the last also rounds to the type the
 * tensor-core scan reads.  Rows must be whole 16-byte pieces (K % 4 == 0 for fp32, K % 8 == 0 for bf16),
 * at most 128 of them, and x / out 16-byte aligned; otherwise GRMX_ERR_UNSUPPORTED.  out may alias x
 * when the two types are equal.
 * Replaces F.normalize(key_proj(x)) / F.normalize(query_proj(x)) (grm/core/paper_grm.py:491-493, 301, 312);
 * the reference has no native counterpart.
 */
int grmx_normalize_rows(const void* x, void* out, int64_t N, int64_t K, float eps, int in_dtype, int out_dtype,
                        void* stream);

/*
 * Two 64-wide projections of the same input with the L2 normalisation in the epilogue, in one pass over x:
 *   out_a[n,:] = normalize(x[n,:] W[0:64,:]^T + bias[0:64]),  out_b[n,:] = normalize(x[n,:] W[64:128,:]^T + bias[64:128])
 * x bf16 [rows, D], weights bf16 [128, D] (the two weight matrices stacked), bias float32 [128] or NULL,
 * out_a / out_b bf16 [rows, 64]; normalize(y) = y / max(||y||_2, eps).  One tcgen05 product per tile of 128
 * rows with the stacked weights resident in shared memory; products accumulate in fp32 and the norm is taken
 * of the fp32 sums.  Covers K == 64 and D a multiple of 64 up to 512, 16-byte aligned tensors;
 * GRMX_ERR_UNSUPPORTED otherwise (project with a GEMM and call grmx_normalize_rows).
 * Replaces F.normalize(key_proj(x)) and F.normalize(query_proj(x)) (grm/core/paper_grm.py:491-493); the
 * reference has no native counterpart.
 */
int grmx_project_normalize(const void* x_bf16, const void* weights_bf16, const float* bias, void* out_a_bf16,
                           void* out_b_bf16, int64_t rows, int64_t D, int64_t K, float eps, void* stream);

/*
 * archive[b, slot, :] = memory[b, :] and, when archive_bf16 is not NULL, the same values rounded to
 * bf16 into archive_bf16[b, slot, :].  memory float32 [B,row_elems] (row_elems = H*K), archive float32
 * [B,S,row_elems], archive_bf16 bf16 [B,S,row_elems] or NULL.  One pass over the state: the bf16 ring is
 * what a caller multiplies with when it applies the queries of a segment to all archived matrices at once.
 * Follows the append of the reference's _BatchMemoryArchive (grm/core/paper_grm.py:31-44, 721-725) on a
 * preallocated device ring; the reference has no native counterpart.
 */
int grmx_archive_push(const float* memory, float* archive, void* archive_bf16, int64_t B, int64_t S,
                      int64_t slot, int64_t row_elems, void* stream);

/*
 * Device error word: bit 0 = gather index out of range, bit 1 = a bounded
 * wait inside a kernel gave up.  grmx_device_error_word copies the word of
 * the current device to *out (synchronises that stream); reset clears it.
 */
int grmx_device_error_word(uint32_t* out, void* stream);
int grmx_device_error_reset(void* stream);

/*
 * Self-test of the bounded waits: launches one small CTA whose warps wait, with the kernels' own
 * wait routine and a limit of `wait_limit` polls, on an mbarrier that nothing ever completes.
 * The wait gives up, the CTA-wide abort flag stops the other warps, bit 1 of the device error
 * word is set and the kernel returns: the context stays usable.  No counterpart in the reference.
 */
int grmx_selftest_bounded_wait(uint32_t wait_limit, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GRMX_H_ */
