// Parameter block shared by the two kernel families of the linear-memory scan.
#pragma once

#include "common.cuh"

namespace grmx {

struct ScanParams {
  const void* keys;      // [B,T,K] io dtype
  const void* values;    // [B,T,H] io dtype
  const void* queries;   // [B,T,K] io dtype
  const void* memory_in; // [B,H,K] state dtype, element strides below
  void* hidden_out;      // [B,T,H] io dtype
  void* memory_out;      // [B,H,K] state dtype, dense; may be null
  int64_t B, T, K, H;
  int64_t m_row_stride, m_col_stride;
  float decay;
  float update_coeff;
  float hidden_scale;
  float memory_out_scale;
  int reverse;
  int first_step_no_decay;
  // Optional: the state after every snap_chunks * 128 tokens (forward scans whose T is a multiple of
  // that), [H,K] fp32 dense at snapshots + b * snap_batch_stride + j * snap_stride (elements), scaled
  // like memory_out.  Only the warp-specialised tensor-core kernel writes them.
  float* snapshots = nullptr;
  int64_t snap_batch_stride = 0;
  int64_t snap_stride = 0;
  int snap_chunks = 0;
};

// fp32 CUDA-core scan: any K <= 256, any H, any T.
int launch_scan_ffma(const ScanParams& p, int io_dtype, int state_dtype, cudaStream_t stream);

// tcgen05 chunked scan: bf16 operands, fp32 state.  `why` receives the reason
// when the shape is outside what the tensor-core kernel covers.
bool scan_tcgen05_supported(const ScanParams& p, int io_dtype, int state_dtype, const char** why);
int launch_scan_tcgen05(const ScanParams& p, cudaStream_t stream);

// How a call is cut along T so that few batch rows still fill the GPU.  pieces == 1 means no cut.
struct SplitInfo {
  int pieces;              // CTAs per batch row
  int chunks_per_piece;    // 128-token chunks handled by each of them
  const float* partials;   // [B, pieces-1, subs, H, K] fp32: local state contribution of pieces
                           // 0..pieces-2, each as the sum of `subs` terms (computed by separate CTAs);
                           // nullptr with pieces > 1: every piece derives its start state itself
  int subs = 1;
  // Uneven pieces (only without partials): piece q owns chunks [starts[q], starts[q+1]).  A piece
  // that derives its own start state pays for every chunk before it, so later pieces are shorter.
  static constexpr int kMaxPieces = 64;
  int use_starts = 0;
  int starts[kMaxPieces + 1] = {0};
};

// Warp-specialised variant of the tcgen05 scan (d_k = d_v = 64); same coverage rules otherwise.
bool scan_tcgen05_pipe_supported(const ScanParams& p);
int launch_scan_tcgen05_pipe(const ScanParams& p, const SplitInfo& split, cudaStream_t stream);

// The same for heads of d_k = 128: one CTA per (row, 64 value features) with both key halves in one
// product, every q / k / v tile read once and every output tile written once.  Forward scans only.
bool scan_tcgen05_wide_supported(const ScanParams& p);
int launch_scan_tcgen05_wide(const ScanParams& p, cudaStream_t stream);

// Heads of d_k = 128 whose value width is a multiple of 128: one CTA per (row, 128 value features), so
// that q and k tiles also cross from L2 to the SMs once.  Forward scans only.
bool scan_tcgen05_square_supported(const ScanParams& p);
int launch_scan_tcgen05_square(const ScanParams& p, cudaStream_t stream);

// Cutting along T: bytes of scratch the cut needs for this call (0 when a cut would not help or
// the shape is not covered), and the launch that runs the piece-state kernel followed by the scan.
int64_t scan_tcgen05_split_scratch_bytes(const ScanParams& p, int sm_count = 0);   // 0: the current device
int launch_scan_tcgen05_split(const ScanParams& p, void* scratch, int64_t scratch_bytes, cudaStream_t stream);
// The same cut without a workspace: one launch, every piece derives its start state itself with a
// pre-pass over the chunks before its own (state recurrence only).  Falls back to the uncut scan
// when a cut does not apply.
int launch_scan_tcgen05_selfcut(const ScanParams& p, cudaStream_t stream);

}  // namespace grmx
