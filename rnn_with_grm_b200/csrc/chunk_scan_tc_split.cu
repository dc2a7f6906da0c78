// Cutting a scan along T so that a handful of batch rows still fills the GPU.
//
// The scan is linear in its start state, so a row can be cut into pieces that run as
// separate CTAs once every piece knows the state it starts from.  That state is
//   M_start(q+1) = decay^(tokens of piece q) * M_start(q) + L_q,
//   L_q = sum over the tokens j of piece q of coeff * decay^(n_q - 1 - step_j) v_j k_j^T,
// and L_q depends on k and v of piece q only.  `piece_state_kernel` below computes the
// L_q of every piece but the last, each as the sum of `subs` terms over consecutive runs of
// chunks so that this kernel fills the GPU too (one CTA per term: TMA-fed tcgen05.mma
// accumulating Vw^T Kc in TMEM, no rescaling between chunks because the decay of the whole
// piece is folded into the per-token weights) into a scratch buffer the caller provides; the
// scan kernel launched after it on the same stream rebuilds each piece's start state from
// memory_in and those L_q in its prologue.  Stream order is the only synchronisation
// between the two kernels: no CTA ever waits for another.
//
// Cost: k and v of all pieces but the last are read twice (the second time mostly from L2)
// and their Vw^T Kc products are computed twice.
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

using namespace tc;

constexpr int kChunk = 128;
constexpr int kD = 64;
constexpr int kStages = 3;
constexpr int kThreads = 192;          // warps 0-3: Vw passes + final read-out, warp 4: MMA, warp 5: TMA
constexpr int kMmaWarp = 4;
constexpr int kTmaWarp = 5;
constexpr uint32_t kTmemCols = 64;
constexpr int kTileBytes = kChunk * kD * 2;
constexpr int kStageBytes = 2 * kTileBytes;          // k, v
constexpr int kOffVw = kStages * kStageBytes;
constexpr int kOffBars = kOffVw + 2 * kTileBytes;
constexpr int kOffMisc = kOffBars + 16 * 8;
constexpr int kSmemAlloc = kOffMisc + 32 + 1024;

__global__ void __launch_bounds__(kThreads, 1)
piece_state_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   ScanParams p, SplitInfo split, float* partials, uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full = bars;            // [3]
  uint64_t* bar_stage_free = bars + 3;  // [3]
  uint64_t* bar_vw_ready = bars + 6;    // [2] 128 arrivals
  uint64_t* bar_d_done = bars + 8;      // [2] commit
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int64_t b = blockIdx.x % p.B;
  const int piece = static_cast<int>(blockIdx.x / p.B) / split.subs;
  const int sub = static_cast<int>(blockIdx.x / p.B) % split.subs;
  const int T = static_cast<int>(p.T);
  const bool rev = p.reverse != 0;
  // pieces before the last are full; this CTA covers chunks [sub_begin, sub_begin + n_chunks) of its piece
  const int per_sub = (split.chunks_per_piece + split.subs - 1) / split.subs;
  const int sub_begin = sub * per_sub;
  const int n_chunks = max(0, min(per_sub, split.chunks_per_piece - sub_begin));
  const int c_begin = piece * split.chunks_per_piece + sub_begin;
  const int piece_tokens = min(split.chunks_per_piece * kChunk, T - piece * split.chunks_per_piece * kChunk);
  auto chunk_len = [&](int c) { return min(kChunk, T - c * kChunk); };
  auto chunk_token0 = [&](int c) { return rev ? T - (c + 1) * kChunk : c * kChunk; };

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_stage_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_vw_ready[i], 128);
      mbar_init(&bar_d_done[i], 1);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  auto stage_k = [&](int s) { return smem + s * kStageBytes; };
  auto stage_v = [&](int s) { return smem + s * kStageBytes + kTileBytes; };
  auto vw_buf = [&](int i) { return smem + kOffVw + i * kTileBytes; };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  if (warp == kTmaWarp) {
    if (lane == 0) {
      int issued = 0;
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c % kStages;
        if (c >= kStages) GRMX_WAIT(&bar_stage_free[s], c / kStages - 1)
        mbar_expect_tx(&bar_full[s], kStageBytes);
        const int t0 = chunk_token0(c_begin + c);
        tma_load_3d(stage_k(s), &map_k, &bar_full[s], 0, t0, static_cast<int>(b));
        tma_load_3d(stage_v(s), &map_v, &bar_full[s], 0, t0, static_cast<int>(b));
        issued = c + 1;
      }
      if (*s_abort) {
        for (int c = issued > kStages ? issued - kStages : 0; c < issued; ++c) {
          mbar_wait_quiet(&bar_full[c % kStages], (c / kStages) & 1);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_m = make_idesc(kD, kD, 1, 1);
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c % kStages;
        GRMX_WAIT(&bar_vw_ready[c & 1], c / 2)
        tc_fence_after();
        const uint64_t dk_mn = smem_desc(smem_u32(stage_k(s)), kTileBytes, 1024);
        const uint64_t dvw = smem_desc(smem_u32(vw_buf(c & 1)), kTileBytes, 1024);
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk) {
          tc_mma_bf16(tmem_base, desc_add(dvw, kk * 2048), desc_add(dk_mn, kk * 2048), idesc_m,
                      (c > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&bar_d_done[c & 1]);
        tc_commit(&bar_stage_free[s]);
      }
    }
  } else {
    // ---- Vw passes, then the read-out of the accumulated contribution ----
    const int row = tid;
    const int step = rev ? kChunk - 1 - row : row;
    bool ok = true;
    for (int c = 0; c < n_chunks && ok; ++c) {
      ok = false;
      do {
        GRMX_WAIT(&bar_full[c % kStages], c / kStages)
        if (c >= 2) GRMX_WAIT(&bar_d_done[c & 1], c / 2 - 1)
        ok = true;
      } while (false);
      if (!ok) break;
      // weight of this token: every later token of the piece decays it once more
      const int later = piece_tokens - 1 - ((sub_begin + c) * kChunk + step);
      const float w = step < chunk_len(c_begin + c) ? p.update_coeff * powf(p.decay, static_cast<float>(later)) : 0.0f;
      scaled_row_copy(stage_v(c % kStages), vw_buf(c & 1), row, w);
      fence_proxy_async();
      mbar_arrive(&bar_vw_ready[c & 1]);
    }
    const int last = n_chunks - 1;
    float* out = partials +
                 (((b * (split.pieces - 1) + piece) * split.subs + sub) * kD + (warp * 16 + (lane & 15))) * kD;
    if (n_chunks == 0) {
      // a term without chunks (uneven division) contributes nothing
      if (lane < 16) {
        for (int j = 0; j < kD; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else if (ok && mbar_wait(&bar_d_done[last & 1], (last / 2) & 1, s_abort)) {
      tc_fence_after();
      // M = 64 accumulator: lanes 0-15 of each 32-lane quarter hold rows 16*warp + lane
      const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < kD; c0 += 32) {
        float v[32];
        tc_ld32(tmem_lane + c0, v);
        if (lane < 16) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            *reinterpret_cast<float4*>(out + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
        }
      }
    }
  }
#undef GRMX_WAIT

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *s_abort && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

int sm_count_of_current_device() {
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) cudaDeviceGetAttribute(&cached[device], cudaDevAttrMultiProcessorCount, device);
  return cached[device];
}

// Pieces per row: the largest power of two that still gives every piece two chunks or more and
// keeps rows x pieces within one wave of the GPU (one CTA per SM).
int pick_pieces(const ScanParams& p, int sms) {
  if (!scan_tcgen05_pipe_supported(p)) return 1;
  const int64_t n_chunks = (p.T + kChunk - 1) / kChunk;
  const int64_t ctas_per_piece = p.B * (p.H / kD);     // one CTA per row and 64-wide block of value features
  int pieces = 1;
  while (ctas_per_piece * pieces * 2 <= sms && n_chunks / (pieces * 2) >= 2) pieces *= 2;
  return pieces;
}

// Terms per piece state: the largest power of two that keeps the piece-state kernel within one
// wave and gives every term two chunks or more.
int pick_subs(const ScanParams& p, int pieces, int chunks_per_piece, int sms) {
  int subs = 1;
  while (p.B * (pieces - 1) * subs * 2 <= sms && chunks_per_piece / (subs * 2) >= 2) subs *= 2;
  return subs;
}

// the cut for this call on a device of `sms` multiprocessors (0: the current device); pieces == 1 when
// a cut does not apply
SplitInfo plan_split(const ScanParams& p, int sms = 0) {
  if (sms <= 0) sms = sm_count_of_current_device();
  const int64_t n_chunks = (p.T + kChunk - 1) / kChunk;
  SplitInfo split{1, static_cast<int>(n_chunks), nullptr, 1};
  const int pieces = pick_pieces(p, sms);
  if (pieces <= 1) return split;
  const int per_piece = static_cast<int>((n_chunks + pieces - 1) / pieces);
  if (static_cast<int64_t>(per_piece) * (pieces - 1) >= n_chunks) return split;   // every piece must own a chunk
  split.pieces = pieces;
  split.chunks_per_piece = per_piece;
  split.subs = pick_subs(p, pieces, per_piece, sms);
  return split;
}

}  // namespace

int64_t scan_tcgen05_split_scratch_bytes(const ScanParams& p, int sms) {
  if (p.K != kD || p.H != kD) return 0;                // the two-kernel cut exists for 64 x 64 heads only
  const SplitInfo split = plan_split(p, sms);
  if (split.pieces <= 1) return 0;
  return p.B * (split.pieces - 1) * split.subs * kD * kD * static_cast<int64_t>(sizeof(float));
}

namespace {

// Piece boundaries for the cut without a workspace.  Piece q runs the state recurrence alone over the
// chunks before it (cost kPrepassCost per chunk, measured relative to a full chunk) and then its own
// chunks, so equal pieces would leave the last one finishing long after the first.  Boundaries are
// chosen so that all pieces take about the same time: own(q) = own(0) - kPrepassCost * begin(q).
void balance_pieces(SplitInfo* split, int64_t n_chunks) {
  constexpr double kPrepassCost = 0.54;
  const int pieces = split->pieces;
  auto end_of = [&](double first) {         // where the last piece ends if piece 0 owns `first` chunks
    double begin = 0.0;
    for (int q = 0; q < pieces; ++q) begin += std::max(first - kPrepassCost * begin, 0.0);
    return begin;
  };
  double lo = 0.0, hi = static_cast<double>(n_chunks);
  for (int it = 0; it < 60; ++it) {
    const double mid = 0.5 * (lo + hi);
    (end_of(mid) < static_cast<double>(n_chunks) ? lo : hi) = mid;
  }
  const double first = hi;
  double begin = 0.0;
  split->starts[0] = 0;
  for (int q = 0; q < pieces; ++q) {
    begin += std::max(first - kPrepassCost * begin, 0.0);
    int edge = static_cast<int>(std::lround(begin));
    // every piece owns at least one chunk, and enough chunks are left for the pieces behind it
    edge = std::max(edge, split->starts[q] + 1);
    edge = std::min<int64_t>(edge, n_chunks - (pieces - 1 - q));
    split->starts[q + 1] = edge;
  }
  split->starts[pieces] = static_cast<int>(n_chunks);
  split->use_starts = 1;
}

}  // namespace

int launch_scan_tcgen05_selfcut(const ScanParams& p, cudaStream_t stream) {
  static const bool disabled = [] {
    const char* env = getenv("GRMX_SCAN_CUT");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  SplitInfo split = plan_split(p);
  if (disabled) split = SplitInfo{1, static_cast<int>((p.T + kChunk - 1) / kChunk), nullptr, 1};
  split.partials = nullptr;
  split.subs = 1;
  // Beyond four pieces the pre-pass of the last piece (more than half of the row) sets the time, and
  // every further piece only re-reads k and v once more.
  split.pieces = std::min(split.pieces, 4);
  if (split.pieces > 1) balance_pieces(&split, (p.T + kChunk - 1) / kChunk);
  return launch_scan_tcgen05_pipe(p, split, stream);
}

int launch_scan_tcgen05_split(const ScanParams& p, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
  const int64_t n_chunks = (p.T + kChunk - 1) / kChunk;
  SplitInfo split = plan_split(p);
  const int pieces = split.pieces;
  const int64_t need = p.B * (pieces - 1) * split.subs * kD * kD * static_cast<int64_t>(sizeof(float));
  if (pieces <= 1 || p.K != kD || p.H != kD || scratch == nullptr || scratch_bytes < need ||
      (reinterpret_cast<uintptr_t>(scratch) & 15u) != 0) {
    return launch_scan_tcgen05_selfcut(p, stream);
  }
  split.partials = static_cast<const float*>(scratch);

  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(piece_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "piece-state kernel: cannot reserve %d bytes of shared memory: %s", kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_k, map_v;
  if (!make_token_map(&map_k, p.keys, p.B, p.T, kD) || !make_token_map(&map_v, p.values, p.B, p.T, kD)) {
    return fail(GRMX_ERR_LAUNCH, "piece-state kernel: cuTensorMapEncodeTiled failed");
  }
  piece_state_kernel<<<static_cast<unsigned>(p.B * (pieces - 1) * split.subs), kThreads, kSmemAlloc, stream>>>(
      map_k, map_v, p, split, static_cast<float*>(scratch), device_error_word_ptr());
  int rc = check_launch("piece_state_kernel");
  if (rc != GRMX_OK) return rc;
  return launch_scan_tcgen05_pipe(p, split, stream);
}

}  // namespace grmx

// ---------------------------------------------------------------------------------------
// Entry point for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs the scan: a serving
// loop that has handed all of the device memory to its own pool, code running inside a
// real-time callback where an allocation may block on the driver, or a plugin sandbox that is
// only given the buffers of its inputs and outputs.  For them the workspace of the T-cut scan
// lives in the library image instead: a fixed array in device memory, reserved on every GPU
// that loads the library for as long as the process lives.
namespace grmx {
namespace {

constexpr int64_t kStaticScratchBytes = 4ll << 20;   // 4 MiB = 256 piece states of 64 x 64 fp32
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so the address is asked for once
// per device (with that device current) and remembered.
int static_scratch_address(float** out) {
  static std::mutex mutex;
  static float* cached[64] = {nullptr};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= 64) {
    return fail(GRMX_ERR_DEVICE, "grmx_chunk_scan_fwd_static: no usable current device");
  }
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return fail(GRMX_ERR_DEVICE, "grmx_chunk_scan_fwd_static: cudaGetSymbolAddress failed: %s",
                  cudaGetErrorString(err));
    }
    cached[device] = static_cast<float*>(ptr);
  }
  *out = cached[device];
  return GRMX_OK;
}

// The one comparison that decides whether a call fits the built-in workspace.
int static_scratch_admit(int64_t need_bytes, const char* who) {
  if (need_bytes > kStaticScratchBytes) {
    return fail(GRMX_ERR_UNSUPPORTED,
                "%s: this call needs %lld bytes of workspace, the built-in one holds %lld; use "
                "grmx_chunk_scan_fwd_ws with a buffer of your own or fewer rows per call",
                who, (long long)need_bytes, (long long)kStaticScratchBytes);
  }
  return GRMX_OK;
}

}  // namespace
}  // namespace grmx

extern "C" int64_t grmx_static_scratch_capacity(void) { return grmx::kStaticScratchBytes; }

extern "C" int grmx_static_scratch_admits(int64_t need_bytes) {
  if (need_bytes < 0) return grmx::fail(GRMX_ERR_ARG, "grmx_static_scratch_admits: negative size");
  return grmx::static_scratch_admit(need_bytes, "grmx_static_scratch_admits");
}

extern "C" int64_t grmx_chunk_scan_scratch_bytes_on(int64_t B, int64_t T, int64_t K, int64_t H, int sm_count) {
  if (B <= 0 || T <= 0 || K <= 0 || H <= 0 || sm_count <= 0) return 0;
  grmx::ScanParams p = {};
  p.B = B; p.T = T; p.K = K; p.H = H;
  return grmx::scan_tcgen05_split_scratch_bytes(p, sm_count);
}

extern "C" int grmx_chunk_scan_fwd_static(const void* keys, const void* values, const void* queries,
                                          const void* memory_in, void* hidden_out, void* memory_out,
                                          int64_t B, int64_t T, int64_t K, int64_t H, float decay,
                                          void* stream) {
  using namespace grmx;
  const char* who = "grmx_chunk_scan_fwd_static";
  GRMX_REQUIRE(B >= 0 && T >= 0 && K > 0 && H > 0, "%s: bad sizes", who);
  if (B == 0) return GRMX_OK;
  GRMX_REQUIRE(T > 0, "%s: T must be positive", who);
  GRMX_REQUIRE(keys && values && queries && memory_in && hidden_out && memory_out, "%s: NULL tensor pointer", who);
  ScanParams p;
  p.keys = keys; p.values = values; p.queries = queries; p.memory_in = memory_in;
  p.hidden_out = hidden_out; p.memory_out = memory_out;
  p.B = B; p.T = T; p.K = K; p.H = H;
  p.m_row_stride = K; p.m_col_stride = 1;
  p.decay = decay; p.update_coeff = (1.0f - decay) * (1.0f / sqrtf(static_cast<float>(K)));
  p.hidden_scale = 1.0f; p.memory_out_scale = 1.0f; p.reverse = 0; p.first_step_no_decay = 0;
  const char* why = "";
  if (!scan_tcgen05_supported(p, GRMX_BF16, GRMX_F32, &why)) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: only the bf16 tensor-core scan is offered here: %s", who, why);
  }
  int rc = static_scratch_admit(scan_tcgen05_split_scratch_bytes(p), who);
  if (rc != GRMX_OK) return rc;
  float* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != GRMX_OK) return rc;
  return launch_scan_tcgen05_split(p, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

