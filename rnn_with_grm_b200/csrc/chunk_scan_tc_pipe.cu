// Warp-specialised, pipelined tcgen05 kernel of the linear-memory scan
// (d_k = d_v = 64, bf16 operands, fp32 state in registers, chunks of 128 tokens).
//
// Per chunk c, with Q, Kc, Vc the chunk's [128 x 64] tiles and M the carried state:
//
//   [S | R] = Q [Kc ; Mb]^T       128 x 192 x 64, one product: S = Q Kc^T, R = Q Mb^T, Mb = bf16(M_{c-1})
//   U  = Vw^T Kc                  Vw_j = coeff * decay^(len-1-j) v_j       (the chunk's own contribution)
//   A  = P Vc                     P_ij = hs * coeff * decay^(i-j) S_ij (j <= i)         TMEM x smem
//   M  = decay^len M + U          fp32 FMA in registers
//   out_i = hs * decay^(i+1) R_i + A_i                                    fp32, in the epilogue
//
// which is the closed form of the reference chunk (grm/core/cuda_ops.py:218-254) with the state
// carried across chunks as in grm/csrc/grm_cuda.cpp:67-83.  No tensor-core product waits for a
// tensor-core product of the chunk before it except through the state, and the state costs one
// register FMA and one shared-memory store per chunk: the rest is a pipeline.  Roles:
//
//   warp 20      issuer A: [S | R]_c; owns the TMEM allocation
//   warp 21      issuer B: U_c, up to two chunks ahead
//   warp 22      issuer C: A_c
//   warp 23      loader: TMA ring of three stages, refilled as soon as a chunk's tiles are dead
//                (issuers run as whole warps with one elected lane executing the instruction)
//   warps 16-19  state group: Vw_c, the decay-scaled copy of V; the state, one row per thread in
//                lanes 0-15 of each warp (the layout of a 64-row accumulator),
//                M_c = decay^len M_{c-1} + U_c, and its bf16 copy behind the K tile of chunk c+1
//   warps 0-7    P groups 0 and 1: S_c -> P_c (decay mask, bf16, written back into the TMEM
//                columns of S_c), two 32-column blocks per group
//   warps 8-15   epilogue groups 2 and 3: R_c, A_c -> out -> shared memory -> TMA store, 32 output
//                columns per group; runs beside the P pass of the next chunk
//
// P never touches shared memory: A = P Vc takes its left operand from TMEM.  Shared memory holds
// three stages [q | k | Mb | v] (the state copy sits right behind k so that [Kc ; Mb] is one
// operand) and two Vw buffers.  TMEM (512 columns): two buffers of 192 columns
// [S -> P (0-63) , A (64-127) | R (128-191)], used by alternate chunks, and two U buffers.  Every
// hand-off is an mbarrier; a waiter is never more than one phase behind its producer (protocol
// comment in the kernel) and every wait is bounded: on expiry the CTA-wide abort flag is raised,
// all roles drain, the error word gets bit 1, TMEM is freed and the kernel returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

using namespace tc;

constexpr int kChunk = 128;
constexpr int kD = 64;                 // d_k == d_v
constexpr int kStages = 3;
constexpr int kThreads = 768;          // 24 warps; registers are re-divided between the roles at entry
constexpr int kComputeGroups = 4;      // warps 0-15, four per group
constexpr int kComputeThreads = kComputeGroups * 128;
constexpr int kStateWarp0 = 16;        // warps 16-19
constexpr int kStateThreads = 128;
constexpr int kIssuerA = 20;           // [S | R]; also owns the TMEM allocation
constexpr int kIssuerB = 21;           // U
constexpr int kIssuerC = 22;           // A = P V
constexpr int kLoader = 23;            // TMA
// registers per thread after the re-division (768 threads start with 80 each)
constexpr int kRegsCompute = 72;
constexpr int kRegsState = 128;
constexpr int kRegsIssue = 40;
// setmaxnreg.inc can only take what the other warps of the CTA have released with setmaxnreg.dec (it
// blocks until then), so the books have to balance within the launch allocation
constexpr int kRegsLaunch = 80;        // 65536 / 768, rounded down to a multiple of 8
static_assert(kComputeThreads * kRegsCompute + kStateThreads * kRegsState + 128 * kRegsIssue <= kThreads * kRegsLaunch,
              "the state group would wait for registers that nobody releases");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColBuf = 0;        // + 192 * (c & 1): S (0-127) -> P (0-63, bf16 pairs), A (64-127), R (128-191)
constexpr uint32_t kBufCols = 192;
constexpr uint32_t kColA = 64;         // within a buffer
constexpr uint32_t kColR = 128;        // within a buffer
constexpr uint32_t kColU = 384;        // + 64 * (c & 1): U, lanes 0-15 of each quarter

constexpr int kTileBytes = kChunk * kD * 2;          // 16 KiB: one [128 x 64] bf16 tile
constexpr int kMbBytes = kD * kD * 2;                // 8 KiB: [64 x 64] bf16
constexpr int kStageQ = 0;
constexpr int kStageK = kTileBytes;
constexpr int kStageMb = 2 * kTileBytes;             // directly behind k
constexpr int kStageV = 2 * kTileBytes + kMbBytes;
constexpr int kStageBytes = 3 * kTileBytes + kMbBytes;
constexpr int kTxBytes = 3 * kTileBytes;             // what TMA delivers per stage
constexpr int kOffStage = 0;
constexpr int kOffVw = kStages * kStageBytes;        // two buffers
// Decay weights of P, reversed (entry m holds weight(d = 127 - m), zero for d < 0) and stored as
// four copies shifted by 0..3 entries so that any run of 32 weights can be read with aligned
// 16-byte loads; copies are 264 floats apart, which keeps the eight lanes of a load phase on
// distinct banks.
constexpr int kWcopy = 264;
constexpr int kOutBytes = kChunk * 32 * 2;             // 8 KiB: [128 x 32] bf16, one per compute group
constexpr int kOffOut = kOffVw + 2 * kTileBytes;
constexpr int kOffWtab = kOffOut + 2 * kOutBytes;
constexpr int kOffPow = kOffWtab + 4 * kWcopy * 4;   // float[kChunk + 4]: decay^j
constexpr int kOffBars = kOffPow + (kChunk + 4) * 4;
constexpr int kNumBars = 36;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemTotal = kOffMisc + 32;
constexpr int kSmemAlloc = kSmemTotal + 1024;
static_assert(kSmemAlloc <= 232448, "shared memory plan exceeds 227 KiB");
static_assert(kStageBytes % 1024 == 0 && kStageMb % 1024 == 0 && kStageV % 1024 == 0, "swizzle atoms are 1 KiB");

// 16-byte load through the coherent path (ld.global, never ld.global.nc)
__device__ __forceinline__ float4 ld_coherent_f4(const float4* ptr) {
  float4 v;
  asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr) : "memory");
  return v;
}

// descriptor + byte offset (the start-address field holds addr >> 4 in its low 14 bits)

// kSnapshots: also write the state at segment ends (ScanParams::snapshots).  A variant of its own:
// the test in the state group's loop costs the plain scan a tenth of its speed.
template <bool kSnapshots>
__global__ void __launch_bounds__(kThreads, 1)
linear_scan_tc_pipe_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                           ScanParams p, SplitInfo split, int x_k, int accumulate_out,
                           uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_wtab = reinterpret_cast<float*>(smem + kOffWtab);
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full = bars;              // [3] TMA bytes landed                             (1 + tx)
  uint64_t* bar_s_done = bars + 4;        // [2] [S | R]_c complete                           (commit)
  uint64_t* bar_p_ready = bars + 6;       // [2] P_c in TMEM                                  (256)
  uint64_t* bar_vw_ready = bars + 8;      // [2] Vw_c written                                 (128)
  uint64_t* bar_u_done = bars + 10;       // [2] U_c complete                                 (commit)
  uint64_t* bar_a_done = bars + 12;       // [2] A_c complete                                 (commit)
  uint64_t* bar_buf_free = bars + 14;     // [2] epilogue c has read R_c and A_c              (256)
  uint64_t* bar_mb_ready = bars + 16;     // [3] bf16 copy of the state before chunk c        (128)
  uint64_t* bar_u_free = bars + 20;       // [2] U_c folded into the state                    (128)
  uint64_t* bar_stage_free = bars + 22;   // [3] U_c and A_c complete: the tiles of chunk c are dead (2)
  uint64_t* bar_s_read = bars + 26;       // [2] P group 0 has S block 1 in registers         (128)
  uint64_t* bar_out_ready = bars + 30;    // [2] epilogue group h has written its half of the output tile (128)
  uint64_t* bar_out_free = bars + 32;     // [2] the store of that half tile has read it      (1)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // The call may be cut along T into `split.pieces` pieces of `split.chunks_per_piece` chunks, one
  // CTA per (piece, row), piece-major.  Piece q > 0 starts from the state that the pieces before it
  // leave behind, rebuilt in its prologue from memory_in and their local contributions in
  // `split.partials` (written by the piece-state kernel that runs before this one).
  // Heads wider than 64 run as 64 x 64 blocks of the state, which are independent recurrences:
  // block (vb, a) scans the value features 64vb.. against the key/query features x_k = 64a.., and the
  // outputs of the blocks of one vb add up (one launch per a; launches after the first add to what
  // is there).  The value block is the fastest index of the grid, so the CTAs that read the same
  // q and k tiles are neighbours in time and share them through L2.
  const int n_vb = static_cast<int>(p.H / kD);
  const int vb = static_cast<int>(blockIdx.x % n_vb);
  const int64_t b = (blockIdx.x / n_vb) % p.B;
  const int piece = static_cast<int>(blockIdx.x / n_vb / p.B);
  const int x_v = vb * kD;
  const int T = static_cast<int>(p.T);
  const int total_chunks = (T + kChunk - 1) / kChunk;
  const int c_begin = split.use_starts ? split.starts[piece] : piece * split.chunks_per_piece;
  const int n_chunks = split.use_starts ? split.starts[piece + 1] - c_begin
                                        : min(split.chunks_per_piece, total_chunks - c_begin);   // chunks this CTA writes
  // Without the states of the earlier pieces (split.partials == nullptr) the CTA derives its start
  // state itself: a pre-pass over the `pre` chunks before its own runs only the state recurrence on
  // them (k and v tiles, Vw, U, the register update) and none of the per-token work.  Local chunk
  // index c covers pre-pass and own chunks alike, c = 0 .. n_all-1, global chunk g0 + c; the roles
  // and barriers that exist only for own chunks count them as f = c - pre.
  const int pre = (split.partials == nullptr) ? c_begin : 0;
  const int n_all = pre + n_chunks;
  const int g0 = c_begin - pre;
  const bool rev = p.reverse != 0;
  // Global chunk g covers processing steps [128g, 128g + len).  Forward, tile row r is step r of
  // the chunk; in a reverse scan the tile is still loaded in memory order, so row r is step
  // 127 - r and the tile of a short last chunk starts at a negative token (TMA fills with 0).
  auto chunk_len = [&](int g) { return min(kChunk, T - g * kChunk); };
  auto chunk_token0 = [&](int g) { return rev ? T - (g + 1) * kChunk : g * kChunk; };
  auto first_offset = [&](int g) { return (g == 0 && p.first_step_no_decay) ? 1 : 0; };

  // ---- set-up (all threads) ----
  // Launched as a programmatic dependent of the kernel before it in the stream (see the host side),
  // this grid may start while that kernel is still running: the set-up below touches no global
  // memory, and everything after it sits behind griddepcontrol.wait, which returns once the earlier
  // grid has completed and its writes are visible.  The first instruction lets the grid AFTER this
  // one do the same; it takes effect when every CTA of this grid has issued it, i.e. is resident.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_mb_ready[i], kStateThreads);
      mbar_init(&bar_stage_free[i], 2);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s_done[i], 1);
      mbar_init(&bar_p_ready[i], 256);
      mbar_init(&bar_s_read[i], 128);
      mbar_init(&bar_out_ready[i], 128);
      mbar_init(&bar_out_free[i], 1);
      mbar_init(&bar_vw_ready[i], kStateThreads);
      mbar_init(&bar_u_done[i], 1);
      mbar_init(&bar_a_done[i], 1);
      mbar_init(&bar_buf_free[i], 256);
      mbar_init(&bar_u_free[i], kStateThreads);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int j = tid; j <= kChunk; j += kThreads) s_pow[j] = powf(p.decay, static_cast<float>(j));
  for (int j = tid; j < 4 * kWcopy; j += kThreads) {
    const int copy = j / kWcopy;
    const int m = j % kWcopy + copy;           // forward: weight(row - col), reverse: weight(col - row)
    const int d = rev ? m - 127 : 127 - m;
    s_wtab[j] = d >= 0 ? p.hidden_scale * p.update_coeff * powf(p.decay, static_cast<float>(d)) : 0.0f;
  }
  if (warp == kIssuerA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  asm volatile("griddepcontrol.wait;" ::: "memory");   // no-op for a launch without the attribute

  auto stage = [&](int c) { return smem + kOffStage + (c % kStages) * kStageBytes; };
  auto vw_buf = [&](int c) { return smem + kOffVw + (c & 1) * kTileBytes; };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  // Protocol.  Chunks are numbered locally, c = 0 .. n_all-1; "X(c)" is the completion of barrier
  // X that belongs to chunk c (phase c/2 of X[c&1], phase c/3 of X[c%3]).  Barriers that only own
  // chunks use (s_done, p_ready, a_done, buf_free, mb_ready, s_read, out_*) count f = c - pre instead;
  // below, c stands for f on those.  A pre-pass chunk involves the loader, issuer B and the state
  // group only, and the state group makes both arrivals on its stage_free.  A waiter is
  // never more than one completion behind, because the producer's next completion on the same
  // barrier needs something that comes after the waiter's wait:
  //   loader:   TMA of c    needs stage_free(c-3): one arrival after u_done(c-3) (state group), one
  //                         after a_done(c-3) (issuer C), which also follows [S | R]_{c-3}
  //   issuer A: [S | R]_c   needs full(c), mb_ready(c), buf_free(c-2)
  //   state:    Vw_c        needs full(c) and u_done(c-2) (waited for M_{c-2}, earlier in program order)
  //             M_c         needs u_done(c); its bf16 copy goes behind the K tile of chunk c+1, whose
  //                         stage is known to be free because full(c+1) was waited for Vw_{c+1}
  //   issuer B: U_c         needs vw_ready(c), u_free(c-2)
  //   issuer C: A_c         needs p_ready(c)
  //   P pass c  needs s_done(c) (group 1 also s_read(c) before it stores); epilogue c needs a_done(c)
  // mb_ready has three barriers (X[c%3], phase c/3): mb_ready(c+3) follows Vw_{c+3} in the state
  // group's program order, hence the TMA of chunk c+3, hence a_done(c) and [S | R]_c, which issuer
  // A issues after passing mb_ready(c); with two barriers the loads of the prologue would leave a
  // window.

  // The register file is re-divided at the top of each role (setmaxnreg works on groups of four
  // warps): the state group keeps a 64-register state row per thread, the compute groups need
  // little more than one 32-column block, the issuers next to nothing.
  if (warp >= kIssuerA) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
  if (warp == kIssuerA) {
    // ===================================================================== issuer A: [S | R]
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_sr = make_idesc(kChunk, kChunk + kD, 0, 0);
    for (int f = 0; f < n_chunks; ++f) {
      const int c = pre + f;
      GRMX_WAIT(&bar_mb_ready[f % 3], f / 3)
      GRMX_WAIT(&bar_full[c % kStages], c / kStages)
      if (f >= 2) GRMX_WAIT(&bar_buf_free[f & 1], f / 2 - 1)
      tc_fence_after();
      const uint8_t* st = stage(c);
      const uint64_t dq = smem_desc(smem_u32(st + kStageQ), 16, 1024);
      const uint64_t dkm = smem_desc(smem_u32(st + kStageK), 16, 1024);   // 128 rows of k, then 64 of Mb
      const uint32_t d_tmem = tmem_base + kColBuf + kBufCols * (f & 1);
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        tc_mma_bf16_if(leader, d_tmem, desc_add(dq, kk * 32), desc_add(dkm, kk * 32), idesc_sr, kk > 0);
      }
      tc_commit_if(leader, &bar_s_done[f & 1]);
    }
  } else if (warp == kLoader) {
    // ===================================================================== loader: TMA ring
    const uint32_t leader = elect_one();
    int loads_issued = 0;
    for (int c = 0; c < n_all; ++c) {
      if (c >= kStages) GRMX_WAIT(&bar_stage_free[c % kStages], c / kStages - 1)
      uint8_t* st = stage(c);
      uint64_t* bar = &bar_full[c % kStages];
      const bool own = c >= pre;                      // the pre-pass needs no queries
      mbar_expect_tx_if(leader, bar, own ? kTxBytes : 2 * kTileBytes);
      const int t0 = chunk_token0(g0 + c);
      if (own) tma_load_3d_if(leader, st + kStageQ, &map_q, bar, x_k, t0, static_cast<int>(b));
      tma_load_3d_if(leader, st + kStageK, &map_k, bar, x_k, t0, static_cast<int>(b));
      tma_load_3d_if(leader, st + kStageV, &map_v, bar, x_v, t0, static_cast<int>(b));
      loads_issued = c + 1;
    }
    if (*s_abort) {
      // let the copies still in flight land before the shared memory is released
      for (int c = loads_issued > kStages ? loads_issued - kStages : 0; c < loads_issued; ++c) {
        mbar_wait_quiet(&bar_full[c % kStages], (c / kStages) & 1);
      }
    }
  } else if (warp == kIssuerB) {
    // ===================================================================== issuer B: U
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_u = make_idesc(kD, kD, 1, 1);
    for (int c = 0; c < n_all; ++c) {
      GRMX_WAIT(&bar_vw_ready[c & 1], c / 2)
      if (c >= 2) GRMX_WAIT(&bar_u_free[c & 1], c / 2 - 1)
      tc_fence_after();
      const uint64_t dvw = smem_desc(smem_u32(vw_buf(c)), kTileBytes, 1024);
      const uint64_t dk_mn = smem_desc(smem_u32(stage(c) + kStageK), kTileBytes, 1024);
      const uint32_t u_tmem = tmem_base + kColU + 64u * (c & 1);
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        tc_mma_bf16_if(leader, u_tmem, desc_add(dvw, kk * 2048), desc_add(dk_mn, kk * 2048), idesc_u, kk > 0);
      }
      tc_commit_if(leader, &bar_u_done[c & 1]);
    }
  } else if (warp == kIssuerC) {
    // ===================================================================== issuer C: A = P V
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_a = make_idesc(kChunk, kD, 0, 1);
    for (int f = 0; f < n_chunks; ++f) {
      const int c = pre + f;
      GRMX_WAIT(&bar_p_ready[f & 1], f / 2)
      tc_fence_after();
      const uint64_t dv_mn = smem_desc(smem_u32(stage(c) + kStageV), kTileBytes, 1024);
      const uint32_t buf = tmem_base + kColBuf + kBufCols * (f & 1);    // P: 16 tokens = 8 columns
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        tc_mma_bf16_ts_if(leader, buf + kColA, buf + 8u * kk, desc_add(dv_mn, kk * 2048), idesc_a, kk > 0);
      }
      tc_commit_if(leader, &bar_a_done[f & 1]);
      // The next P pass is a whole chunk period away, so this warp has the time to see A_c finish
      // and to hand the stage back to the loader at once.
      GRMX_WAIT(&bar_a_done[f & 1], f / 2)
      if (leader) mbar_arrive(&bar_stage_free[c % kStages]);
    }
  }
  } else if (warp >= kStateWarp0) {
    // ===================================================================== state group (warps 16-19)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsState));
    const int row = tid - kStateWarp0 * 32;   // token row of the copy
    const int step = rev ? kChunk - 1 - row : row;
    const int quarter = warp - kStateWarp0;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const bool owns_row = lane < 16;          // 64-row accumulator: lanes 0-15 of each quarter
    const int state_row = quarter * 16 + (lane & 15);
    float m[kD];                              // state row, fp32

    auto write_mb = [&](int c) {              // the state before chunk c, behind that chunk's K tile
      uint8_t* mrow = stage(c) + kStageMb + state_row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint4 w;
        w.x = pack_bf16(m[ch * 8 + 0], m[ch * 8 + 1]);
        w.y = pack_bf16(m[ch * 8 + 2], m[ch * 8 + 3]);
        w.z = pack_bf16(m[ch * 8 + 4], m[ch * 8 + 5]);
        w.w = pack_bf16(m[ch * 8 + 6], m[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(mrow + ((ch ^ (state_row & 7)) * 16)) = w;
      }
    };
    auto copy_chunk = [&](int c) {
      const int g = g0 + c;
      const int len = chunk_len(g);
      const float w_v = step < len ? p.update_coeff * s_pow[len - 1 - step] : 0.0f;
      scaled_row_copy<4>(stage(c) + kStageV, vw_buf(c), row, w_v);
      fence_proxy_async();
      mbar_arrive(&bar_vw_ready[c & 1]);
    };

    // state at the start of this CTA's chunks
    {
      const float* m_in = static_cast<const float*>(p.memory_in) + b * p.H * p.K;
      const float* src = m_in + (x_v + state_row) * p.m_row_stride + x_k * p.m_col_stride;
      const bool vec = p.m_col_stride == 1 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
      // Plain (coherent) loads: as a programmatic dependent this grid is alive while the grid before it
      // still writes memory_in (a state carried from call to call) and the piece states, so the
      // read-only data path, which assumes the data never changes during the kernel, is not used.
      if (owns_row && vec) {
#pragma unroll
        for (int j = 0; j < kD / 4; ++j) {
          const float4 x = ld_coherent_f4(reinterpret_cast<const float4*>(src) + j);
          m[4 * j] = x.x; m[4 * j + 1] = x.y; m[4 * j + 2] = x.z; m[4 * j + 3] = x.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < kD; ++j) m[j] = owns_row ? src[j * p.m_col_stride] : 0.0f;
      }
      // pieces before this one: M <- decay^(tokens of piece q - offset) M + partial_q
      for (int q = 0; q < piece && split.partials != nullptr; ++q) {
        const int q_tokens = min(split.chunks_per_piece * kChunk, T - q * split.chunks_per_piece * kChunk);
        const float gq = powf(p.decay, static_cast<float>(q_tokens - first_offset(q * split.chunks_per_piece)));
        if (owns_row) {
#pragma unroll
          for (int j = 0; j < kD; ++j) m[j] *= gq;
          for (int sub = 0; sub < split.subs; ++sub) {
            const float4* part = reinterpret_cast<const float4*>(
                split.partials + (((b * (split.pieces - 1) + q) * split.subs + sub) * kD + state_row) * kD);
#pragma unroll
            for (int j = 0; j < kD / 4; ++j) {
              const float4 x = ld_coherent_f4(part + j);
              m[4 * j] += x.x;
              m[4 * j + 1] += x.y;
              m[4 * j + 2] += x.z;
              m[4 * j + 3] += x.w;
            }
          }
        }
      }
      if (pre == 0) {
        if (owns_row) write_mb(0);            // TMA never writes this part of a stage
        fence_proxy_async();
        mbar_arrive(&bar_mb_ready[0]);        // completion 0: the state before the first own chunk
      }
    }

    do {
      GRMX_WAIT(&bar_full[0], 0)
      copy_chunk(0);
      if (n_all > 1) {
        GRMX_WAIT(&bar_full[1], 0)
        copy_chunk(1);
      }
      for (int c = 0; c < n_all; ++c) {
        const bool last = c + 1 == n_all;
        // ---- M_c = decay^len M_{c-1} + U_c ----
        GRMX_WAIT(&bar_u_done[c & 1], c / 2)
        // a pre-pass chunk has no A product: both arrivals of its stage come from here
        if (row == 0 || (row == 1 && c < pre)) mbar_arrive(&bar_stage_free[c % kStages]);
        tc_fence_after();
        {
          const float carry = s_pow[chunk_len(g0 + c) - first_offset(g0 + c)];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t u[32];
            tc_ld32_async(tmem_lane + kColU + 64u * (c & 1) + 32u * half, u);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) m[32 * half + j] = fmaf(carry, m[32 * half + j], __uint_as_float(u[j]));
          }
        }
        tc_fence_before();
        mbar_arrive(&bar_u_free[c & 1]);
        if constexpr (kSnapshots) {
        if (c >= pre && owns_row && (g0 + c + 1) % p.snap_chunks == 0) {
          // a segment ends with this chunk: its state goes to the caller's archive
          float* snap = p.snapshots + b * p.snap_batch_stride + ((g0 + c + 1) / p.snap_chunks - 1) * p.snap_stride +
                        (x_v + state_row) * p.K + x_k;
#pragma unroll
          for (int j = 0; j < kD; j += 4) {
            *reinterpret_cast<float4*>(snap + j) =
                make_float4(m[j] * p.memory_out_scale, m[j + 1] * p.memory_out_scale, m[j + 2] * p.memory_out_scale,
                            m[j + 3] * p.memory_out_scale);
          }
        }
        }
        if (!last) {
          if (c + 1 >= pre) {                 // the next chunk is an own chunk: [S | R] needs the state
            if (owns_row) write_mb(c + 1);
            fence_proxy_async();
            mbar_arrive(&bar_mb_ready[(c + 1 - pre) % 3]);
          }
        } else if (owns_row && p.memory_out != nullptr && piece + 1 == split.pieces) {
          float* m_out = static_cast<float*>(p.memory_out) + b * p.H * p.K + (x_v + state_row) * p.K + x_k;
#pragma unroll
          for (int j = 0; j < kD; j += 4) {
            float4 o;
            o.x = m[j] * p.memory_out_scale;
            o.y = m[j + 1] * p.memory_out_scale;
            o.z = m[j + 2] * p.memory_out_scale;
            o.w = m[j + 3] * p.memory_out_scale;
            *reinterpret_cast<float4*>(m_out + j) = o;
          }
        }
        // ---- Vw of chunk c+2 into the buffer that U_c has read ----
        if (c + 2 < n_all) {
          GRMX_WAIT(&bar_full[(c + 2) % kStages], (c + 2) / kStages)
          copy_chunk(c + 2);
        }
      }
    } while (false);
  } else {
    // ===================================================================== compute groups (warps 0-15)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsCompute));
    // Groups 0 and 1 turn S into P, groups 2 and 3 write the output: the P pass of chunk c+1 and
    // the epilogue of chunk c run side by side.  Warp w of a group owns rows 32w .. 32w+31.
    const int g = warp >> 2;
    const int quarter = warp & 3;
    const int row = tid & 127;                // token row within the chunk == TMEM lane
    const int step = rev ? kChunk - 1 - row : row;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kColBuf;

    if (g < 2) {
      // ---- P groups: group g turns the 32-column blocks 2g and 2g+1 of S into P ----
      // Blocks above block w (below it in a reverse scan) are all zero.  P block blk (16 packed
      // columns) lands on S columns 16*blk .. 16*blk+15: group 0 overwrites S block 0 after
      // reading it; group 1 overwrites S block 1, which group 0 reads second, and waits for
      // s_read(c) before it stores.
      for (int f = 0; f < n_chunks; ++f) {
        const uint32_t buf_row = lane_base + kBufCols * (f & 1);
        GRMX_WAIT(&bar_s_done[f & 1], f / 2)
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int blk = 2 * g + k;
          const bool nz = rev ? blk >= quarter : blk <= quarter;
          uint32_t sv[32], pk[16];
          if (nz) {
            tc_ld32_async(buf_row + 32u * blk, sv);
            tc_wait_ld();
          }
          if (g == 0 && k == 1) {
            tc_fence_before();
            mbar_arrive(&bar_s_read[f & 1]);
          }
          if (nz) {
            const int m0 = 127 - row + 32 * blk;            // reversed-table index of column 32*blk
            const float4* wv = reinterpret_cast<const float4*>(s_wtab + (m0 & 3) * kWcopy + (m0 & ~3));
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const float4 w4 = wv[t];
              pk[2 * t] = pack_bf16(__uint_as_float(sv[4 * t]) * w4.x, __uint_as_float(sv[4 * t + 1]) * w4.y);
              pk[2 * t + 1] = pack_bf16(__uint_as_float(sv[4 * t + 2]) * w4.z, __uint_as_float(sv[4 * t + 3]) * w4.w);
            }
          } else {
#pragma unroll
            for (int t = 0; t < 16; ++t) pk[t] = 0u;
          }
          if (g == 1 && k == 0) {
            GRMX_WAIT(&bar_s_read[f & 1], f / 2)
          }
          tc_st16_async(buf_row + 16u * blk, pk);
        }
        if (*s_abort) break;
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bar_p_ready[f & 1]);
      }
    } else {
      // ---- epilogue groups: group 2+h writes the output columns 32h .. 32h+31 ----
      // out_i = hs * decay^(i+1) R_i + A_i -> bf16 -> HBM.  The half tile goes out as one TMA store
      // from shared memory (plain 16-byte stores at a 128-byte stride cost the load/store unit one
      // line per lane).  A store may not start at a negative token, which the short last chunk of
      // a reverse scan does: that one is written with plain stores.  The hand-offs run for every
      // chunk so that phases stay e.
      const int h = g - 2;
      uint8_t* s_out = smem + kOffOut + h * kOutBytes;
      for (int e = 0; e < n_chunks; ++e) {
        const uint32_t buf_row = lane_base + kBufCols * (e & 1);
        GRMX_WAIT(&bar_a_done[e & 1], e / 2)
        tc_fence_after();
        const int ge = c_begin + e;           // global chunk (own chunks start at c_begin whatever the pre-pass)
        const bool row_live = step < chunk_len(ge);
        const float r_scale = row_live ? p.hidden_scale * s_pow[step + 1 - first_offset(ge)] : 0.0f;
        const int t0 = chunk_token0(ge);
        const bool by_tma = t0 >= 0;
        if (e >= 1) {
          if (row == 0) {
            bulk_wait_read();
            mbar_arrive(&bar_out_free[h]);
          }
          GRMX_WAIT(&bar_out_free[h], e - 1)
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t av[16], rv[16];
          tc_ld16_async(buf_row + kColA + 32u * h + 16u * half, av);
          tc_ld16_async(buf_row + kColR + 32u * h + 16u * half, rv);
          tc_wait_ld();
          if (half == 1) {
            tc_fence_before();
            mbar_arrive(&bar_buf_free[e & 1]);   // the values are in registers: the buffer may be reused
          }
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[i] = fmaf(r_scale, __uint_as_float(rv[ch * 8 + i]), __uint_as_float(av[ch * 8 + i]));
            }
            uint4 w;
            const int piece16 = 2 * half + ch;              // 16-byte piece of the 64-byte half row
            __nv_bfloat16* out_row = static_cast<__nv_bfloat16*>(p.hidden_out) +
                                     (b * p.T + static_cast<int64_t>(t0) + row) * p.H + x_v + 32 * h + piece16 * 8;
            if (accumulate_out && row_live) {
              // a later key/query block of a wide head: add to the sum of the blocks before it
              const uint4 prev = *reinterpret_cast<const uint4*>(out_row);
              const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&prev);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(pp[i]);
                o[2 * i] += f.x;
                o[2 * i + 1] += f.y;
              }
            }
            w.x = pack_bf16(o[0], o[1]);
            w.y = pack_bf16(o[2], o[3]);
            w.z = pack_bf16(o[4], o[5]);
            w.w = pack_bf16(o[6], o[7]);
            if (by_tma) {
              // 64-byte rows, 64-byte swizzle: piece j of row r sits at position j ^ ((r >> 1) & 3)
              *reinterpret_cast<uint4*>(s_out + row * 64 + ((piece16 ^ ((row >> 1) & 3)) * 16)) = w;
            } else if (row_live) {
              *reinterpret_cast<uint4*>(out_row) = w;
            }
          }
        }
        fence_proxy_async();
        mbar_arrive(&bar_out_ready[h]);
        if (row == 0) {
          GRMX_WAIT(&bar_out_ready[h], e)
          if (by_tma) {
            tma_store_3d(s_out, &map_o, x_v + 32 * h, t0, static_cast<int>(b));
            bulk_commit();
          }
        }
      }
      if (row == 0) bulk_wait_read();   // the last store still reads shared memory
    }
  }
#undef GRMX_WAIT

  // ---- teardown (all threads) ----
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *s_abort && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
  if (warp == kIssuerA) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

}  // namespace

bool scan_tcgen05_pipe_supported(const ScanParams& p) {
  return p.K % kD == 0 && p.H % kD == 0 && p.K >= kD && p.H >= kD && p.K <= 1024 && p.H <= 4096;
}

int launch_scan_tcgen05_pipe(const ScanParams& p, const SplitInfo& split, cudaStream_t stream) {
  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(linear_scan_tc_pipe_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemAlloc);
      if (attr_status == cudaSuccess) {
        attr_status = cudaFuncSetAttribute(linear_scan_tc_pipe_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kSmemAlloc);
      }
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cannot reserve %d bytes of shared memory: %s", kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_k, map_v, map_o;
  if (!make_token_map(&map_q, p.queries, p.B, p.T, p.K) || !make_token_map(&map_k, p.keys, p.B, p.T, p.K) ||
      !make_token_map(&map_v, p.values, p.B, p.T, p.H) || !make_token_half_map(&map_o, p.hidden_out, p.B, p.T, p.H)) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cuTensorMapEncodeTiled failed");
  }
  // one launch per 64-wide block of key/query features; the blocks of value features are in the grid
  const int64_t blocks = p.B * split.pieces * (p.H / kD);
  if (blocks > 0x7fffffffLL) return fail(GRMX_ERR_UNSUPPORTED, "tcgen05 scan: grid too large");
  for (int x_k = 0; x_k < static_cast<int>(p.K); x_k += kD) {
    // programmatic stream serialisation: the set-up of this grid (barriers, TMEM, decay tables) and its
    // launch latency overlap the tail of the kernel before it; GRMX_SCAN_PDL=off launches plainly
    static const bool pdl = [] {
      const char* e = getenv("GRMX_SCAN_PDL");
      return e == nullptr || strcmp(e, "off") != 0;
    }();
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(blocks));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemAlloc;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl ? 1 : 0;
    const cudaError_t launched =
        p.snapshots != nullptr
            ? cudaLaunchKernelEx(&config, linear_scan_tc_pipe_kernel<true>, map_q, map_k, map_v, map_o, p, split, x_k,
                                 x_k > 0 ? 1 : 0, device_error_word_ptr())
            : cudaLaunchKernelEx(&config, linear_scan_tc_pipe_kernel<false>, map_q, map_k, map_v, map_o, p, split, x_k,
                                 x_k > 0 ? 1 : 0, device_error_word_ptr());
    if (launched != cudaSuccess) {
      return fail(GRMX_ERR_LAUNCH, "linear_scan_tcgen05_pipe: launch failed: %s", cudaGetErrorString(launched));
    }
    const int rc = check_launch("linear_scan_tcgen05_pipe");
    if (rc != GRMX_OK) return rc;
  }
  return GRMX_OK;
}

}  // namespace grmx
