// Warp-specialised tcgen05 kernel of the linear-memory scan for heads of d_k = 128 whose value
// width is a multiple of 128 (bf16 operands, fp32 state in registers, chunks of 128 tokens, forward
// scans).
//
// One CTA owns one batch row and one 128-wide block of value features for the whole call, so with
// d_v = 128 every q, k and v tile goes from L2 to exactly one SM and every output tile leaves one SM:
// the scan is bound by the rate at which the SMs can pull bytes out of L2, and a row shared between
// two CTAs pays for q and k twice there even though DRAM sees them once.  The price is that nothing
// but the q and k rings is double-buffered -- shared memory (227 KiB) and TMEM (512 columns) are both
// used to the last unit -- which the arithmetic can afford: a chunk's dependent chain is about half
// the time its 128 KiB take to arrive.
//
// Per chunk c, with Q, Kc, Vc the chunk's [128 x 128] tiles and M^T [128 (d_k) x 128 (d_v)] the
// transposed block of the carried state:
//
//   S   = Q Kc^T                  128 x 128 x 128   K-major x K-major
//   R   = Q Mb^T                  128 x 128 x 128   K-major x MN-major, Mb^T = bf16(M^T_{c-1})
//   U^T = Kc^T Vw                 128 x 128 x 128   MN-major x MN-major, Vw_j = coeff * decay^(len-1-j) v_j
//   A   = P Vc                    128 x 128 x 128   TMEM x MN-major, P_ij = hs * coeff * decay^(i-j) S_ij (j <= i)
//   M^T = decay^len M^T + U^T     fp32 FMA in registers, one d_k row and 64 value features per thread
//   out_i = hs * decay^(i+1) R_i + A_i
//
// the closed form of the reference chunk (grm/core/cuda_ops.py:218-254) with the state carried across
// chunks as in grm/csrc/grm_cuda.cpp:67-83; the reference kernel covers d_k <= 128 in one pass too
// (grm/csrc/chunk_update.cu:17,508).
//
// Roles (20 warps, registers re-divided between them at entry):
//   warp 16      issuer A: S_c, then the store of out_{c-1}; owns the TMEM allocation
//   warp 17      issuer B: U^T_c
//   warp 18      issuer C: R_c, then A_c
//   warp 19      loader: q and k rings of two stages, one v stage
//   warps 8-15   state groups (value features 0-63 and 64-127): Vw_c, the state update, its bf16 copy
//   warps 0-7    compute groups (columns 0-63 and 64-127): S_c -> P_c, then R_c, A_c -> out_c
//
// Shared memory: q ring 2 x 32 KiB, k ring 2 x 32 KiB, v 32 KiB, Vw 32 KiB, Mb^T 32 KiB (a
// [128 x 128] tile is two [128 x 64] sub-tiles 16 KiB apart, each with the 128-byte swizzle).  The
// output tile of chunk c is staged in the q stage of chunk c, which S_c and R_c have finished with by
// then, and the stage is handed back to the loader when the store has read it.  TMEM: S -> P columns
// 0-127, A 128-255, R 256-383, U^T 384-511.
// Every hand-off is an mbarrier and every wait is bounded: on expiry the CTA-wide abort flag is
// raised, all roles drain, the error word gets bit 1, TMEM is freed and the kernel returns.
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
constexpr int kDK = 128;               // d_k
constexpr int kDV = 128;               // value features per CTA
constexpr int kThreads = 640;
constexpr int kComputeThreads = 256;   // warps 0-7
constexpr int kStateWarp0 = 8;
constexpr int kStateThreads = 256;     // warps 8-15
constexpr int kIssuerA = 16;
constexpr int kIssuerB = 17;
constexpr int kIssuerC = 18;
constexpr int kLoader = 19;
constexpr int kRegsCompute = 88;
constexpr int kRegsState = 128;
constexpr int kRegsIssue = 48;
constexpr int kRegsLaunch = 96;        // 65536 / 640, rounded down to a multiple of 8
static_assert(kComputeThreads * kRegsCompute + kStateThreads * kRegsState + 128 * kRegsIssue <= kThreads * kRegsLaunch,
              "the state groups would wait for registers that nobody releases");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColA = 128;
constexpr uint32_t kColR = 256;
constexpr uint32_t kColU = 384;

constexpr int kSub = kChunk * 64 * 2;                  // 16 KiB: one [128 x 64] bf16 sub-tile
constexpr int kTile = 2 * kSub;                        // 32 KiB: a [128 x 128] tile
constexpr int kOffQ = 0;                               // 2 stages
constexpr int kOffK = 2 * kTile;                       // 2 stages
constexpr int kOffV = 4 * kTile;
constexpr int kOffVw = 5 * kTile;
constexpr int kOffMb = 6 * kTile;                      // [128 (d_k) x 128 (d_v)] bf16
constexpr int kOffTables = 7 * kTile;
// Decay weights of P, reversed: entry m holds weight(row - col = 127 - m).  A 32-column block that is not
// all zero starts at m0 = 127 - row + 32 * blk <= 127 and reads 32 entries, zero beyond m = 127.  Two
// copies, shifted by 0 and 1 entries, let any such run be read with aligned 8-byte loads.
constexpr int kWcopy = 164;
constexpr int kOffWtab = kOffTables;
constexpr int kOffPow = kOffWtab + 2 * kWcopy * 4;
constexpr int kOffBars = kOffPow + (kChunk + 4) * 4;
constexpr int kNumBars = 24;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemTotal = kOffMisc + 32;
// The plan needs a 1 KiB-aligned base (swizzle atoms).  The whole opt-in maximum is requested and the
// base is rounded up inside the kernel; the dynamic shared memory of a kernel without static shared
// memory starts on a 1 KiB boundary in practice, so the rounding is zero, and the kernel checks that
// the rounded plan still fits before it touches anything.
constexpr int kSmemAlloc = 232448;
static_assert(kSmemTotal <= kSmemAlloc, "shared memory plan exceeds 227 KiB");
static_assert(kOffBars % 8 == 0, "barriers are 8-byte aligned");

// k-step kk (16 features) of a K-major [128 x 128] tile held as two sub-tiles
__device__ __forceinline__ uint32_t kmajor_step(int kk) { return static_cast<uint32_t>((kk >> 2) * kSub + (kk & 3) * 32); }

template <bool kSnapshots>
__global__ void __launch_bounds__(kThreads, 1)
linear_scan_tc_square_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                             ScanParams p, uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_wtab = reinterpret_cast<float*>(smem + kOffWtab);
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full_q = bars;            // [2] TMA bytes landed                                         (1 + tx)
  uint64_t* bar_full_k = bars + 2;        // [2]
  uint64_t* bar_q_free = bars + 4;        // [2] S_c, R_c complete and out_c read by its store            (2 commits + 1)
  uint64_t* bar_k_free = bars + 6;        // [2] S_c and U_c complete                                     (2 commits)
  uint64_t* bar_out_ready = bars + 8;     //     the compute groups have written out_c                    (256)
  uint64_t* bar_full_v = bars + 10;       //     v_c landed                                               (1 + tx)
  uint64_t* bar_v_free = bars + 11;       //     A_c complete and Vw_c copied                             (1 commit + 256)
  uint64_t* bar_s_done = bars + 12;       //     S_c complete                                             (commit)
  uint64_t* bar_r_done = bars + 13;       //     R_c complete                                             (commit)
  uint64_t* bar_a_done = bars + 14;       //     A_c complete: P_c consumed, the S columns are free       (commit)
  uint64_t* bar_u_done = bars + 15;       //     U_c complete: Vw_c consumed                              (commit)
  uint64_t* bar_p_ready = bars + 16;      //     P_c in TMEM                                              (256)
  uint64_t* bar_s_read = bars + 17;       //     compute group 0 has S block 1 in registers               (128)
  uint64_t* bar_ra_free = bars + 18;      //     the compute groups have read R_c and A_c                 (256)
  uint64_t* bar_mb_ready = bars + 19;     //     bf16 copy of the state before chunk c                    (256)
  uint64_t* bar_vw_ready = bars + 20;     //     Vw_c written                                             (256)
  uint64_t* bar_u_free = bars + 21;       //     U_c folded into the state                                (256)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (static_cast<int>(smem - smem_raw) + kSmemTotal > kSmemAlloc) {
    // the base of the dynamic shared memory is further from a 1 KiB boundary than the plan leaves room for
    if (tid == 0 && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
    return;
  }
  const int n_vb = static_cast<int>(p.H / kDV);
  const int vb = static_cast<int>(blockIdx.x % n_vb);
  const int b = static_cast<int>(blockIdx.x / n_vb);
  const int x_v = vb * kDV;
  const int T = static_cast<int>(p.T);
  const int n_chunks = (T + kChunk - 1) / kChunk;
  auto chunk_len = [&](int c) { return min(kChunk, T - c * kChunk); };

  // ---- set-up (all threads): touches no global memory, so it may overlap the kernel before this one ----
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_full_q[i], 1);
      mbar_init(&bar_full_k[i], 1);
      mbar_init(&bar_q_free[i], 3);
      mbar_init(&bar_k_free[i], 2);
    }
    mbar_init(bar_out_ready, kComputeThreads);
    mbar_init(bar_full_v, 1);
    mbar_init(bar_v_free, 1 + kStateThreads);
    mbar_init(bar_s_done, 1);
    mbar_init(bar_r_done, 1);
    mbar_init(bar_a_done, 1);
    mbar_init(bar_u_done, 1);
    mbar_init(bar_p_ready, kComputeThreads);
    mbar_init(bar_s_read, 128);
    mbar_init(bar_ra_free, kComputeThreads);
    mbar_init(bar_mb_ready, kStateThreads);
    mbar_init(bar_vw_ready, kStateThreads);
    mbar_init(bar_u_free, kStateThreads);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int j = tid; j <= kChunk; j += kThreads) s_pow[j] = powf(p.decay, static_cast<float>(j));
  for (int j = tid; j < 2 * kWcopy; j += kThreads) {
    const int copy = j / kWcopy;
    const int d = 127 - (j % kWcopy + copy);
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
  asm volatile("griddepcontrol.wait;" ::: "memory");

  auto q_stage = [&](int c) { return smem + kOffQ + (c & 1) * kTile; };
  auto k_stage = [&](int c) { return smem + kOffK + (c & 1) * kTile; };
  uint8_t* const v_tile = smem + kOffV;
  uint8_t* const vw_tile = smem + kOffVw;
  uint8_t* const mb_tile = smem + kOffMb;

  // out_c leaves from the q stage it was staged in (rows beyond T are clipped by the store); the stage
  // goes back to the loader when the store has read it
  auto store_out = [&](int c, uint32_t leader) {
    if (leader) {
      tma_store_3d(q_stage(c), &map_o, x_v, c * kChunk, b);
      tma_store_3d(q_stage(c) + kSub, &map_o, x_v + 64, c * kChunk, b);
      bulk_commit();
      bulk_wait_read();
      mbar_arrive(&bar_q_free[c & 1]);
    }
    __syncwarp();
  };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  // Protocol.  "X(c)" is the completion of barrier X that belongs to chunk c: phase c/2 of X[c&1] for
  // the two-stage rings, phase c of X for everything else.  A waiter is never more than one completion
  // behind, because the producer's next completion on the same barrier needs something that comes after
  // the waiter's wait:
  //   loader:   k(c) needs k_free(c-2) = S_{c-2} and U_{c-2} retired; q(c) needs q_free(c-2) = S_{c-2}, R_{c-2}
  //             retired and out_{c-2} read by its stores; v(c) needs v_free(c-1) = A_{c-1} retired and
  //             Vw_{c-1} copied
  //   issuer A: S_c needs full_q(c), full_k(c), a_done(c-1); the store of out_{c-1} needs out_ready(c-1)
  //   issuer B: U_c needs vw_ready(c), full_k(c), u_free(c-1)
  //   issuer C: R_c needs mb_ready(c), full_q(c), ra_free(c-1); A_c needs p_ready(c) and full_v(c)
  //   state:    Vw_c needs full_v(c) and u_done(c-1) (waited for in the iteration before); M_c needs
  //             u_done(c); Mb of chunk c+1 overwrites the one R_c read: r_done(c)
  //   compute:  P pass c needs s_done(c); out_c needs r_done(c) and a_done(c)
  if (warp >= kIssuerA) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
  if (warp == kIssuerA) {
    // ===================================================================== issuer A: S = Q Kc^T
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc(kChunk, kChunk, 0, 0);
    for (int c = 0; c < n_chunks; ++c) {
      GRMX_WAIT(&bar_full_q[c & 1], c / 2)
      GRMX_WAIT(&bar_full_k[c & 1], c / 2)
      if (c >= 1) GRMX_WAIT(bar_a_done, c - 1)
      tc_fence_after();
      const uint64_t dq = smem_desc(smem_u32(q_stage(c)), 16, 1024);
      const uint64_t dk = smem_desc(smem_u32(k_stage(c)), 16, 1024);
#pragma unroll
      for (int kk = 0; kk < kDK / 16; ++kk) {
        tc_mma_bf16_if(leader, tmem_base, desc_add(dq, kmajor_step(kk)), desc_add(dk, kmajor_step(kk)), idesc_s, kk > 0);
      }
      tc_commit_if(leader, bar_s_done);
      tc_commit_if(leader, &bar_q_free[c & 1]);
      tc_commit_if(leader, &bar_k_free[c & 1]);
      // out_{c-1} is being written while S_c runs: store it from here, where waiting until the store has
      // read its source delays nothing (a compute warp that waited would be late for the next P pass)
      if (c >= 1) {
        GRMX_WAIT(bar_out_ready, c - 1)
        store_out(c - 1, leader);
      }
    }
    if (!*s_abort && mbar_wait(bar_out_ready, static_cast<uint32_t>(n_chunks - 1) & 1u, s_abort)) {
      store_out(n_chunks - 1, leader);
    }
  } else if (warp == kLoader) {
    // ===================================================================== loader
    const uint32_t leader = elect_one();
    int issued = 0;                           // copies issued so far, in the order k, q, v of every chunk
    for (int c = 0; c < n_chunks; ++c) {
      const int t0 = c * kChunk;
      if (c >= 2) GRMX_WAIT(&bar_k_free[c & 1], c / 2 - 1)
      mbar_expect_tx_if(leader, &bar_full_k[c & 1], kTile);
      tma_load_3d_if(leader, k_stage(c), &map_k, &bar_full_k[c & 1], 0, t0, b);
      tma_load_3d_if(leader, k_stage(c) + kSub, &map_k, &bar_full_k[c & 1], 64, t0, b);
      ++issued;
      if (c >= 2) GRMX_WAIT(&bar_q_free[c & 1], c / 2 - 1)
      mbar_expect_tx_if(leader, &bar_full_q[c & 1], kTile);
      tma_load_3d_if(leader, q_stage(c), &map_q, &bar_full_q[c & 1], 0, t0, b);
      tma_load_3d_if(leader, q_stage(c) + kSub, &map_q, &bar_full_q[c & 1], 64, t0, b);
      ++issued;
      if (c >= 1) GRMX_WAIT(bar_v_free, c - 1)
      mbar_expect_tx_if(leader, bar_full_v, kTile);
      tma_load_3d_if(leader, v_tile, &map_v, bar_full_v, x_v, t0, b);
      tma_load_3d_if(leader, v_tile + kSub, &map_v, bar_full_v, x_v + 64, t0, b);
      ++issued;
    }
    if (*s_abort) {
      // let the copies still in flight land before the shared memory is released
      const int done_k = (issued + 2) / 3, done_q = (issued + 1) / 3, done_v = issued / 3;
      for (int c = max(done_q - 2, 0); c < done_q; ++c) mbar_wait_quiet(&bar_full_q[c & 1], (c / 2) & 1);
      for (int c = max(done_k - 2, 0); c < done_k; ++c) mbar_wait_quiet(&bar_full_k[c & 1], (c / 2) & 1);
      if (done_v > 0) mbar_wait_quiet(bar_full_v, (done_v - 1) & 1);
    }
  } else if (warp == kIssuerB) {
    // ===================================================================== issuer B: U^T = Kc^T Vw
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_u = make_idesc(kDK, kDV, 1, 1);
    const uint64_t dvw = smem_desc(smem_u32(vw_tile), kSub, 1024);
    for (int c = 0; c < n_chunks; ++c) {
      GRMX_WAIT(bar_vw_ready, c)
      GRMX_WAIT(&bar_full_k[c & 1], c / 2)
      if (c >= 1) GRMX_WAIT(bar_u_free, c - 1)
      tc_fence_after();
      // both operands MN-major: 16 tokens per instruction = 2048 bytes, the two 64-feature sub-tiles
      // of a tile 16 KiB apart (leading offset)
      const uint64_t dk_mn = smem_desc(smem_u32(k_stage(c)), kSub, 1024);
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        tc_mma_bf16_if(leader, tmem_base + kColU, desc_add(dk_mn, kk * 2048), desc_add(dvw, kk * 2048), idesc_u, kk > 0);
      }
      tc_commit_if(leader, bar_u_done);
      tc_commit_if(leader, &bar_k_free[c & 1]);
    }
  } else if (warp == kIssuerC) {
    // ===================================================================== issuer C: R = Q Mb^T, A = P V
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_r = make_idesc(kChunk, kDV, 0, 1);
    constexpr uint32_t idesc_a = make_idesc(kChunk, kDV, 0, 1);
    const uint64_t dmb = smem_desc(smem_u32(mb_tile), kSub, 1024);
    const uint64_t dv_mn = smem_desc(smem_u32(v_tile), kSub, 1024);
    for (int c = 0; c < n_chunks; ++c) {
      GRMX_WAIT(bar_mb_ready, c)
      GRMX_WAIT(&bar_full_q[c & 1], c / 2)
      if (c >= 1) GRMX_WAIT(bar_ra_free, c - 1)
      tc_fence_after();
      {
        const uint64_t dq = smem_desc(smem_u32(q_stage(c)), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < kDK / 16; ++kk) {
          tc_mma_bf16_if(leader, tmem_base + kColR, desc_add(dq, kmajor_step(kk)), desc_add(dmb, kk * 2048), idesc_r, kk > 0);
        }
        tc_commit_if(leader, bar_r_done);
        tc_commit_if(leader, &bar_q_free[c & 1]);
      }
      GRMX_WAIT(bar_p_ready, c)
      GRMX_WAIT(bar_full_v, c)
      tc_fence_after();
      {
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk) {   // P: 16 tokens = 8 columns
          tc_mma_bf16_ts_if(leader, tmem_base + kColA, tmem_base + 8u * kk, desc_add(dv_mn, kk * 2048), idesc_a, kk > 0);
        }
        tc_commit_if(leader, bar_a_done);
        tc_commit_if(leader, bar_v_free);
      }
    }
  }
  } else if (warp >= kStateWarp0) {
    // ===================================================================== state groups (warps 8-15)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsState));
    const int st = tid - kStateWarp0 * 32;
    const int half = st >> 7;                 // value features 64*half .. 64*half+63: sub-tile `half` of v, Vw, Mb^T
    const int row = st & 127;                 // token row of the Vw copy == d_k row of the state == TMEM lane
    const int quarter = (warp - kStateWarp0) & 3;
    const uint32_t tmem_u = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kColU + 64u * half;
    float m[64];                              // state[x_v + 64*half + j][row], j = 0..63

    auto write_mb = [&]() {                   // one 128-byte swizzled line of Mb^T
      uint8_t* mrow = mb_tile + half * kSub + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint4 w;
        w.x = pack_bf16(m[ch * 8 + 0], m[ch * 8 + 1]);
        w.y = pack_bf16(m[ch * 8 + 2], m[ch * 8 + 3]);
        w.z = pack_bf16(m[ch * 8 + 4], m[ch * 8 + 5]);
        w.w = pack_bf16(m[ch * 8 + 6], m[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(mrow + ((ch ^ (row & 7)) * 16)) = w;
      }
    };

    // state at the start (coalesced across the warp: `row` is the fastest index of memory_in)
    {
      const float* src = static_cast<const float*>(p.memory_in) + static_cast<int64_t>(b) * p.H * p.K +
                         static_cast<int64_t>(x_v + 64 * half) * p.m_row_stride + static_cast<int64_t>(row) * p.m_col_stride;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        float x;
        asm volatile("ld.global.f32 %0, [%1];" : "=f"(x) : "l"(src + j * p.m_row_stride) : "memory");
        m[j] = x;
      }
      write_mb();
      fence_proxy_async();
      mbar_arrive(bar_mb_ready);
    }

    for (int c = 0; c < n_chunks; ++c) {
      const bool last = c + 1 == n_chunks;
      const int len = chunk_len(c);
      // ---- Vw_c: the buffer is the one U_{c-1} read, and u_done(c-1) was waited for below ----
      GRMX_WAIT(bar_full_v, c)
      {
        const float w_v = row < len ? p.update_coeff * s_pow[len - 1 - row] : 0.0f;
        scaled_row_copy<4>(v_tile + half * kSub, vw_tile + half * kSub, row, w_v);
        fence_proxy_async();
        mbar_arrive(bar_vw_ready);
        mbar_arrive(bar_v_free);
      }
      // ---- M^T_c = decay^len M^T_{c-1} + U^T_c ----
      GRMX_WAIT(bar_u_done, c)
      tc_fence_after();
      {
        const float carry = s_pow[len];
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t u[32];
          tc_ld32_async(tmem_u + 32u * part, u);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) m[32 * part + j] = fmaf(carry, m[32 * part + j], __uint_as_float(u[j]));
        }
      }
      tc_fence_before();
      mbar_arrive(bar_u_free);
      if (!last) {
        // ---- the state before chunk c+1 replaces the copy that R_c read ----
        GRMX_WAIT(bar_r_done, c)
        write_mb();
        fence_proxy_async();
        mbar_arrive(bar_mb_ready);
      }
      if constexpr (kSnapshots) {
        if ((c + 1) % p.snap_chunks == 0) {
          // a segment ends with this chunk: its state goes to the caller's archive, [H, K] row-major
          float* snap = p.snapshots + static_cast<int64_t>(b) * p.snap_batch_stride +
                        static_cast<int64_t>((c + 1) / p.snap_chunks - 1) * p.snap_stride +
                        static_cast<int64_t>(x_v + 64 * half) * p.K + row;
#pragma unroll
          for (int j = 0; j < 64; ++j) snap[static_cast<int64_t>(j) * p.K] = m[j] * p.memory_out_scale;
        }
      }
      if (last && p.memory_out != nullptr) {
        float* m_out = static_cast<float*>(p.memory_out) + (static_cast<int64_t>(b) * p.H + x_v + 64 * half) * p.K + row;
#pragma unroll
        for (int j = 0; j < 64; ++j) m_out[static_cast<int64_t>(j) * p.K] = m[j] * p.memory_out_scale;
      }
    }
  } else {
    // ===================================================================== compute groups (warps 0-7)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsCompute));
    const int g = warp >> 2;                  // columns 64g .. 64g+63 of S, and of the output
    const int quarter = warp & 3;
    const int row = tid & 127;                // token row within the chunk == TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    for (int c = 0; c < n_chunks; ++c) {
      // ---- S_c -> P_c: group g turns the 32-column blocks 2g and 2g+1 of S into P ----
      // Blocks above block `quarter` are all zero.  P block blk (16 packed columns) lands on S columns
      // 16*blk .. 16*blk+15: group 0 overwrites S block 0 after reading it; group 1 overwrites S block 1,
      // which group 0 reads second, and waits for s_read(c) before it stores.
      GRMX_WAIT(bar_s_done, c)
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int blk = 2 * g + k;
        const bool nz = blk <= quarter;
        uint32_t sv[32], pk[16];
        if (nz) {
          tc_ld32_async(lane_base + 32u * blk, sv);
          tc_wait_ld();
        }
        if (g == 0 && k == 1) {
          tc_fence_before();
          mbar_arrive(bar_s_read);
        }
        if (nz) {
          const int m0 = 127 - row + 32 * blk;            // reversed-table index of column 32*blk
          const float2* wv = reinterpret_cast<const float2*>(s_wtab + (m0 & 1) * kWcopy + (m0 & ~1));
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const float2 w2 = wv[t];
            pk[t] = pack_bf16(__uint_as_float(sv[2 * t]) * w2.x, __uint_as_float(sv[2 * t + 1]) * w2.y);
          }
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) pk[t] = 0u;
        }
        if (g == 1 && k == 0) {
          GRMX_WAIT(bar_s_read, c)
        }
        tc_st16_async(lane_base + 16u * blk, pk);
      }
      if (*s_abort) break;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_ready);

      // ---- out_c: group g writes columns 64g .. 64g+63, i.e. sub-tile g of the q stage of this chunk,
      //      which S_c and R_c have finished with; out_i = hs * decay^(i+1) R_i + A_i -> bf16; issuer A
      //      stores the tile ----
      GRMX_WAIT(bar_r_done, c)
      GRMX_WAIT(bar_a_done, c)
      tc_fence_after();
      const float r_scale = row < chunk_len(c) ? p.hidden_scale * s_pow[row + 1] : 0.0f;
      uint8_t* s_out = q_stage(c) + g * kSub + row * 128;
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t av[16], rv[16];
        tc_ld16_async(lane_base + kColA + 64u * g + 16u * piece, av);
        tc_ld16_async(lane_base + kColR + 64u * g + 16u * piece, rv);
        tc_wait_ld();
        if (piece == 3) {
          tc_fence_before();
          mbar_arrive(bar_ra_free);            // the values are in registers: R and A may be overwritten
        }
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            o[i] = fmaf(r_scale, __uint_as_float(rv[ch * 8 + i]), __uint_as_float(av[ch * 8 + i]));
          }
          uint4 w;
          w.x = pack_bf16(o[0], o[1]);
          w.y = pack_bf16(o[2], o[3]);
          w.z = pack_bf16(o[4], o[5]);
          w.w = pack_bf16(o[6], o[7]);
          const int piece16 = 2 * piece + ch;             // 16-byte piece of the 128-byte row
          *reinterpret_cast<uint4*>(s_out + ((piece16 ^ (row & 7)) * 16)) = w;
        }
      }
      fence_proxy_async();
      mbar_arrive(bar_out_ready);
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

bool scan_tcgen05_square_supported(const ScanParams& p) {
  static const bool disabled = [] {
    const char* env = getenv("GRMX_SCAN_SQUARE");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  return !disabled && p.K == kDK && p.H >= kDV && p.H % kDV == 0 && p.H <= 4096 && !p.reverse && !p.first_step_no_decay &&
         p.T >= 1 && p.B * (p.H / kDV) <= 0x7fffffffLL && p.B <= 0x7fffffffLL;
}

int launch_scan_tcgen05_square(const ScanParams& p, cudaStream_t stream) {
  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(linear_scan_tc_square_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemAlloc);
      if (attr_status == cudaSuccess) {
        attr_status = cudaFuncSetAttribute(linear_scan_tc_square_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kSmemAlloc);
      }
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "square tcgen05 scan: cannot reserve %d bytes of shared memory: %s", kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_k, map_v, map_o;
  if (!make_token_map(&map_q, p.queries, p.B, p.T, p.K) || !make_token_map(&map_k, p.keys, p.B, p.T, p.K) ||
      !make_token_map(&map_v, p.values, p.B, p.T, p.H) || !make_token_map(&map_o, p.hidden_out, p.B, p.T, p.H)) {
    return fail(GRMX_ERR_LAUNCH, "square tcgen05 scan: cuTensorMapEncodeTiled failed");
  }
  static const bool pdl = [] {
    const char* e = getenv("GRMX_SCAN_PDL");
    return e == nullptr || strcmp(e, "off") != 0;
  }();
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.B * (p.H / kDV)));
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
          ? cudaLaunchKernelEx(&config, linear_scan_tc_square_kernel<true>, map_q, map_k, map_v, map_o, p, device_error_word_ptr())
          : cudaLaunchKernelEx(&config, linear_scan_tc_square_kernel<false>, map_q, map_k, map_v, map_o, p, device_error_word_ptr());
  if (launched != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "linear_scan_tcgen05_square: launch failed: %s", cudaGetErrorString(launched));
  }
  return check_launch("linear_scan_tcgen05_square");
}

}  // namespace grmx
