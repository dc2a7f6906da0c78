// Warp-specialised tcgen05 kernel of the linear-memory scan for heads of d_k = 128
// (bf16 operands, fp32 state in registers, chunks of 128 tokens, forward scans).
//
// One CTA owns one batch row and one 64-wide block of value features for the whole call; the two
// (or more) CTAs of a row are neighbours in the grid, run at the same time and share the row's q and
// k tiles through L2, so every tile comes from HBM once and every output tile is written once.
// Per chunk c, with Q, Kc the chunk's [128 x 128] tiles, Vc its [128 x 64] block of values and
// M^T [128 (d_k) x 64 (d_v)] the transposed block of the carried state:
//
//   S   = Q Kc^T                  128 x 128 x 128   K-major x K-major
//   R   = Q Mb^T                  128 x  64 x 128   K-major x MN-major, Mb^T = bf16(M^T_{c-1})
//   U^T = Kc^T Vw                 128 x  64 x 128   MN-major x MN-major, Vw_j = coeff * decay^(len-1-j) v_j
//   A   = P Vc                    128 x  64 x 128   TMEM x MN-major, P_ij = hs * coeff * decay^(i-j) S_ij (j <= i)
//   M^T = decay^len M^T + U^T     fp32 FMA in registers, one d_k row per thread
//   out_i = hs * decay^(i+1) R_i + A_i
//
// the closed form of the reference chunk (grm/core/cuda_ops.py:218-254) with the state carried across
// chunks as in grm/csrc/grm_cuda.cpp:67-83; the reference kernel covers d_k <= 128 in one pass too
// (grm/csrc/chunk_update.cu:17,508).  The state is kept transposed because a 128-row accumulator
// gives every thread of the state group one row: U^T has d_k = 128 rows where U would have 64.
//
// Roles (24 warps, registers re-divided between them at entry):
//   warp 20      issuer A: S_c; owns the TMEM allocation
//   warp 21      issuer B: U^T_c (needs nothing of the state: the recurrence is one FMA behind it)
//   warp 22      issuer C: R_c (needs the state before chunk c), then A_c
//   warp 23      loader: three TMA rings of two stages each -- q, k, v -- refilled independently as
//                soon as the last product that reads a tile has retired
//   warps 16-19  state group: Vw_c, the state update and its bf16 copy Mb^T
//   warps 0-7    P groups: S_c -> P_c (decay mask, bf16, written back into the TMEM columns of S_c)
//   warps 8-15   epilogue groups: R_c, A_c -> out -> shared memory -> TMA store
//
// Shared memory: q ring 2 x 32 KiB and k ring 2 x 32 KiB (a [128 x 128] tile is two [128 x 64]
// sub-tiles 16 KiB apart, each with the 128-byte swizzle), v ring 2 x 16 KiB, Mb^T 16 KiB, Vw 2 x 16 KiB,
// two output half tiles.  TMEM (512 columns): two buffers of 192 columns
// [S -> P (0-63) , A (64-127) | R (128-191)] used by alternate chunks, two U^T buffers of 64.
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
constexpr int kDV = 64;                // value features per CTA
constexpr int kThreads = 768;
constexpr int kStateWarp0 = 16;
constexpr int kStateThreads = 128;
constexpr int kIssuerA = 20;
constexpr int kIssuerB = 21;
constexpr int kIssuerC = 22;
constexpr int kLoader = 23;
constexpr int kRegsCompute = 72;
constexpr int kRegsState = 128;
constexpr int kRegsIssue = 40;
constexpr int kRegsLaunch = 80;        // 65536 / 768, rounded down to a multiple of 8
static_assert(512 * kRegsCompute + kStateThreads * kRegsState + 128 * kRegsIssue <= kThreads * kRegsLaunch,
              "the state group would wait for registers that nobody releases");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kBufCols = 192;     // buffer (c & 1) starts at column 192 * (c & 1)
constexpr uint32_t kColA = 64;
constexpr uint32_t kColR = 128;
constexpr uint32_t kColU = 384;        // + 64 * (c & 1)

constexpr int kSub = kChunk * 64 * 2;                  // 16 KiB: one [128 x 64] bf16 sub-tile
constexpr int kOffQ = 0;                               // 2 stages x 2 sub-tiles
constexpr int kOffK = 4 * kSub;
constexpr int kOffV = 8 * kSub;                        // 2 stages x 1 sub-tile
constexpr int kOffMb = 10 * kSub;                      // [128 (d_k) x 64 (d_v)] bf16
constexpr int kOffVw = 11 * kSub;                      // two buffers, used by alternate chunks
constexpr int kOutBytes = kChunk * 32 * 2;             // 8 KiB: [128 x 32] bf16, one per epilogue group
constexpr int kOffOut = 13 * kSub;
constexpr int kOffTables = kOffOut + 2 * kOutBytes;
// Decay weights of P, reversed: entry m holds weight(row - col = 127 - m).  A 32-column block that is not
// all zero starts at m0 = 127 - row + 32 * blk <= 127 and reads 32 entries, zero beyond m = 127.  Two
// copies, shifted by 0 and 1 entries, let any such run be read with aligned 8-byte loads.
constexpr int kWcopy = 164;
constexpr int kOffWtab = kOffTables;
constexpr int kOffPow = kOffWtab + 2 * kWcopy * 4;
constexpr int kOffBars = kOffPow + (kChunk + 4) * 4;
constexpr int kNumBars = 40;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemTotal = kOffMisc + 32;
// The plan needs a 1 KiB-aligned base (swizzle atoms).  The whole opt-in maximum is requested and the
// base is rounded up inside the kernel; what is left over is the room for that rounding (the dynamic
// shared memory of a kernel without static shared memory starts on a 1 KiB boundary in practice, so the
// rounding is zero), and the kernel checks that the rounded plan still fits before it touches anything.
constexpr int kSmemAlloc = 232448;
static_assert(kSmemTotal + 512 <= kSmemAlloc, "shared memory plan exceeds 227 KiB");
static_assert(kOffBars % 8 == 0, "barriers are 8-byte aligned");

// k-step kk (16 features) of a K-major [128 x 128] tile held as two sub-tiles
__device__ __forceinline__ uint32_t kmajor_step(int kk) { return static_cast<uint32_t>((kk >> 2) * kSub + (kk & 3) * 32); }

template <bool kSnapshots>
__global__ void __launch_bounds__(kThreads, 1)
linear_scan_tc_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                           ScanParams p, uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_wtab = reinterpret_cast<float*>(smem + kOffWtab);
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full_q = bars;            // [2] TMA bytes landed                                    (1 + tx)
  uint64_t* bar_full_k = bars + 2;        // [2]
  uint64_t* bar_full_v = bars + 4;        // [2]
  uint64_t* bar_q_free = bars + 6;        // [2] S_c and R_c complete                                (2 commits)
  uint64_t* bar_k_free = bars + 8;        // [2] S_c and U_c complete                                (2 commits)
  uint64_t* bar_v_free = bars + 10;       // [2] A_c complete and Vw_c copied                        (1 commit + 128)
  uint64_t* bar_s_done = bars + 12;       // [2] S_c complete                                        (commit)
  uint64_t* bar_r_done = bars + 14;       // [2] R_c complete                                        (commit)
  uint64_t* bar_a_done = bars + 16;       // [2] A_c complete                                        (commit)
  uint64_t* bar_u_done = bars + 18;       // [2] U_c complete                                        (commit)
  uint64_t* bar_p_ready = bars + 20;      // [2] P_c in TMEM                                         (256)
  uint64_t* bar_s_read = bars + 22;       // [2] P group 0 has S block 1 in registers                (128)
  uint64_t* bar_buf_free = bars + 24;     // [2] epilogue c has read R_c and A_c                     (256)
  uint64_t* bar_mb_ready = bars + 26;     // [2] bf16 copy of the state before chunk c               (128)
  uint64_t* bar_vw_ready = bars + 28;     // [2] Vw_c written                                        (128)
  uint64_t* bar_u_free = bars + 30;       // [2] U_c folded into the state                           (128)
  uint64_t* bar_out_ready = bars + 32;    // [2] epilogue group h has written its half tile          (128)
  uint64_t* bar_out_free = bars + 34;     // [2] the store of that half tile has read it             (1)
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
  const int vb = static_cast<int>(blockIdx.x % n_vb);     // fastest: the CTAs of a row run together
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
      mbar_init(&bar_full_v[i], 1);
      mbar_init(&bar_q_free[i], 2);
      mbar_init(&bar_k_free[i], 2);
      mbar_init(&bar_v_free[i], 1 + kStateThreads);
      mbar_init(&bar_s_done[i], 1);
      mbar_init(&bar_r_done[i], 1);
      mbar_init(&bar_a_done[i], 1);
      mbar_init(&bar_u_done[i], 1);
      mbar_init(&bar_p_ready[i], 256);
      mbar_init(&bar_s_read[i], 128);
      mbar_init(&bar_buf_free[i], 256);
      mbar_init(&bar_mb_ready[i], kStateThreads);
      mbar_init(&bar_vw_ready[i], kStateThreads);
      mbar_init(&bar_u_free[i], kStateThreads);
      mbar_init(&bar_out_ready[i], 128);
      mbar_init(&bar_out_free[i], 1);
    }
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

  auto q_stage = [&](int c) { return smem + kOffQ + (c & 1) * 2 * kSub; };
  auto k_stage = [&](int c) { return smem + kOffK + (c & 1) * 2 * kSub; };
  auto v_stage = [&](int c) { return smem + kOffV + (c & 1) * kSub; };
  auto mb_buf = [&](int) { return smem + kOffMb; };
  auto vw_buf = [&](int c) { return smem + kOffVw + (c & 1) * kSub; };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  // Protocol.  "X(c)" is the completion of barrier X that belongs to chunk c: phase c/2 of X[c&1].  A
  // waiter is never more than one completion behind, because the producer's next completion on the
  // same barrier needs something that comes after the waiter's wait:
  //   loader:   q(c) needs q_free(c-2) = S_{c-2} and R_{c-2} retired; k(c) needs k_free(c-2) = S_{c-2} and
  //             U_{c-2}; v(c) needs v_free(c-2) = A_{c-2} retired and Vw_{c-2} copied
  //   issuer A: S_c needs full_q(c), full_k(c), buf_free(c-2)
  //   issuer B: U_c needs full_k(c), vw_ready(c), u_free(c-2)
  //   issuer C: R_c needs full_q(c), mb_ready(c), buf_free(c-2); A_c needs p_ready(c) (which follows
  //             s_done(c)) and full_v(c)
  //   state:    M_c needs u_done(c); Mb of chunk c+1 overwrites the one R_c read: needs r_done(c);
  //             Vw_{c+1} overwrites the one U_{c-1} read (u_done(c-1), waited for one iteration earlier) and
  //             needs full_v(c+1)
  //   P pass c needs s_done(c); epilogue c needs a_done(c) and r_done(c)
  if (warp >= kIssuerA) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
  if (warp == kIssuerA) {
    // ===================================================================== issuer A: S = Q Kc^T
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc(kChunk, kChunk, 0, 0);
    for (int c = 0; c < n_chunks; ++c) {
      GRMX_WAIT(&bar_full_q[c & 1], c / 2)
      GRMX_WAIT(&bar_full_k[c & 1], c / 2)
      if (c >= 2) GRMX_WAIT(&bar_buf_free[c & 1], c / 2 - 1)
      tc_fence_after();
      const uint64_t dq = smem_desc(smem_u32(q_stage(c)), 16, 1024);
      const uint64_t dk = smem_desc(smem_u32(k_stage(c)), 16, 1024);
      const uint32_t d_tmem = tmem_base + kBufCols * (c & 1);
#pragma unroll
      for (int kk = 0; kk < kDK / 16; ++kk) {
        tc_mma_bf16_if(leader, d_tmem, desc_add(dq, kmajor_step(kk)), desc_add(dk, kmajor_step(kk)), idesc_s, kk > 0);
      }
      tc_commit_if(leader, &bar_s_done[c & 1]);
      tc_commit_if(leader, &bar_q_free[c & 1]);
      tc_commit_if(leader, &bar_k_free[c & 1]);
    }
  } else if (warp == kLoader) {
    // ===================================================================== loader: three TMA rings
    const uint32_t leader = elect_one();
    int done_q = 0, done_k = 0, done_v = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int t0 = c * kChunk;
      if (c >= 2) GRMX_WAIT(&bar_k_free[c & 1], c / 2 - 1)
      mbar_expect_tx_if(leader, &bar_full_k[c & 1], 2 * kSub);
      tma_load_3d_if(leader, k_stage(c), &map_k, &bar_full_k[c & 1], 0, t0, b);
      tma_load_3d_if(leader, k_stage(c) + kSub, &map_k, &bar_full_k[c & 1], 64, t0, b);
      done_k = c + 1;
      if (c >= 2) GRMX_WAIT(&bar_q_free[c & 1], c / 2 - 1)
      mbar_expect_tx_if(leader, &bar_full_q[c & 1], 2 * kSub);
      tma_load_3d_if(leader, q_stage(c), &map_q, &bar_full_q[c & 1], 0, t0, b);
      tma_load_3d_if(leader, q_stage(c) + kSub, &map_q, &bar_full_q[c & 1], 64, t0, b);
      done_q = c + 1;
      if (c >= 2) GRMX_WAIT(&bar_v_free[c & 1], c / 2 - 1)
      mbar_expect_tx_if(leader, &bar_full_v[c & 1], kSub);
      tma_load_3d_if(leader, v_stage(c), &map_v, &bar_full_v[c & 1], x_v, t0, b);
      done_v = c + 1;
    }
    if (*s_abort) {
      // let the copies still in flight land before the shared memory is released
      for (int c = max(done_q - 2, 0); c < done_q; ++c) mbar_wait_quiet(&bar_full_q[c & 1], (c / 2) & 1);
      for (int c = max(done_k - 2, 0); c < done_k; ++c) mbar_wait_quiet(&bar_full_k[c & 1], (c / 2) & 1);
      for (int c = max(done_v - 2, 0); c < done_v; ++c) mbar_wait_quiet(&bar_full_v[c & 1], (c / 2) & 1);
    }
  } else if (warp == kIssuerB) {
    // ===================================================================== issuer B: U^T = Kc^T Vw
    // Nothing here waits for the state: U_c needs the k tile, the scaled copy of v and a free
    // accumulator only, so the state recurrence is one register FMA per chunk behind this product.
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_u = make_idesc(kDK, kDV, 1, 1);
    for (int c = 0; c < n_chunks; ++c) {
      const uint64_t dvw = smem_desc(smem_u32(vw_buf(c)), kSub, 1024);
      GRMX_WAIT(&bar_vw_ready[c & 1], c / 2)
      GRMX_WAIT(&bar_full_k[c & 1], c / 2)
      if (c >= 2) GRMX_WAIT(&bar_u_free[c & 1], c / 2 - 1)
      tc_fence_after();
      // A = Kc^T: the k tile read MN-major, its two 64-feature sub-tiles 16 KiB apart (leading offset)
      const uint64_t dk_mn = smem_desc(smem_u32(k_stage(c)), kSub, 1024);
      const uint32_t u_tmem = tmem_base + kColU + 64u * (c & 1);
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        tc_mma_bf16_if(leader, u_tmem, desc_add(dk_mn, kk * 2048), desc_add(dvw, kk * 2048), idesc_u, kk > 0);
      }
      tc_commit_if(leader, &bar_u_done[c & 1]);
      tc_commit_if(leader, &bar_k_free[c & 1]);
    }
  } else if (warp == kIssuerC) {
    // ===================================================================== issuer C: R = Q Mb^T, A = P V
    // R_c is ready to go early in the chunk (it needs the state before the chunk), A_c late (it needs
    // P_c), and both feed the epilogue of the chunk: one warp issues them in that order.
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_r = make_idesc(kChunk, kDV, 0, 1);
    constexpr uint32_t idesc_a = make_idesc(kChunk, kDV, 0, 1);
    for (int c = 0; c < n_chunks; ++c) {
      const uint32_t buf = tmem_base + kBufCols * (c & 1);
      const uint64_t dmb = smem_desc(smem_u32(mb_buf(c)), kSub, 1024);
      GRMX_WAIT(&bar_mb_ready[c & 1], c / 2)
      GRMX_WAIT(&bar_full_q[c & 1], c / 2)
      if (c >= 2) GRMX_WAIT(&bar_buf_free[c & 1], c / 2 - 1)
      tc_fence_after();
      {
        const uint64_t dq = smem_desc(smem_u32(q_stage(c)), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < kDK / 16; ++kk) {
          tc_mma_bf16_if(leader, buf + kColR, desc_add(dq, kmajor_step(kk)), desc_add(dmb, kk * 2048), idesc_r, kk > 0);
        }
        tc_commit_if(leader, &bar_r_done[c & 1]);
        tc_commit_if(leader, &bar_q_free[c & 1]);
      }
      GRMX_WAIT(&bar_p_ready[c & 1], c / 2)
      GRMX_WAIT(&bar_full_v[c & 1], c / 2)
      tc_fence_after();
      {
        const uint64_t dv_mn = smem_desc(smem_u32(v_stage(c)), kSub, 1024);     // P: 16 tokens = 8 columns
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk) {
          tc_mma_bf16_ts_if(leader, buf + kColA, buf + 8u * kk, desc_add(dv_mn, kk * 2048), idesc_a, kk > 0);
        }
        tc_commit_if(leader, &bar_a_done[c & 1]);
        tc_commit_if(leader, &bar_v_free[c & 1]);
      }
    }
  }
  } else if (warp >= kStateWarp0) {
    // ===================================================================== state group (warps 16-19)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsState));
    const int row = tid - kStateWarp0 * 32;   // token row of the Vw copy == d_k row of the state == TMEM lane
    const int quarter = warp - kStateWarp0;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m[kDV];                             // row `row` of M^T: state[x_v + j][row], j = 0..63

    auto write_mb = [&](int c) {              // row `row` of Mb^T (the state before chunk c): one 128-byte swizzled line
      uint8_t* mrow = mb_buf(c) + row * 128;
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
    auto copy_chunk = [&](int c) {            // Vw_c, then the v tile of chunk c is released
      const int len = chunk_len(c);
      const float w_v = row < len ? p.update_coeff * s_pow[len - 1 - row] : 0.0f;
      scaled_row_copy<4>(v_stage(c), vw_buf(c), row, w_v);
      fence_proxy_async();
      mbar_arrive(&bar_vw_ready[c & 1]);
      mbar_arrive(&bar_v_free[c & 1]);
    };

    // state at the start: column `row` of this CTA's [64 x 128] block of memory_in (coalesced across the warp)
    {
      const float* src = static_cast<const float*>(p.memory_in) + static_cast<int64_t>(b) * p.H * p.K +
                         static_cast<int64_t>(x_v) * p.m_row_stride + static_cast<int64_t>(row) * p.m_col_stride;
#pragma unroll
      for (int j = 0; j < kDV; ++j) {
        float x;
        asm volatile("ld.global.f32 %0, [%1];" : "=f"(x) : "l"(src + j * p.m_row_stride) : "memory");
        m[j] = x;
      }
      write_mb(0);
      fence_proxy_async();
      mbar_arrive(&bar_mb_ready[0]);
    }

    do {
      GRMX_WAIT(&bar_full_v[0], 0)
      copy_chunk(0);
      for (int c = 0; c < n_chunks; ++c) {
        const bool last = c + 1 == n_chunks;
        // ---- Vw of chunk c+1 first: its v tile landed long ago and its buffer is the one U_{c-1} read
        //      (u_done(c-1) was waited for in the iteration before), so U_{c+1} can be issued as soon as
        //      its k tile is there and nothing of the state recurrence holds it back ----
        if (!last) {
          GRMX_WAIT(&bar_full_v[(c + 1) & 1], (c + 1) / 2)
          copy_chunk(c + 1);
        }
        // ---- M^T_c = decay^len M^T_{c-1} + U^T_c ----
        GRMX_WAIT(&bar_u_done[c & 1], c / 2)
        tc_fence_after();
        {
          const float carry = s_pow[chunk_len(c)];
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
        if (!last) {
          // ---- the state before chunk c+1 replaces the copy that R_c read ----
          GRMX_WAIT(&bar_r_done[c & 1], c / 2)
          write_mb(c + 1);
          fence_proxy_async();
          mbar_arrive(&bar_mb_ready[(c + 1) & 1]);
        }
        if constexpr (kSnapshots) {
          if ((c + 1) % p.snap_chunks == 0) {
            // a segment ends with this chunk: its state goes to the caller's archive, [H, K] row-major
            float* snap = p.snapshots + static_cast<int64_t>(b) * p.snap_batch_stride +
                          static_cast<int64_t>((c + 1) / p.snap_chunks - 1) * p.snap_stride +
                          static_cast<int64_t>(x_v) * p.K + row;
#pragma unroll
            for (int j = 0; j < kDV; ++j) snap[static_cast<int64_t>(j) * p.K] = m[j] * p.memory_out_scale;
          }
        }
        if (last && p.memory_out != nullptr) {
          float* m_out = static_cast<float*>(p.memory_out) + (static_cast<int64_t>(b) * p.H + x_v) * p.K + row;
#pragma unroll
          for (int j = 0; j < kDV; ++j) m_out[static_cast<int64_t>(j) * p.K] = m[j] * p.memory_out_scale;
        }
      }
    } while (false);
  } else {
    // ===================================================================== compute groups (warps 0-15)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsCompute));
    const int g = warp >> 2;
    const int quarter = warp & 3;
    const int row = tid & 127;                // token row within the chunk == TMEM lane
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    if (g < 2) {
      // ---- P groups: group g turns the 32-column blocks 2g and 2g+1 of S into P ----
      // Blocks above block `quarter` are all zero.  P block blk (16 packed columns) lands on S columns
      // 16*blk .. 16*blk+15: group 0 overwrites S block 0 after reading it; group 1 overwrites S block 1,
      // which group 0 reads second, and waits for s_read(c) before it stores.
      for (int c = 0; c < n_chunks; ++c) {
        const uint32_t buf_row = lane_base + kBufCols * (c & 1);
        GRMX_WAIT(&bar_s_done[c & 1], c / 2)
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int blk = 2 * g + k;
          const bool nz = blk <= quarter;
          uint32_t sv[32], pk[16];
          if (nz) {
            tc_ld32_async(buf_row + 32u * blk, sv);
            tc_wait_ld();
          }
          if (g == 0 && k == 1) {
            tc_fence_before();
            mbar_arrive(&bar_s_read[c & 1]);
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
            GRMX_WAIT(&bar_s_read[c & 1], c / 2)
          }
          tc_st16_async(buf_row + 16u * blk, pk);
        }
        if (*s_abort) break;
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bar_p_ready[c & 1]);
      }
    } else {
      // ---- epilogue groups: group 2+h writes the output columns 32h .. 32h+31 of this CTA's value block ----
      // out_i = hs * decay^(i+1) R_i + A_i -> bf16 -> shared memory -> one TMA store per half tile (rows
      // beyond T are clipped by the store)
      const int h = g - 2;
      uint8_t* s_out = smem + kOffOut + h * kOutBytes;
      for (int e = 0; e < n_chunks; ++e) {
        const uint32_t buf_row = lane_base + kBufCols * (e & 1);
        GRMX_WAIT(&bar_r_done[e & 1], e / 2)
        GRMX_WAIT(&bar_a_done[e & 1], e / 2)
        tc_fence_after();
        const float r_scale = row < chunk_len(e) ? p.hidden_scale * s_pow[row + 1] : 0.0f;
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
            w.x = pack_bf16(o[0], o[1]);
            w.y = pack_bf16(o[2], o[3]);
            w.z = pack_bf16(o[4], o[5]);
            w.w = pack_bf16(o[6], o[7]);
            const int piece16 = 2 * half + ch;              // 16-byte piece of the 64-byte half row
            // 64-byte rows, 64-byte swizzle: piece j of row r sits at position j ^ ((r >> 1) & 3)
            *reinterpret_cast<uint4*>(s_out + row * 64 + ((piece16 ^ ((row >> 1) & 3)) * 16)) = w;
          }
        }
        fence_proxy_async();
        mbar_arrive(&bar_out_ready[h]);
        if (row == 0) {
          GRMX_WAIT(&bar_out_ready[h], e)
          tma_store_3d(s_out, &map_o, x_v + 32 * h, e * kChunk, b);
          bulk_commit();
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

bool scan_tcgen05_wide_supported(const ScanParams& p) {
  static const bool disabled = [] {
    const char* env = getenv("GRMX_SCAN_WIDE");
    return env != nullptr && strcmp(env, "off") == 0;
  }();
  return !disabled && p.K == kDK && p.H >= kDV && p.H % kDV == 0 && p.H <= 4096 && !p.reverse && !p.first_step_no_decay &&
         p.T >= 1 && p.B * (p.H / kDV) <= 0x7fffffffLL && p.B <= 0x7fffffffLL;
}

int launch_scan_tcgen05_wide(const ScanParams& p, cudaStream_t stream) {
  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(linear_scan_tc_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemAlloc);
      if (attr_status == cudaSuccess) {
        attr_status = cudaFuncSetAttribute(linear_scan_tc_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kSmemAlloc);
      }
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "wide tcgen05 scan: cannot reserve %d bytes of shared memory: %s", kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_k, map_v, map_o;
  if (!make_token_map(&map_q, p.queries, p.B, p.T, p.K) || !make_token_map(&map_k, p.keys, p.B, p.T, p.K) ||
      !make_token_map(&map_v, p.values, p.B, p.T, p.H) || !make_token_half_map(&map_o, p.hidden_out, p.B, p.T, p.H)) {
    return fail(GRMX_ERR_LAUNCH, "wide tcgen05 scan: cuTensorMapEncodeTiled failed");
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
          ? cudaLaunchKernelEx(&config, linear_scan_tc_wide_kernel<true>, map_q, map_k, map_v, map_o, p, device_error_word_ptr())
          : cudaLaunchKernelEx(&config, linear_scan_tc_wide_kernel<false>, map_q, map_k, map_v, map_o, p, device_error_word_ptr());
  if (launched != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "linear_scan_tcgen05_wide: launch failed: %s", cudaGetErrorString(launched));
  }
  return check_launch("linear_scan_tcgen05_wide");
}

}  // namespace grmx
