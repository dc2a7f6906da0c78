// Warp-specialised, pipelined tcgen05 kernel of the linear-memory scan
// (d_k = d_v = 64, bf16 operands, fp32 state in TMEM, chunks of 128 tokens).
//
// Per chunk c, with Q, Kc, Vc the chunk's [128 x 64] tiles and M the carried state:
//
//   S  = Q Kc^T                                   128 x 128 x 64   smem x smem
//   O  = Qs Mb^T           Qs_i = hs * decay^(i+1) q_i,  Mb = bf16(M_{c-1})
//   M  = decay^len M + Vw^T Kc       Vw_j = coeff * decay^(len-1-j) v_j        (state, TMEM)
//   O += P Vc              P_ij = hs * coeff * decay^(i-j) S_ij (j <= i)       TMEM x smem
//   out = O
//
// which is the closed form of the reference chunk (grm/core/cuda_ops.py:218-254) with the state
// carried across chunks as in grm/csrc/grm_cuda.cpp:67-83.  Roles:
//
//   warp 12      issuer A (one thread): O_c(P part) | S_{c+2} | TMA loads of chunk c+3 (3-stage ring)
//   warp 13      issuer B (one thread): O_c(state part), M_c  -- the only products on the
//                recurrence, so that the serial chain is state pass -> 12 MMAs -> state pass
//   warps 8-11   copy group: Vw_c and Qs_c, the two decay-scaled copies, ahead of the issuer
//   warps 0-3    compute group 0, chunks 0, 2, 4, ...
//   warps 4-7    compute group 1, chunks 1, 3, 5, ...
//                each: S_c -> P_c (decay mask, bf16, written back into the TMEM columns of S_c),
//                      state pass (M_c -> bf16 copy for the next chunk, rescale in TMEM),
//                      epilogue (O_c -> bf16 -> HBM)
//
// P never touches shared memory: O += P Vc takes its A operand from TMEM.  TMEM (512 columns):
// two S/P buffers (one per compute group), two O buffers, the state.  Every hand-off is an
// mbarrier; a waiter is never more than one phase behind its producer (protocol comment in the
// kernel) and every wait is bounded: on expiry the CTA-wide abort flag is raised, all roles drain,
// the error word gets bit 1, TMEM is freed and the kernel returns.
#include <cuda.h>

#include <mutex>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

using namespace tc;

constexpr int kChunk = 128;
constexpr int kD = 64;                 // d_k == d_v
constexpr int kStages = 3;
constexpr int kThreads = 448;          // 14 warps (registers are granted as for 16: 128 per thread)
constexpr int kCopyWarp0 = 8;          // warps 8-11, one token row per thread
constexpr int kCopyThreads = 128;
constexpr int kIssuerA = 12;           // S, P part of O, TMA; also owns the TMEM allocation
constexpr int kIssuerB = 13;           // state part of O, state update
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;          // + 128 * group : S (128 cols), then P in cols 0-63 (bf16 pairs)
constexpr uint32_t kColO = 256;        // + 64 * group  : O
constexpr uint32_t kColM = 384;        // state: 64 columns, lanes 0-15 of each quarter

constexpr int kTileBytes = kChunk * kD * 2;          // 16 KiB: one [128 x 64] bf16 tile
constexpr int kStageBytes = 3 * kTileBytes;          // q, k, v
constexpr int kOffStage = 0;
constexpr int kOffVw = kStages * kStageBytes;        // two buffers
constexpr int kOffQs = kOffVw + 2 * kTileBytes;      // two buffers
constexpr int kOffMb = kOffQs + 2 * kTileBytes;      // [64 x 64] bf16
// Decay weights of P, reversed (entry m holds weight(d = 127 - m), zero for d < 0) and stored as
// four copies shifted by 0..3 entries so that any run of 32 weights can be read with aligned
// 16-byte loads; copies are 264 floats apart, which keeps the eight lanes of a load phase on
// distinct banks.
constexpr int kWcopy = 264;
constexpr int kOffWtab = kOffMb + kD * kD * 2;
constexpr int kOffPow = kOffWtab + 4 * kWcopy * 4;   // float[kChunk + 4]: decay^j
constexpr int kOffBars = kOffPow + (kChunk + 4) * 4;
constexpr int kNumBars = 24;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemTotal = kOffMisc + 32;
constexpr int kSmemAlloc = kSmemTotal + 1024;
static_assert(kSmemAlloc <= 232448, "shared memory plan exceeds 227 KiB");

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// descriptor + byte offset (the start-address field holds addr >> 4 in its low 14 bits)
__device__ __forceinline__ uint64_t desc_add(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

__global__ void __launch_bounds__(kThreads, 1)
linear_scan_tc_pipe_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, ScanParams p, SplitInfo split,
                           uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_wtab = reinterpret_cast<float*>(smem + kOffWtab);
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full = bars;              // [3] TMA bytes landed                             (1 + tx)
  uint64_t* bar_s_done = bars + 6;        // [2] S_c complete                                 (commit)
  uint64_t* bar_p_ready = bars + 8;       // [2] P_c in TMEM                                  (128)
  uint64_t* bar_vq_ready = bars + 10;     // [2] Vw_c and Qs_c written                        (128)
  uint64_t* bar_d_done = bars + 12;       // [2] state part of O_c and M_c complete           (commit)
  uint64_t* bar_o_done = bars + 14;       // [2] O_c complete                                 (commit)
  uint64_t* bar_o_free = bars + 16;       // [2] epilogue c has read O_c                      (128)
  uint64_t* bar_state_ready = bars + 18;  // [1] bf16 state copy + rescaled TMEM state        (128)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // The call may be cut along T into `split.pieces` pieces of `split.chunks_per_piece` chunks, one
  // CTA per (piece, row), piece-major.  Piece q > 0 starts from the state that the pieces before it
  // leave behind, rebuilt in its prologue from memory_in and their local contributions in
  // `split.partials` (written by the piece-state kernel that runs before this one).
  const int64_t b = blockIdx.x % p.B;
  const int piece = static_cast<int>(blockIdx.x / p.B);
  const int T = static_cast<int>(p.T);
  const int total_chunks = (T + kChunk - 1) / kChunk;
  const int c_begin = piece * split.chunks_per_piece;
  const int n_chunks = min(split.chunks_per_piece, total_chunks - c_begin);   // chunks of this CTA
  const bool rev = p.reverse != 0;
  // Global chunk g covers processing steps [128g, 128g + len).  Forward, tile row r is step r of
  // the chunk; in a reverse scan the tile is still loaded in memory order, so row r is step
  // 127 - r and the tile of a short last chunk starts at a negative token (TMA fills with 0).
  auto chunk_len = [&](int g) { return min(kChunk, T - g * kChunk); };
  auto chunk_token0 = [&](int g) { return rev ? T - (g + 1) * kChunk : g * kChunk; };
  auto first_offset = [&](int g) { return (g == 0 && p.first_step_no_decay) ? 1 : 0; };

  // ---- set-up (all threads) ----
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar_full[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s_done[i], 1);
      mbar_init(&bar_p_ready[i], 128);
      mbar_init(&bar_vq_ready[i], kCopyThreads);
      mbar_init(&bar_d_done[i], 1);
      mbar_init(&bar_o_done[i], 1);
      mbar_init(&bar_o_free[i], 128);
    }
    mbar_init(bar_state_ready, 128);
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

  uint8_t* s_mb = smem + kOffMb;
  auto stage_q = [&](int s) { return smem + kOffStage + s * kStageBytes; };
  auto stage_k = [&](int s) { return stage_q(s) + kTileBytes; };
  auto stage_v = [&](int s) { return stage_q(s) + 2 * kTileBytes; };
  auto vw_buf = [&](int i) { return smem + kOffVw + i * kTileBytes; };
  auto qs_buf = [&](int i) { return smem + kOffQs + i * kTileBytes; };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  // Protocol.  Chunks are numbered locally, c = 0 .. n_chunks-1; "X(c)" is the completion of
  // barrier X that belongs to chunk c (phase c/2 of X[c&1], phase c/3 of X[c%3]).  A waiter is
  // never more than one completion behind, because the producer's next completion on the same
  // barrier needs something that comes after the waiter's wait:
  //   issuer B: O_c(state part), M_c need vq_ready(c)    <- copy group     <- full(c), d_done(c-2)
  //                                       state_ready(c) <- state pass c-1 <- d_done(c-1)
  //                                       o_free(c-2)    <- epilogue c-2   <- o_done(c-2)
  //   issuer A: O_c(P part)          needs p_ready(c)    <- P pass c       <- s_done(c)
  //                                        d_done(c)     (the state part is accumulated first)
  //             S_{c+2}              needs o_done(c) (O_c reads its S/P buffer) and full(c+2)
  //             TMA of chunk c+3     needs o_done(c): every reader of stage c%3 has retired

  if (warp == kIssuerA) {
    // ===================================================================== issuer A + TMA
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kChunk, kChunk, 0, 0);
      constexpr uint32_t idesc_op = make_idesc(kChunk, kD, 0, 1);
      int loads_issued = 0;

      auto issue_loads = [&](int c) {
        const int s = c % kStages;
        mbar_expect_tx(&bar_full[s], kStageBytes);
        const int t0 = chunk_token0(c_begin + c);
        tma_load_3d(stage_q(s), &map_q, &bar_full[s], 0, t0, static_cast<int>(b));
        tma_load_3d(stage_k(s), &map_k, &bar_full[s], 0, t0, static_cast<int>(b));
        tma_load_3d(stage_v(s), &map_v, &bar_full[s], 0, t0, static_cast<int>(b));
        loads_issued = c + 1;
      };
      auto issue_s = [&](int c) {
        const int s = c % kStages;
        const uint64_t dq = smem_desc(smem_u32(stage_q(s)), 16, 1024);
        const uint64_t dk = smem_desc(smem_u32(stage_k(s)), 16, 1024);
        const uint32_t d_tmem = tmem_base + kColS + 128u * (c & 1);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          tc_mma_bf16(d_tmem, desc_add(dq, kk * 32), desc_add(dk, kk * 32), idesc_s, kk > 0);
        }
        tc_commit(&bar_s_done[c & 1]);
      };

      for (int c = 0; c < n_chunks && c < kStages; ++c) issue_loads(c);
      do {
        GRMX_WAIT(&bar_full[0], 0)
        tc_fence_after();
        issue_s(0);
        if (n_chunks > 1) {
          GRMX_WAIT(&bar_full[1], 0)
          tc_fence_after();
          issue_s(1);
        }
        for (int c = 0; c < n_chunks; ++c) {
          const int s = c % kStages;
          const int g = c & 1;
          GRMX_WAIT(&bar_p_ready[g], c / 2)
          GRMX_WAIT(&bar_d_done[g], c / 2)
          tc_fence_after();
          {
            const uint64_t dv_mn = smem_desc(smem_u32(stage_v(s)), kTileBytes, 1024);
            const uint32_t p_tmem = tmem_base + kColS + 128u * g;   // 16 tokens of P = 8 columns
            const uint32_t o_tmem = tmem_base + kColO + 64u * g;
#pragma unroll
            for (int kk = 0; kk < kChunk / 16; ++kk) {
              tc_mma_bf16_ts(o_tmem, p_tmem + 8u * kk, desc_add(dv_mn, kk * 2048), idesc_op, 1u);
            }
            tc_commit(&bar_o_done[g]);
          }
          if (c + 2 < n_chunks) {
            GRMX_WAIT(&bar_full[(c + 2) % kStages], (c + 2) / kStages)
            GRMX_WAIT(&bar_o_done[g], c / 2)       // O_c has consumed P_c: the S/P buffer is free
            tc_fence_after();
            issue_s(c + 2);
            if (c + 3 < n_chunks) issue_loads(c + 3);   // stage c % 3: all its readers retired with O_c
          }
        }
      } while (false);
      if (*s_abort) {
        // let the copies still in flight land before the shared memory is released
        for (int c = loads_issued > kStages ? loads_issued - kStages : 0; c < loads_issued; ++c) {
          mbar_wait_quiet(&bar_full[c % kStages], (c / kStages) & 1);
        }
      }
    }
  } else if (warp == kIssuerB) {
    // ===================================================================== issuer B
    if (lane == 0) {
      constexpr uint32_t idesc_oq = make_idesc(kChunk, kD, 0, 0);
      constexpr uint32_t idesc_m = make_idesc(kD, kD, 1, 1);
      const uint64_t desc_mb = smem_desc(smem_u32(s_mb), 16, 1024);
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c % kStages;
        const int g = c & 1;
        GRMX_WAIT(&bar_vq_ready[g], c / 2)
        if (c >= 2) GRMX_WAIT(&bar_o_free[g], c / 2 - 1)
        GRMX_WAIT(bar_state_ready, c)
        tc_fence_after();
        const uint64_t dqs = smem_desc(smem_u32(qs_buf(g)), 16, 1024);
        const uint64_t dk_mn = smem_desc(smem_u32(stage_k(s)), kTileBytes, 1024);
        const uint64_t dvw = smem_desc(smem_u32(vw_buf(g)), kTileBytes, 1024);
        const uint32_t o_tmem = tmem_base + kColO + 64u * g;
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk) {
          tc_mma_bf16(tmem_base + kColM, desc_add(dvw, kk * 2048), desc_add(dk_mn, kk * 2048), idesc_m, 1u);
        }
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          tc_mma_bf16(o_tmem, desc_add(dqs, kk * 32), desc_add(desc_mb, kk * 32), idesc_oq, kk > 0);
        }
        tc_commit(&bar_d_done[g]);
      }
    }
  } else if (warp >= kCopyWarp0) {
    // ===================================================================== copy group (warps 8-11)
    const int row = tid - kCopyWarp0 * 32;
    const int step = rev ? kChunk - 1 - row : row;
    for (int c = 0; c < n_chunks; ++c) {
      GRMX_WAIT(&bar_full[c % kStages], c / kStages)
      if (c >= 2) GRMX_WAIT(&bar_d_done[c & 1], c / 2 - 1)
      const int g = c_begin + c;
      const int len = chunk_len(g);
      const bool live = step < len;
      const float w_v = live ? p.update_coeff * s_pow[len - 1 - step] : 0.0f;
      const float w_q = live ? p.hidden_scale * s_pow[step + 1 - first_offset(g)] : 0.0f;
      scaled_row_copy(stage_v(c % kStages), vw_buf(c & 1), row, w_v);
      scaled_row_copy(stage_q(c % kStages), qs_buf(c & 1), row, w_q);
      fence_proxy_async();
      mbar_arrive(&bar_vq_ready[c & 1]);
    }
  } else {
    // ===================================================================== compute groups (warps 0-7)
    const int g = warp >> 2;                  // group 0: even chunks, group 1: odd chunks
    const int quarter = warp & 3;
    const int row = tid & 127;                // token row within the chunk == TMEM lane
    const int step = rev ? kChunk - 1 - row : row;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_row = tmem_lane + kColS + 128u * g;
    const uint32_t o_row = tmem_lane + kColO + 64u * g;
    const bool owns_row = lane < 16;          // M = 64 accumulator: lanes 0-15 of each quarter
    const int state_row = quarter * 16 + (lane & 15);
    // decay applied to the carried state over chunk c (the state in TMEM is kept pre-scaled by it)
    auto carry_of = [&](int c) { return s_pow[chunk_len(c_begin + c) - first_offset(c_begin + c)]; };

    auto write_mb = [&](const float (&v)[32], int c0) {
      uint8_t* mrow = s_mb + state_row * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int chunk16 = (c0 / 8 + ch) ^ (state_row & 7);
        uint4 w;
        w.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
        w.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
        w.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
        w.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(mrow + chunk16 * 16) = w;
      }
    };

    if (g == 0) {
      // state at the start of this CTA's chunks -> bf16 copy + TMEM (pre-scaled by the first carry)
      const float* m_in = static_cast<const float*>(p.memory_in) + b * kD * kD;
      const bool dense = p.m_col_stride == 1;
#pragma unroll 1
      for (int c0 = 0; c0 < kD; c0 += 32) {
        float v[32];
        if (owns_row && dense) {
          const float4* src = reinterpret_cast<const float4*>(m_in + state_row * p.m_row_stride + c0);
          const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (vec) {
              const float4 x = __ldg(src + j);
              v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) v[4 * j + e] = m_in[state_row * p.m_row_stride + c0 + 4 * j + e];
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = owns_row ? m_in[state_row * p.m_row_stride + (c0 + j) * p.m_col_stride] : 0.0f;
          }
        }
        // pieces before this one: M <- decay^(tokens of piece q - offset) M + partial_q
        for (int q = 0; q < piece; ++q) {
          const int q_tokens = min(split.chunks_per_piece * kChunk, T - q * split.chunks_per_piece * kChunk);
          const float gq = powf(p.decay, static_cast<float>(q_tokens - first_offset(q * split.chunks_per_piece)));
          if (owns_row) {
            const float4* part = reinterpret_cast<const float4*>(
                split.partials + ((b * (split.pieces - 1) + q) * kD + state_row) * kD + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 x = __ldg(part + j);
              v[4 * j] = fmaf(gq, v[4 * j], x.x);
              v[4 * j + 1] = fmaf(gq, v[4 * j + 1], x.y);
              v[4 * j + 2] = fmaf(gq, v[4 * j + 2], x.z);
              v[4 * j + 3] = fmaf(gq, v[4 * j + 3], x.w);
            }
          }
        }
        if (owns_row) write_mb(v, c0);
        const float carry = carry_of(0);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= carry;
        tc_st32(tmem_lane + kColM + c0, v);
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_state_ready);   // completion 0
    }

    for (int c = g; c < n_chunks; c += 2) {
      const bool last = c + 1 == n_chunks;
      // ---- P pass: S_c -> P_c in place ----
      // Warp w owns rows 32w..32w+31, so 32-column blocks above block w (below it in a reverse
      // scan) are all zero.  P block b (16 packed columns) overwrites the S columns 16b..16b+15,
      // which belong to S blocks 0 and 1: those two are in registers before anything is stored.
      GRMX_WAIT(&bar_s_done[g], c / 2)
      tc_fence_after();
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        // P block blk lands on S columns 16*blk..16*blk+15, i.e. inside S block blk/2, which has been
        // read by the time it is overwritten (blocks are visited in increasing order)
        uint32_t pk[16];
        if (rev ? blk >= quarter : blk <= quarter) {
          uint32_t sv[32];
          tc_ld32_async(s_row + 32u * blk, sv);
          const int m0 = 127 - row + 32 * blk;            // reversed-table index of column 32*blk
          const float4* wv = reinterpret_cast<const float4*>(s_wtab + (m0 & 3) * kWcopy + (m0 & ~3));
          tc_wait_ld();
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
        tc_st16_async(s_row + 16u * blk, pk);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bar_p_ready[g]);

      // ---- state pass: M_c is complete ----
      GRMX_WAIT(&bar_d_done[g], c / 2)
      tc_fence_after();
      {
        float* m_out = (last && p.memory_out != nullptr && piece + 1 == split.pieces)
                           ? static_cast<float*>(p.memory_out) + b * kD * kD
                           : nullptr;
        const float carry = last ? 0.0f : carry_of(c + 1);
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 32) {
          float v[32];
          tc_ld32(tmem_lane + kColM + c0, v);
          if (last) {
            if (owns_row && m_out != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o;
                o.x = v[j] * p.memory_out_scale;
                o.y = v[j + 1] * p.memory_out_scale;
                o.z = v[j + 2] * p.memory_out_scale;
                o.w = v[j + 3] * p.memory_out_scale;
                *reinterpret_cast<float4*>(m_out + state_row * kD + c0 + j) = o;
              }
            }
          } else {
            if (owns_row) write_mb(v, c0);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= carry;
            tc_st32(tmem_lane + kColM + c0, v);
          }
        }
        if (!last) {
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(bar_state_ready);   // completion c + 1
        }
      }

      // ---- epilogue: O_c -> bf16 -> HBM ----
      GRMX_WAIT(&bar_o_done[g], c / 2)
      tc_fence_after();
      {
        const bool row_live = step < chunk_len(c_begin + c);
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.hidden_out) +
                             (b * p.T + static_cast<int64_t>(chunk_token0(c_begin + c)) + row) * kD;
        uint32_t o[2][32];
        tc_ld32_async(o_row, o[0]);
        tc_ld32_async(o_row + 32u, o[1]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bar_o_free[g]);     // the values are in registers: the O buffer may be reused
        if (row_live) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(o[h][ch * 8 + 0]), __uint_as_float(o[h][ch * 8 + 1]));
              w.y = pack_bf16(__uint_as_float(o[h][ch * 8 + 2]), __uint_as_float(o[h][ch * 8 + 3]));
              w.z = pack_bf16(__uint_as_float(o[h][ch * 8 + 4]), __uint_as_float(o[h][ch * 8 + 5]));
              w.w = pack_bf16(__uint_as_float(o[h][ch * 8 + 6]), __uint_as_float(o[h][ch * 8 + 7]));
              *reinterpret_cast<uint4*>(out + 32 * h + ch * 8) = w;
            }
          }
        }
      }
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

bool scan_tcgen05_pipe_supported(const ScanParams& p) { return p.K == kD && p.H == kD; }

int launch_scan_tcgen05_pipe(const ScanParams& p, const SplitInfo& split, cudaStream_t stream) {
  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(linear_scan_tc_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemAlloc);
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cannot reserve %d bytes of shared memory: %s", kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_k, map_v;
  if (!make_token_map(&map_q, p.queries, p.B, p.T, kD) || !make_token_map(&map_k, p.keys, p.B, p.T, kD) ||
      !make_token_map(&map_v, p.values, p.B, p.T, kD)) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cuTensorMapEncodeTiled failed");
  }
  linear_scan_tc_pipe_kernel<<<static_cast<unsigned>(p.B * split.pieces), kThreads, kSmemAlloc, stream>>>(
      map_q, map_k, map_v, p, split, device_error_word_ptr());
  return check_launch("linear_scan_tcgen05_pipe");
}

}  // namespace grmx
