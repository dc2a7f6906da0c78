// Per-token retrieval on the tensor cores: gather + apply-query + gate-weighted sum + residual +
// LayerNorm for tokens that each choose R of the S archived matrices of their batch row, without
// the gathered [B, Q, R, H, K] tensor of the reference (grm/core/paper_grm.py:229-234), without its
// apply-query over that tensor (grm/core/paper_grm.py:301-307, grm/csrc/apply_query.cu:14-75) and
// without a candidate tensor [B, Q, S, H] either.
//
// For a tile of 128 tokens of one batch row
//
//   contrib[t, :] = sum_r gate[t, r] * M[idx[t, r]] q[t]  =  sum_s M_s (g_s[t] q[t]),
//   g_s[t] = sum of the gates of token t whose route is slot s (zero when it chose another slot),
//
// which is ONE product per slot accumulated in the same TMEM accumulator: A_s = diag(g_s) Q, the
// tile's queries scaled row by row (bf16, built by CUDA cores from the one q tile in shared memory),
// times B_s = M_s [H x K] as it lies in the bf16 archive ring (K-major, loaded by TMA).  Slots that no
// token of the tile chose are skipped.  The epilogue adds the online state, normalises the row
// (grm/core/aggregator.py:104-105, 116-118, 144) and writes bf16; a token without any live route keeps
// its online state untouched (grm/core/paper_grm.py:620-621).
//
// Persistent CTAs, one tile at a time.  Roles: warps 0-3 epilogue (thread = token row = TMEM lane),
// warps 4-7 build A_s, warp 8 loads (TMA), warp 9 issues the products.  Shared memory: the q tile, two
// A buffers, two stages for B_s (H x 128 bytes each).  TMEM: one accumulator [128 x H] fp32.  All
// waits are bounded; on expiry the CTA raises its abort flag, drains, sets bit 1 of the device error
// word and returns.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

using namespace tc;

constexpr int kTile = 128;
constexpr int kK = 64;
constexpr int kMaxH = 512;
constexpr int kMaxSlots = 32;
constexpr int kMaxRoutes = 8;
constexpr int kThreads = 320;
constexpr int kBuilderWarp0 = 4;
constexpr int kLoaderWarp = 8;
constexpr int kIssuerWarp = 9;

constexpr int kTileBytes = kTile * kK * 2;            // 16 KiB: [128 x 64] bf16
constexpr int kStageBytes = kMaxH * kK * 2;           // 64 KiB: [512 x 64] bf16
constexpr int kOffQ = 0;
constexpr int kOffA = kTileBytes;                     // two buffers
constexpr int kOffB = 3 * kTileBytes;                 // two stages
constexpr int kOffLn = kOffB + 2 * kStageBytes;       // float weight[512], bias[512]
constexpr int kOffLive = kOffLn + 2 * kMaxH * 4;      // uint8 live[2][128]
constexpr int kOffBars = kOffLive + 2 * kTile;
constexpr int kNumBars = 16;
constexpr int kOffMisc = kOffBars + kNumBars * 8;     // tmem address, abort flag, slot masks
constexpr int kSmemTotal = kOffMisc + 64;
constexpr int kSmemAlloc = kSmemTotal + 1024;
static_assert(kSmemAlloc <= 232448, "shared memory plan exceeds 227 KiB");

struct Params {
  const int64_t* indices;   // [B, Q, R]
  const float* gates;       // [B, Q, R]
  const __nv_bfloat16* online;   // [B, Q, H] or null
  const float* ln_weight;   // [H] or null
  const float* ln_bias;     // [H] or null
  __nv_bfloat16* out;       // [B, Q, H]
  int B, S, Q, R, H;
  int tiles_per_row;
  int n_tiles;
  float eps;
  int mode;
};

// The slot mask of a tile is kept as one word per builder warp (each warp writes its own, nobody has to
// clear anything); readers OR the four.
__device__ __forceinline__ uint32_t tile_mask(const uint32_t* words) { return words[0] | words[1] | words[2] | words[3]; }

__global__ void __launch_bounds__(kThreads, 1)
retrieve_fuse_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_ring,
                        Params p, uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_lnw = reinterpret_cast<float*>(smem + kOffLn);
  float* s_lnb = s_lnw + kMaxH;
  uint8_t* s_live = smem + kOffLive;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full_q = bars;          // [1] q tile landed                              (1 + tx)
  uint64_t* bar_q_free = bars + 1;      // [1] the builders are done with the q tile      (128)
  uint64_t* bar_full_b = bars + 2;      // [2] B_s landed                                 (1 + tx)
  uint64_t* bar_b_free = bars + 4;      // [2] the product that read the stage retired    (commit)
  uint64_t* bar_a_ready = bars + 6;     // [2] A_s written                                (128)
  uint64_t* bar_a_free = bars + 8;      // [2] the product that read the buffer retired   (commit)
  uint64_t* bar_mask_ready = bars + 10; // [2] slot mask and live flags of the tile       (128)
  uint64_t* bar_mask_free = bars + 12;  // [2] loader, issuer and epilogue have read them (1 + 1 + 128)
  uint64_t* bar_acc_ready = bars + 14;  // [1] all products of the tile retired           (commit)
  uint64_t* bar_acc_free = bars + 15;   // [1] the epilogue has read the accumulator      (128)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);
  uint32_t* s_mask = reinterpret_cast<uint32_t*>(smem + kOffMisc + 16);   // [2][4]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int H = p.H;
  const uint32_t tmem_cols = H > 256 ? 512u : (H > 128 ? 256u : (H > 64 ? 128u : 64u));

  if (tid == 0) {
    mbar_init(bar_full_q, 1);
    mbar_init(bar_q_free, 128);
    mbar_init(bar_acc_ready, 1);
    mbar_init(bar_acc_free, 128);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_full_b[i], 1);
      mbar_init(&bar_b_free[i], 1);
      mbar_init(&bar_a_ready[i], 128);
      mbar_init(&bar_a_free[i], 1);
      mbar_init(&bar_mask_ready[i], 128);
      mbar_init(&bar_mask_free[i], 130);
    }
    *s_abort = 0;
    for (int i = 0; i < 8; ++i) s_mask[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int j = tid; j < H; j += kThreads) {
    s_lnw[j] = p.ln_weight != nullptr ? p.ln_weight[j] : 1.0f;
    s_lnb[j] = p.ln_bias != nullptr ? p.ln_bias[j] : 0.0f;
  }
  if (warp == kIssuerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  uint8_t* const q_smem = smem + kOffQ;
  auto a_smem = [&](int n) { return smem + kOffA + (n & 1) * kTileBytes; };
  auto b_smem = [&](int n) { return smem + kOffB + (n & 1) * kStageBytes; };
  // Tiles in an order that puts the late (many visible slots, expensive) tiles of every batch row first.
  auto tile_of = [&](int it, int* b, int* t0) {
    const int o = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
    if (o >= p.n_tiles) return false;
    *b = o % p.B;
    *t0 = (p.tiles_per_row - 1 - o / p.B) * kTile;
    return true;
  };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  if (warp == kLoaderWarp) {
    // ===================================================================== loader
    if ((tid & 31) == 0) {
      int n = 0, nq = 0, b = 0, t0 = 0;
      const uint32_t stage_tx = static_cast<uint32_t>((H + 127) / 128) * kTileBytes;   // whole boxes of 128 rows
      for (int it = 0; tile_of(it, &b, &t0); ++it) {
        if (it >= 1) GRMX_WAIT(bar_q_free, it - 1)
        mbar_expect_tx(bar_full_q, kTileBytes);
        tma_load_3d(q_smem, &map_q, bar_full_q, 0, t0, b);
        ++nq;
        GRMX_WAIT(&bar_mask_ready[it & 1], it / 2)
        const uint32_t mask = tile_mask(s_mask + 4 * (it & 1));
        mbar_arrive(&bar_mask_free[it & 1]);
        bool ok = true;
        for (uint32_t rest = mask; rest != 0 && ok; rest &= rest - 1) {
          const int s = __ffs(rest) - 1;
          ok = false;
          do {
            if (n >= 2) GRMX_WAIT(&bar_b_free[n & 1], n / 2 - 1)
            mbar_expect_tx(&bar_full_b[n & 1], stage_tx);
            for (int n0 = 0; n0 < H; n0 += 128) {
              tma_load_3d(b_smem(n) + n0 * kK * 2, &map_ring, &bar_full_b[n & 1], 0, s * H + n0, b);
            }
            ++n;
            ok = true;
          } while (false);
        }
        if (!ok) break;
      }
      if (*s_abort) {
        // let copies in flight land before the shared memory is released
        if (nq > 0) mbar_wait_quiet(bar_full_q, (nq - 1) & 1);
        for (int j = n > 2 ? n - 2 : 0; j < n; ++j) mbar_wait_quiet(&bar_full_b[j & 1], (j / 2) & 1);
      }
    }
  } else if (warp == kIssuerWarp) {
    // ===================================================================== issuer
    if ((tid & 31) == 0) {
      int n = 0, na = 0, b = 0, t0 = 0;
      for (int it = 0; tile_of(it, &b, &t0); ++it) {
        GRMX_WAIT(&bar_mask_ready[it & 1], it / 2)
        const uint32_t mask = tile_mask(s_mask + 4 * (it & 1));
        mbar_arrive(&bar_mask_free[it & 1]);
        if (mask == 0) continue;
        if (na >= 1) GRMX_WAIT(bar_acc_free, na - 1)
        bool ok = true, first = true;
        for (uint32_t rest = mask; rest != 0 && ok; rest &= rest - 1) {
          ok = false;
          do {
            GRMX_WAIT(&bar_a_ready[n & 1], n / 2)
            GRMX_WAIT(&bar_full_b[n & 1], n / 2)
            tc_fence_after();
            const uint64_t da = smem_desc(smem_u32(a_smem(n)), 16, 1024);
            for (int n0 = 0; n0 < H; n0 += 256) {
              const int nlen = min(256, H - n0);
              const uint64_t db = smem_desc(smem_u32(b_smem(n) + n0 * kK * 2), 16, 1024);
              const uint32_t idesc = make_idesc(kTile, nlen, 0, 0);
#pragma unroll
              for (int kk = 0; kk < kK / 16; ++kk) {
                tc_mma_bf16(tmem_base + n0, desc_add(da, kk * 32), desc_add(db, kk * 32), idesc, (first && kk == 0) ? 0u : 1u);
              }
            }
            tc_commit(&bar_a_free[n & 1]);
            tc_commit(&bar_b_free[n & 1]);
            first = false;
            ++n;
            ok = true;
          } while (false);
        }
        if (!ok) break;
        tc_commit(bar_acc_ready);
        ++na;
      }
    }
  } else if (warp >= kBuilderWarp0 && warp < kBuilderWarp0 + 4) {
    // ===================================================================== A builders (thread = token row)
    const int row = tid - kBuilderWarp0 * 32;
    int n = 0, b = 0, t0 = 0;
    for (int it = 0; tile_of(it, &b, &t0); ++it) {
      const int token = t0 + row;
      int idx[kMaxRoutes];
      float gate[kMaxRoutes];
      uint32_t mine = 0;
#pragma unroll
      for (int r = 0; r < kMaxRoutes; ++r) {
        idx[r] = -1;
        gate[r] = 0.0f;
        if (r < p.R && token < p.Q) {
          const int64_t at = (static_cast<int64_t>(b) * p.Q + token) * p.R + r;
          const int64_t v = __ldg(p.indices + at);
          if (v >= 0 && v < p.S) {
            idx[r] = static_cast<int>(v);
            gate[r] = __ldg(p.gates + at);
            mine |= 1u << idx[r];
          } else if (v != -1 && error_word != nullptr) {
            atomicOr(error_word, kErrGatherIndex);        // treated as an empty route
          }
        }
      }
      if (it >= 2) GRMX_WAIT(&bar_mask_free[it & 1], it / 2 - 1)
      const uint32_t warp_mask = __reduce_or_sync(0xffffffffu, mine);
      if ((tid & 31) == 0) s_mask[4 * (it & 1) + (warp - kBuilderWarp0)] = warp_mask;
      s_live[(it & 1) * kTile + row] = mine != 0 ? 1 : 0;
      mbar_arrive(&bar_mask_ready[it & 1]);
      GRMX_WAIT(&bar_mask_ready[it & 1], it / 2)
      const uint32_t mask = tile_mask(s_mask + 4 * (it & 1));
      GRMX_WAIT(bar_full_q, it)
      bool ok = true;
      for (uint32_t rest = mask; rest != 0 && ok; rest &= rest - 1) {
        const int s = __ffs(rest) - 1;
        ok = false;
        do {
          if (n >= 2) GRMX_WAIT(&bar_a_free[n & 1], n / 2 - 1)
          float g = 0.0f;
#pragma unroll
          for (int r = 0; r < kMaxRoutes; ++r) g += idx[r] == s ? gate[r] : 0.0f;
          scaled_row_copy<8>(q_smem, a_smem(n), row, g);
          fence_proxy_async();
          mbar_arrive(&bar_a_ready[n & 1]);
          ++n;
          ok = true;
        } while (false);
      }
      if (!ok) break;
      mbar_arrive(bar_q_free);
    }
  } else if (warp < 4) {
    // ===================================================================== epilogue (thread = token row)
    const int row = tid;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float inv_h = 1.0f / static_cast<float>(H);
    int na = 0, b = 0, t0 = 0;
    for (int it = 0; tile_of(it, &b, &t0); ++it) {
      GRMX_WAIT(&bar_mask_ready[it & 1], it / 2)
      const uint32_t mask = tile_mask(s_mask + 4 * (it & 1));
      const bool live = s_live[(it & 1) * kTile + row] != 0;
      mbar_arrive(&bar_mask_free[it & 1]);
      const int token = t0 + row;
      const bool valid = token < p.Q;
      const int64_t base = (static_cast<int64_t>(b) * p.Q + token) * H;
      const uint4* h_row = (p.online != nullptr && valid) ? reinterpret_cast<const uint4*>(p.online + base) : nullptr;
      uint4* o_row = reinterpret_cast<uint4*>(p.out + base);
      if (mask == 0) {
        // nobody in the tile has a route: the online state passes through (zeros in contribution mode)
        if (valid) {
          for (int j = 0; j < H / 8; ++j) {
            o_row[j] = (p.mode == GRMX_FUSE_RESIDUAL_LN && h_row != nullptr) ? __ldg(h_row + j) : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        continue;
      }
      // the row of the online state is needed when the products of the tile are done: ask L2 for it now
      if (p.mode == GRMX_FUSE_RESIDUAL_LN && h_row != nullptr) {
        for (int j = 0; j < H / 64; ++j) asm volatile("prefetch.global.L2 [%0];" ::"l"(h_row + 8 * j));
      }
      GRMX_WAIT(bar_acc_ready, na)
      tc_fence_after();
      if (p.mode == GRMX_FUSE_CONTRIB) {
        for (int c0 = 0; c0 < H; c0 += 32) {
          uint32_t v[32];
          tc_ld32_async(lane_addr + c0, v);
          tc_wait_ld();
          if (valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
              w.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              w.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              w.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
              o_row[c0 / 8 + j] = live ? w : make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
      } else {
        // pass 1: x = contribution + online state, written back over the accumulator; row sum and sum of
        // squares (one pass over TMEM less than a variance about the mean: with rows of at most 512 values
        // of order one the difference of the two means is good to a few parts in a million, far inside the
        // bf16 rounding of the output)
        float sum = 0.0f, sq = 0.0f;
        // the 64 bytes of online state that go with 32 columns are loaded one step ahead
        uint4 ahead[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) ahead[j] = h_row != nullptr ? __ldg(h_row + j) : make_uint4(0u, 0u, 0u, 0u);
        for (int c0 = 0; c0 < H; c0 += 32) {
          uint32_t v[32];
          tc_ld32_async(lane_addr + c0, v);
          uint4 now[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) now[j] = ahead[j];
          if (c0 + 32 < H && h_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) ahead[j] = __ldg(h_row + (c0 + 32) / 8 + j);
          }
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 hw = now[j];
            const uint32_t words[4] = {hw.x, hw.y, hw.z, hw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = __uint_as_float(words[i] << 16), hi = __uint_as_float(words[i] & 0xffff0000u);
              const float x0 = (live ? __uint_as_float(v[8 * j + 2 * i]) : 0.0f) + lo;
              const float x1 = (live ? __uint_as_float(v[8 * j + 2 * i + 1]) : 0.0f) + hi;
              v[8 * j + 2 * i] = __float_as_uint(x0);
              v[8 * j + 2 * i + 1] = __float_as_uint(x1);
              sum += x0 + x1;
              sq = fmaf(x0, x0, fmaf(x1, x1, sq));
            }
          }
          tc_st32_async(lane_addr + c0, v);
        }
        tc_wait_st();
        const float mean = sum * inv_h;
        const float rstd = rsqrtf(fmaxf(sq * inv_h - mean * mean, 0.0f) + p.eps);
        // pass 2: normalise (a token without a live route keeps its online state as it is) and store
        for (int c0 = 0; c0 < H; c0 += 32) {
          uint32_t v[32];
          tc_ld32_async(lane_addr + c0, v);
          tc_wait_ld();
          if (valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float y[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float x = __uint_as_float(v[8 * j + i]);
                const int c = c0 + 8 * j + i;
                y[i] = live ? (x - mean) * rstd * s_lnw[c] + s_lnb[c] : x;
              }
              uint4 w;
              w.x = pack_bf16(y[0], y[1]);
              w.y = pack_bf16(y[2], y[3]);
              w.z = pack_bf16(y[4], y[5]);
              w.w = pack_bf16(y[6], y[7]);
              o_row[c0 / 8 + j] = w;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_acc_free);
      ++na;
    }
  }
#undef GRMX_WAIT

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *s_abort && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
  if (warp == kIssuerWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_retrieve_fuse_tc(const void* archive_bf16, const int64_t* indices, const float* gates,
                                     const void* queries_bf16, const void* online_bf16, const float* ln_weight,
                                     const float* ln_bias, float ln_eps, void* out_bf16, int64_t B, int64_t S,
                                     int64_t Q, int64_t R, int64_t H, int64_t K, int mode, void* stream) {
  using namespace grmx;
  const char* who = "grmx_retrieve_fuse_tc";
  GRMX_REQUIRE(B >= 0 && S >= 0 && Q >= 0 && R >= 0 && H > 0 && K > 0, "%s: bad sizes", who);
  GRMX_REQUIRE(mode == GRMX_FUSE_CONTRIB || mode == GRMX_FUSE_RESIDUAL_LN, "%s: mode must be contrib or residual_ln", who);
  if (K != kK || H % 64 != 0 || H > kMaxH || S > kMaxSlots || R > kMaxRoutes || S < 1 || R < 1) {
    return fail(GRMX_ERR_UNSUPPORTED,
                "%s: covers K == 64, H a multiple of 64 up to 512, 1 <= S <= 32 slots and 1 <= R <= 8 routes "
                "(use grmx_retrieve_fuse otherwise)", who);
  }
  if (B == 0 || Q == 0) return GRMX_OK;
  GRMX_REQUIRE(archive_bf16 && indices && gates && queries_bf16 && out_bf16, "%s: NULL tensor pointer", who);
  GRMX_REQUIRE(mode != GRMX_FUSE_RESIDUAL_LN || online_bf16, "%s: NULL online state", who);
  const uintptr_t align = reinterpret_cast<uintptr_t>(archive_bf16) | reinterpret_cast<uintptr_t>(queries_bf16) |
                          reinterpret_cast<uintptr_t>(online_bf16) | reinterpret_cast<uintptr_t>(out_bf16);
  GRMX_REQUIRE((align & 15u) == 0, "%s: tensors must be 16-byte aligned", who);
  GRMX_REQUIRE(B <= 0x7fffffffLL && Q <= 0x7fff0000LL && S * H <= 0x7fff0000LL, "%s: sizes exceed the tensor-map range", who);
  if (!tc::device_is_sm100() || tc::encode_tiled_fn() == nullptr) {
    return fail(GRMX_ERR_DEVICE, "%s: needs an sm_100 device with tensor-map support", who);
  }
  static std::mutex mutex;
  static bool configured[64] = {false};
  static int sm_count[64] = {0};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(retrieve_fuse_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
      cudaDeviceGetAttribute(&sm_count[device], cudaDevAttrMultiProcessorCount, device);
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "%s: cannot reserve %d bytes of shared memory: %s", who, kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_ring;
  if (!tc::make_token_map(&map_q, queries_bf16, B, Q, kK) || !tc::make_token_map(&map_ring, archive_bf16, B, S * H, kK)) {
    return fail(GRMX_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed", who);
  }
  Params p;
  p.indices = indices;
  p.gates = gates;
  p.online = static_cast<const __nv_bfloat16*>(online_bf16);
  p.ln_weight = ln_weight;
  p.ln_bias = ln_bias;
  p.out = static_cast<__nv_bfloat16*>(out_bf16);
  p.B = static_cast<int>(B); p.S = static_cast<int>(S); p.Q = static_cast<int>(Q); p.R = static_cast<int>(R);
  p.H = static_cast<int>(H);
  p.tiles_per_row = static_cast<int>((Q + kTile - 1) / kTile);
  const int64_t n_tiles = B * p.tiles_per_row;
  GRMX_REQUIRE(n_tiles <= 0x7fffffffLL, "%s: too many tiles", who);
  p.n_tiles = static_cast<int>(n_tiles);
  p.eps = ln_eps;
  p.mode = mode;
  const int sms = device >= 0 && device < 64 && sm_count[device] > 0 ? sm_count[device] : 148;
  const unsigned grid = static_cast<unsigned>(n_tiles < sms ? n_tiles : sms);
  retrieve_fuse_tc_kernel<<<grid, kThreads, kSmemAlloc, static_cast<cudaStream_t>(stream)>>>(map_q, map_ring, p,
                                                                                             device_error_word_ptr());
  return check_launch("retrieve_fuse_tc");
}
