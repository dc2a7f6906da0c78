// Key and query projections with the L2 normalisation in the epilogue:
//
//   k[n, :] = normalize(x[n, :] Wk^T + bk),   q[n, :] = normalize(x[n, :] Wq^T + bq)      (eps as F.normalize)
//
// (grm/core/paper_grm.py:491-493: F.normalize(key_proj(x)), F.normalize(query_proj(x)); the reference runs
// two Linear layers, then norm, clamp and divide as separate passes over their outputs.)  Here x is read
// once: for a tile of 128 rows the two 64-wide projections are one tcgen05 product [128 x 128 x D] whose
// B operand -- the two weight matrices stacked, [128, D] bf16 -- stays in shared memory for the whole
// kernel; the epilogue adds the bias, takes each 64-wide group's norm and writes the rows as the bf16
// tiles the scan kernel loads.  Persistent CTAs; warp 4 loads (TMA ring over the 64-column blocks of x),
// warp 5 issues, warps 0-3 are the epilogue (thread = row = TMEM lane); two accumulators, so the epilogue
// of a tile runs under the products of the next.  Every wait is bounded.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace {

using namespace tc;

constexpr int kTile = 128;              // rows per tile
constexpr int kGroup = 64;              // width of one projection
constexpr int kN = 2 * kGroup;          // both projections side by side
constexpr int kMaxD = 512;
constexpr int kStages = 5;
constexpr int kThreads = 192;
constexpr int kLoaderWarp = 4;
constexpr int kIssuerWarp = 5;
constexpr int kBlockBytes = kTile * 64 * 2;              // 16 KiB: [128 x 64] bf16
constexpr int kOffW = 0;                                 // D / 64 blocks of [128 x 64]
constexpr int kOffX = (kMaxD / 64) * kBlockBytes;        // ring
constexpr int kOffBias = kOffX + kStages * kBlockBytes;  // float[128]
constexpr int kOffBars = kOffBias + kN * 4;
constexpr int kNumBars = 2 * kStages + 5;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemTotal = kOffMisc + 32;
constexpr int kSmemAlloc = kSmemTotal + 1024;
static_assert(kSmemAlloc <= 232448, "shared memory plan exceeds 227 KiB");

__global__ void __launch_bounds__(kThreads, 1)
project_normalize_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const float* __restrict__ bias, __nv_bfloat16* __restrict__ out_a,
                         __nv_bfloat16* __restrict__ out_b, int64_t rows, int d_blocks, int n_tiles, float eps,
                         uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_bias = reinterpret_cast<float*>(smem + kOffBias);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* bar_full_x = bars;                  // [kStages] x block landed                      (1 + tx)
  uint64_t* bar_x_free = bars + kStages;        // [kStages] the products that read it retired   (commit)
  uint64_t* bar_w = bars + 2 * kStages;         // [1] weights landed                            (1 + tx)
  uint64_t* bar_acc_ready = bars + 2 * kStages + 1;   // [2] products of the tile retired         (commit)
  uint64_t* bar_acc_free = bars + 2 * kStages + 3;    // [2] the epilogue has read the accumulator (128)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar_full_x[i], 1);
      mbar_init(&bar_x_free[i], 1);
    }
    mbar_init(bar_w, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_acc_ready[i], 1);
      mbar_init(&bar_acc_free[i], 128);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int j = tid; j < kN; j += kThreads) s_bias[j] = bias != nullptr ? bias[j] : 0.0f;
  if (warp == kIssuerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  auto x_stage = [&](int n) { return smem + kOffX + (n % kStages) * kBlockBytes; };

#define GRMX_WAIT(bar, phase)                                        \
  if (!mbar_wait((bar), static_cast<uint32_t>(phase) & 1u, s_abort)) \
    break;

  if (warp == kLoaderWarp) {
    if ((tid & 31) == 0) {
      mbar_expect_tx(bar_w, static_cast<uint32_t>(d_blocks) * kBlockBytes);
      for (int kb = 0; kb < d_blocks; ++kb) tma_load_3d(smem + kOffW + kb * kBlockBytes, &map_w, bar_w, kb * 64, 0, 0);
      int n = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < d_blocks; ++kb, ++n) {
          ok = false;
          do {
            if (n >= kStages) GRMX_WAIT(&bar_x_free[n % kStages], n / kStages - 1)
            mbar_expect_tx(&bar_full_x[n % kStages], kBlockBytes);
            tma_load_3d(x_stage(n), &map_x, &bar_full_x[n % kStages], kb * 64, tile * kTile, 0);
            ok = true;
          } while (false);
          if (!ok) break;
        }
      }
      if (*s_abort) {
        mbar_wait_quiet(bar_w, 0);
        for (int j = n > kStages ? n - kStages : 0; j < n; ++j) mbar_wait_quiet(&bar_full_x[j % kStages], (j / kStages) & 1);
      }
    }
  } else if (warp == kIssuerWarp) {
    if ((tid & 31) == 0) {
      constexpr uint32_t idesc = make_idesc(kTile, kN, 0, 0);
      int n = 0, it = 0;
      bool ok = mbar_wait(bar_w, 0, s_abort);
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        ok = false;
        do {
          if (it >= 2) GRMX_WAIT(&bar_acc_free[it & 1], it / 2 - 1)
          ok = true;
        } while (false);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(kN) * (it & 1);
        for (int kb = 0; kb < d_blocks && ok; ++kb, ++n) {
          ok = false;
          do {
            GRMX_WAIT(&bar_full_x[n % kStages], n / kStages)
            tc_fence_after();
            const uint64_t da = smem_desc(smem_u32(x_stage(n)), 16, 1024);
            const uint64_t db = smem_desc(smem_u32(smem + kOffW + kb * kBlockBytes), 16, 1024);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              tc_mma_bf16(acc, desc_add(da, kk * 32), desc_add(db, kk * 32), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            tc_commit(&bar_x_free[n % kStages]);
            ok = true;
          } while (false);
        }
        if (!ok) break;
        tc_commit(&bar_acc_ready[it & 1]);
      }
    }
  } else {
    // ===================================================================== epilogue (thread = row)
    const int row = tid;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      GRMX_WAIT(&bar_acc_ready[it & 1], it / 2)
      tc_fence_after();
      const int64_t r = static_cast<int64_t>(tile) * kTile + row;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t v[kGroup];
        tc_ld32_async(lane_addr + kN * (it & 1) + kGroup * g, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tc_ld32_async(lane_addr + kN * (it & 1) + kGroup * g + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tc_wait_ld();
        if (g == 1) {
          tc_fence_before();
          mbar_arrive(&bar_acc_free[it & 1]);          // both groups are in registers
        }
        float sq = 0.0f;
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
          const float y = __uint_as_float(v[j]) + s_bias[kGroup * g + j];
          v[j] = __float_as_uint(y);
          sq = fmaf(y, y, sq);
        }
        const float scale = 1.0f / fmaxf(sqrtf(sq), eps);      // F.normalize: x / max(||x||, eps)
        if (r < rows) {
          uint4* dst = reinterpret_cast<uint4*>((g == 0 ? out_a : out_b) + r * kGroup);
#pragma unroll
          for (int j = 0; j < kGroup / 8; ++j) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[8 * j]) * scale, __uint_as_float(v[8 * j + 1]) * scale);
            w.y = pack_bf16(__uint_as_float(v[8 * j + 2]) * scale, __uint_as_float(v[8 * j + 3]) * scale);
            w.z = pack_bf16(__uint_as_float(v[8 * j + 4]) * scale, __uint_as_float(v[8 * j + 5]) * scale);
            w.w = pack_bf16(__uint_as_float(v[8 * j + 6]) * scale, __uint_as_float(v[8 * j + 7]) * scale);
            dst[j] = w;
          }
        }
      }
    }
  }
#undef GRMX_WAIT

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *s_abort && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
  if (warp == kIssuerWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

}  // namespace
}  // namespace grmx

extern "C" int grmx_project_normalize(const void* x_bf16, const void* weights_bf16, const float* bias, void* out_a_bf16,
                                      void* out_b_bf16, int64_t rows, int64_t D, int64_t K, float eps, void* stream) {
  using namespace grmx;
  const char* who = "grmx_project_normalize";
  GRMX_REQUIRE(rows >= 0 && D > 0 && K > 0, "%s: bad sizes", who);
  if (K != kGroup || D % 64 != 0 || D > kMaxD) {
    return fail(GRMX_ERR_UNSUPPORTED, "%s: covers two projections of width 64 from D a multiple of 64 up to 512", who);
  }
  if (rows == 0) return GRMX_OK;
  GRMX_REQUIRE(x_bf16 && weights_bf16 && out_a_bf16 && out_b_bf16, "%s: NULL tensor pointer", who);
  const uintptr_t align = reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(weights_bf16) |
                          reinterpret_cast<uintptr_t>(out_a_bf16) | reinterpret_cast<uintptr_t>(out_b_bf16);
  GRMX_REQUIRE((align & 15u) == 0, "%s: tensors must be 16-byte aligned", who);
  GRMX_REQUIRE(rows <= 0x7fff0000LL, "%s: too many rows for the tensor map", who);
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
      attr_status = cudaFuncSetAttribute(project_normalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
      cudaDeviceGetAttribute(&sm_count[device], cudaDevAttrMultiProcessorCount, device);
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "%s: cannot reserve %d bytes of shared memory: %s", who, kSmemAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_x, map_w;
  if (!tc::make_token_map(&map_x, x_bf16, 1, rows, D) || !tc::make_token_map(&map_w, weights_bf16, 1, 2 * K, D)) {
    return fail(GRMX_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed", who);
  }
  const int64_t n_tiles = (rows + kTile - 1) / kTile;
  GRMX_REQUIRE(n_tiles <= 0x7fffffffLL, "%s: too many tiles", who);
  const int sms = device >= 0 && device < 64 && sm_count[device] > 0 ? sm_count[device] : 148;
  const unsigned grid = static_cast<unsigned>(n_tiles < sms ? n_tiles : sms);
  project_normalize_kernel<<<grid, kThreads, kSmemAlloc, static_cast<cudaStream_t>(stream)>>>(
      map_x, map_w, bias, static_cast<__nv_bfloat16*>(out_a_bf16), static_cast<__nv_bfloat16*>(out_b_bf16), rows,
      static_cast<int>(D / 64), static_cast<int>(n_tiles), eps, device_error_word_ptr());
  return check_launch("project_normalize");
}
