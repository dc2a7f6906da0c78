// tcgen05 kernel of the linear-memory scan: bf16 operands, fp32 state in TMEM.
//
// One CTA owns one batch row for the whole call and walks it in chunks of
// C = 128 tokens.  Per chunk, with Q, Kc, Vc the chunk's [C x d] tiles (TMA,
// 128-byte swizzle) and M the carried state [d_v x d_k]:
//
//   (1) S   = Q Kc^T                       M=128 N=128   K-major x K-major
//   (3) O2  = Q Mb^T          Mb = bf16(M) M=128 N=d_v   K-major x K-major
//   (4) M   = decay^C M + Vw^T Kc          M=d_v N=d_k   MN-major x MN-major
//             Vw_j = coeff * decay^(C-1-j) v_j   (scaled copy of Vc, bf16)
//   (2) O1  = P Vc,  P_ij = coeff * decay^(i-j) S_ij (j <= i)   K-major x MN-major
//   out_i   = hidden_scale * (O1_i + decay^(i+1) O2_i)
//
// which is the closed form of the reference's chunk (grm/core/cuda_ops.py:
// 218-254) with the state carried in TMEM between chunks.  All four products
// are tcgen05.mma (kind::f16, fp32 accumulate) issued by one thread; the
// accumulators live in TMEM (S/O1 share columns, O2 and the state have their
// own) and are read back with tcgen05.ld by the four warps, one TMEM lane
// (= one token row, or one state row) per thread.
//
// Every wait on an mbarrier is bounded: when the limit is hit the kernel sets
// bit 1 of the device error word, stops issuing work, frees its TMEM and
// returns, so a logic error cannot hang the device.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "scan.cuh"
#include "tc_ptx.cuh"

namespace grmx {
namespace tc {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    } else {
      cudaGetLastError();
    }
  });
  return fn;
}

// [B, T, D] bf16 tensor, box = 64 features x 128 tokens x 1 row, 128-byte swizzle
namespace {

// Encoding a tensor map is a driver call of a few microseconds, and a scan needs four of them;
// callers that run the same buffers again and again (a segment loop, a serving step) would pay
// that on every call.  The last few encodings are kept per thread, keyed by everything that
// goes into them.
struct MapKey {
  const void* base;
  int64_t B, T, D;
  int kind;   // 0: load map (64 x 128 box, 128-byte swizzle), 1: store map (32 x 128 box, 64-byte swizzle)
  bool operator==(const MapKey& o) const {
    return base == o.base && B == o.B && T == o.T && D == o.D && kind == o.kind;
  }
};
constexpr int kMapCacheSlots = 16;
struct MapCache {
  MapKey keys[kMapCacheSlots];
  CUtensorMap maps[kMapCacheSlots];
  int used = 0;
  int next = 0;
};

bool encode_token_map(CUtensorMap* map, const MapKey& key) {
  thread_local MapCache cache;
  for (int i = 0; i < cache.used; ++i) {
    if (cache.keys[i] == key) {
      *map = cache.maps[i];
      return true;
    }
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(key.D), static_cast<cuuint64_t>(key.T),
                              static_cast<cuuint64_t>(key.B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(key.D) * 2, static_cast<cuuint64_t>(key.T) * key.D * 2};
  const cuuint32_t box[3] = {key.kind == 0 ? 64u : 32u, 128, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const bool ok =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(key.base), dims, strides, box, elem_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, key.kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
             key.kind == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  if (ok) {
    const int slot = cache.next;
    cache.keys[slot] = key;
    cache.maps[slot] = *map;
    cache.next = (slot + 1) % kMapCacheSlots;
    if (cache.used < kMapCacheSlots) ++cache.used;
  }
  return ok;
}

}  // namespace

bool make_token_map(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t D) {
  return encode_token_map(map, MapKey{base, B, T, D, 0});
}

bool make_token_half_map(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t D) {
  return encode_token_map(map, MapKey{base, B, T, D, 1});
}

namespace {

// Four warps wait on a barrier that nothing completes.  The first to run out of polls raises the
// abort flag, the others see it at their next check, and the CTA reports through the error word.
__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(uint32_t limit, uint32_t* error_word) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  mbar_wait(&bar, 0, &abort_flag, limit);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
}

}  // namespace

int launch_bounded_wait_selftest(uint32_t limit, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 128, 0, stream>>>(limit, device_error_word_ptr());
  return check_launch("bounded_wait_selftest");
}

bool device_is_sm100() {
  static int cached[64] = {0};   // 0 unknown, 1 yes, 2 no
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return false;
  if (cached[device] == 0) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    cached[device] = major == 10 ? 1 : 2;
  }
  return cached[device] == 1;
}

}  // namespace tc

namespace {

using namespace tc;

constexpr int kChunk = 128;     // tokens per chunk == MMA M for the token-row products
constexpr int kThreads = 128;   // one warpgroup: thread t <-> TMEM lane t
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;      // S, later O1   (128 columns)
constexpr uint32_t kColO2 = 128;   // O2            (d_v columns)
constexpr uint32_t kColM = 256;    // state         (d_k columns, d_v lanes)

// ---------------------------------------------------------------- shared memory plan

template <int K, int V>
struct SmemPlan {
  static constexpr int kQBytes = kChunk * K * 2;
  static constexpr int kVBytes = kChunk * V * 2;
  static constexpr int kStageBytes = 2 * kQBytes + kVBytes;
  static constexpr int kPBytes = kChunk * kChunk * 2;
  static constexpr int kMbBytes = V * K * 2;
  static constexpr int kOffStage = 0;
  static constexpr int kOffP = kStages * kStageBytes;
  static constexpr int kOffVw = kOffP + kPBytes;
  static constexpr int kOffMbHi = kOffVw + kVBytes;
  static constexpr int kOffMbLo = kOffMbHi + kMbBytes;
  static constexpr int kOffPow = kOffMbLo + kMbBytes;                 // float[kChunk + 2]
  static constexpr int kOffBars = kOffPow + (kChunk + 8) * 4;         // mbarriers, 8 bytes each
  static constexpr int kOffMisc = kOffBars + 8 * 8;
  static constexpr int kTotal = kOffMisc + 64;
  static constexpr int kAlloc = kTotal + 1024;                         // slack for 1024-byte alignment
};

// ---------------------------------------------------------------- kernel

template <int K, int V>
__global__ void __launch_bounds__(kThreads, 1)
linear_scan_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, ScanParams p, uint32_t* error_word) {
  using Plan = SmemPlan<K, V>;
  static_assert(K == 64 || K == 128, "d_k must be 64 or 128");
  static_assert(V == 64 || V == 128, "d_v must be 64 or 128");
  constexpr int KB = K / 64;   // 64-wide blocks along d_k
  constexpr int VB = V / 64;   // 64-wide blocks along d_v
  constexpr uint32_t kBlockBytes = kChunk * 128;   // one [128 rows x 128 B] swizzled block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_pow = reinterpret_cast<float*>(smem + Plan::kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::kOffBars);
  uint64_t* bar_full = bars;          // [kStages]
  uint64_t* bar_a = bars + kStages;   // products (1),(3),(4) done
  uint64_t* bar_b = bars + kStages + 1;  // product (2) done
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + Plan::kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + Plan::kOffMisc + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int64_t b = blockIdx.x;
  const int n_chunks = static_cast<int>(p.T / kChunk);

  // ---- set-up ----
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&bar_full[s], 1);
    mbar_init(bar_a, 1);
    mbar_init(bar_b, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int j = tid; j <= kChunk; j += kThreads) s_pow[j] = powf(p.decay, static_cast<float>(j));
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  auto stage_q = [&](int s) { return smem + Plan::kOffStage + s * Plan::kStageBytes; };
  auto stage_k = [&](int s) { return stage_q(s) + Plan::kQBytes; };
  auto stage_v = [&](int s) { return stage_k(s) + Plan::kQBytes; };
  uint8_t* s_p = smem + Plan::kOffP;
  uint8_t* s_vw = smem + Plan::kOffVw;
  uint8_t* s_mb = smem + Plan::kOffMbHi;

  auto issue_loads = [&](int chunk) {
    const int s = chunk % kStages;
    mbar_expect_tx(&bar_full[s], Plan::kStageBytes);
    const int t0 = chunk * kChunk;
    for (int kb = 0; kb < KB; ++kb) {
      tma_load_3d(stage_q(s) + kb * kBlockBytes, &map_q, &bar_full[s], kb * 64, t0, static_cast<int>(b));
      tma_load_3d(stage_k(s) + kb * kBlockBytes, &map_k, &bar_full[s], kb * 64, t0, static_cast<int>(b));
    }
    for (int vb = 0; vb < VB; ++vb) {
      tma_load_3d(stage_v(s) + vb * kBlockBytes, &map_v, &bar_full[s], vb * 64, t0, static_cast<int>(b));
    }
  };
  int loads_issued = 0;   // thread 0 only: chunks whose TMA loads were started / seen complete
  int loads_landed = 0;
  if (tid == 0) {
    issue_loads(0);
    loads_issued = 1;
  }

  // State row owned by this thread: for d_v = 128 TMEM lane t is row t; for d_v = 64 the
  // M = 64 accumulator occupies lanes 0-15 of each 32-lane quarter (row = 16*warp + lane).
  const bool owns_row = (V == 128) || (lane < 16);
  const int state_row = (V == 128) ? tid : (warp * 16 + (lane & 15));

  // initial state -> TMEM (pre-scaled by the first chunk's carry) and bf16 copy for product (3)
  {
    const float* m_in = static_cast<const float*>(p.memory_in) + b * V * K;
    const float carry = s_pow[kChunk];
#pragma unroll 1
    for (int c0 = 0; c0 < K; c0 += 32) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = owns_row ? m_in[state_row * p.m_row_stride + (c0 + j) * p.m_col_stride] : 0.0f;
      }
      if (owns_row) {
        uint8_t* row = s_mb + (c0 / 64) * (V * 128) + state_row * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk16 = ((c0 % 64) / 8 + ch) ^ (state_row & 7);
          uint4 w;
          w.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
          w.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
          w.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
          w.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
          *reinterpret_cast<uint4*>(row + chunk16 * 16) = w;
        }
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= carry;
      tc_st32(tmem_lane + kColM + c0, v);
    }
  }

  constexpr uint32_t idesc_s = make_idesc(kChunk, kChunk, 0, 0);
  constexpr uint32_t idesc_o2 = make_idesc(kChunk, V, 0, 0);
  constexpr uint32_t idesc_m = make_idesc(V, K, 1, 1);
  constexpr uint32_t idesc_o1 = make_idesc(kChunk, V, 0, 1);

  bool ok = true;
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    const int s = chunk % kStages;
    if (tid == 0 && chunk + 1 < n_chunks) {
      issue_loads(chunk + 1);
      loads_issued = chunk + 2;
    }
    if (mbar_wait(&bar_full[s], (chunk / kStages) & 1, s_abort)) {
      loads_landed = chunk + 1;
    } else {
      ok = false;
    }

    // ---- Vw: token row `tid` of Vc scaled by coeff * decay^(C-1-tid) ----
    {
      const float w = p.update_coeff * s_pow[kChunk - 1 - tid];
#pragma unroll
      for (int vb = 0; vb < VB; ++vb) {
        const uint8_t* src = stage_v(s) + vb * kBlockBytes + tid * 128;
        uint8_t* dst = s_vw + vb * kBlockBytes + tid * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int ch = (i + tid) & 7;   // rotate so that 8 neighbouring threads hit 8 bank groups
          uint4 raw = *reinterpret_cast<const uint4*>(src + ch * 16);
          uint32_t* words = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = __uint_as_float(words[j] << 16) * w;
            const float hi = __uint_as_float(words[j] & 0xffff0000u) * w;
            words[j] = pack_bf16(lo, hi);
          }
          *reinterpret_cast<uint4*>(dst + ch * 16) = raw;
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) break;

    if (tid == 0) {
      tc_fence_after();
      // (1) S = Q Kc^T
#pragma unroll
      for (int kk = 0; kk < K / 16; ++kk) {
        const uint32_t off = (kk / 4) * kBlockBytes + (kk % 4) * 32;
        tc_mma_bf16(tmem_base + kColS, smem_desc(smem_u32(stage_q(s)) + off, 16, 1024),
                    smem_desc(smem_u32(stage_k(s)) + off, 16, 1024), idesc_s, kk > 0);
      }
      // (3) O2 = Q Mb^T
#pragma unroll
      for (int kk = 0; kk < K / 16; ++kk) {
        const uint32_t off_q = (kk / 4) * kBlockBytes + (kk % 4) * 32;
        const uint32_t off_m = (kk / 4) * (V * 128) + (kk % 4) * 32;
        tc_mma_bf16(tmem_base + kColO2, smem_desc(smem_u32(stage_q(s)) + off_q, 16, 1024),
                    smem_desc(smem_u32(s_mb) + off_m, 16, 1024), idesc_o2, kk > 0);
      }
      // (4) M += Vw^T Kc   (both operands MN-major: 8-token groups are 1024 B apart)
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        const uint32_t off = kk * 2048;
        tc_mma_bf16(tmem_base + kColM, smem_desc(smem_u32(s_vw) + off, kBlockBytes, 1024),
                    smem_desc(smem_u32(stage_k(s)) + off, kBlockBytes, 1024), idesc_m, 1u);
      }
      tc_commit(bar_a);
    }
    ok = mbar_wait(bar_a, chunk & 1, s_abort) && ok;
    tc_fence_after();

    // ---- S -> P (bf16, decay mask), row `tid` ----
#pragma unroll 1
    for (int c0 = 0; c0 < kChunk; c0 += 32) {
      float v[32];
      tc_ld32(tmem_lane + kColS + c0, v);
      uint8_t* row = s_p + (c0 / 64) * kBlockBytes + tid * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int col = c0 + ch * 8 + j;
          const int d = tid - col;
          x[j] = d >= 0 ? v[ch * 8 + j] * p.update_coeff * s_pow[d] : 0.0f;
        }
        uint4 w;
        w.x = pack_bf16(x[0], x[1]);
        w.y = pack_bf16(x[2], x[3]);
        w.z = pack_bf16(x[4], x[5]);
        w.w = pack_bf16(x[6], x[7]);
        const int chunk16 = ((c0 % 64) / 8 + ch) ^ (tid & 7);
        *reinterpret_cast<uint4*>(row + chunk16 * 16) = w;
      }
    }

    // ---- state: M_c is complete; refresh the bf16 copy, emit on the last chunk, rescale ----
    {
      const bool last = chunk + 1 == n_chunks;
      const float carry = s_pow[kChunk];
      float* m_out = p.memory_out != nullptr ? static_cast<float*>(p.memory_out) + b * V * K : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < K; c0 += 32) {
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
              *reinterpret_cast<float4*>(m_out + state_row * K + c0 + j) = o;
            }
          }
        } else {
          if (owns_row) {
            uint8_t* row = s_mb + (c0 / 64) * (V * 128) + state_row * 128;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              const int chunk16 = ((c0 % 64) / 8 + ch) ^ (state_row & 7);
              uint4 w;
              w.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
              w.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
              w.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
              w.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
              *reinterpret_cast<uint4*>(row + chunk16 * 16) = w;
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= carry;
          tc_st32(tmem_lane + kColM + c0, v);
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (*s_abort) break;

    if (tid == 0) {
      tc_fence_after();
      // (2) O1 = P Vc  (overwrites the S columns)
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        const uint32_t off_p = (kk / 4) * kBlockBytes + (kk % 4) * 32;
        tc_mma_bf16(tmem_base + kColS, smem_desc(smem_u32(s_p) + off_p, 16, 1024),
                    smem_desc(smem_u32(stage_v(s)) + kk * 2048, kBlockBytes, 1024), idesc_o1, kk > 0);
      }
      tc_commit(bar_b);
    }
    ok = mbar_wait(bar_b, chunk & 1, s_abort) && ok;
    tc_fence_after();

    // ---- out row = hidden_scale * (O1 + decay^(tid+1) O2) ----
    {
      const float carry_row = s_pow[tid + 1];
      __nv_bfloat16* out =
          static_cast<__nv_bfloat16*>(p.hidden_out) + (b * p.T + static_cast<int64_t>(chunk) * kChunk + tid) * V;
#pragma unroll 1
      for (int c0 = 0; c0 < V; c0 += 32) {
        float o1[32], o2[32];
        tc_ld32(tmem_lane + kColS + c0, o1);
        tc_ld32(tmem_lane + kColO2 + c0, o2);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            x[j] = p.hidden_scale * fmaf(carry_row, o2[ch * 8 + j], o1[ch * 8 + j]);
          }
          uint4 w;
          w.x = pack_bf16(x[0], x[1]);
          w.y = pack_bf16(x[2], x[3]);
          w.z = pack_bf16(x[4], x[5]);
          w.w = pack_bf16(x[6], x[7]);
          *reinterpret_cast<uint4*>(out + c0 + ch * 8) = w;
        }
      }
    }
    // the TMEM reads above are ordered before the next chunk's MMAs by the
    // fence + barrier that follow the Vw pass at the top of the loop
  }

  if (!ok || *s_abort) {
    if (tid == 0) {
      if (error_word != nullptr) atomicOr(error_word, kErrBoundedWait);
      // let the copies still in flight land before the shared memory is released
      for (int c = loads_landed; c < loads_issued; ++c) {
        mbar_wait_quiet(&bar_full[c % kStages], (c / kStages) & 1);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------- host side

template <int K, int V>
int launch(const ScanParams& p, cudaStream_t stream) {
  using Plan = SmemPlan<K, V>;
  // the attribute is per device: set it on first use of each one
  static std::mutex mutex;
  static bool configured[64] = {false};
  int device = 0;
  cudaGetDevice(&device);
  cudaError_t attr_status = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device >= 0 && device < 64 && !configured[device]) {
      attr_status = cudaFuncSetAttribute(linear_scan_tc_kernel<K, V>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kAlloc);
      configured[device] = attr_status == cudaSuccess;
    }
  }
  if (attr_status != cudaSuccess) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cannot reserve %d bytes of shared memory: %s", Plan::kAlloc,
                cudaGetErrorString(attr_status));
  }
  CUtensorMap map_q, map_k, map_v;
  if (!make_token_map(&map_q, p.queries, p.B, p.T, K) || !make_token_map(&map_k, p.keys, p.B, p.T, K) ||
      !make_token_map(&map_v, p.values, p.B, p.T, V)) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cuTensorMapEncodeTiled failed");
  }
  linear_scan_tc_kernel<K, V><<<static_cast<unsigned>(p.B), kThreads, Plan::kAlloc, stream>>>(
      map_q, map_k, map_v, p, device_error_word_ptr());
  return check_launch("linear_scan_tcgen05");
}

}  // namespace

bool scan_tcgen05_supported(const ScanParams& p, int io_dtype, int state_dtype, const char** why) {
  if (io_dtype != GRMX_BF16 || state_dtype != GRMX_F32) {
    *why = "needs bf16 tokens and an fp32 state";
    return false;
  }
  if (!scan_tcgen05_pipe_supported(p)) {
    *why = "d_k and d_v must be multiples of 64 (d_k <= 1024, d_v <= 4096)";
    return false;
  }
  // the pipelined kernel takes any T, either direction; the single-warpgroup one only whole chunks
  if (p.T < 1) {
    *why = "no tokens";
    return false;
  }
  if (p.B > 0x7fffffffLL || p.T > 0x7fff0000LL) {
    *why = "B or T exceeds the tensor-map coordinate range";
    return false;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(p.keys) | reinterpret_cast<uintptr_t>(p.values) |
                          reinterpret_cast<uintptr_t>(p.queries) | reinterpret_cast<uintptr_t>(p.hidden_out) |
                          reinterpret_cast<uintptr_t>(p.memory_out);
  if (align & 15u) {
    *why = "tensors must be 16-byte aligned";
    return false;
  }
  if (!device_is_sm100()) {
    *why = "the current device is not sm_100";
    return false;
  }
  if (encode_tiled_fn() == nullptr) {
    *why = "cuTensorMapEncodeTiled is unavailable";
    return false;
  }
  *why = "";
  return true;
}

// GRMX_TC_VARIANT=sync selects the single-warpgroup kernel (kept for comparison and as the
// template for other head sizes); anything else uses the pipelined one where it applies.
static bool prefer_sync_variant() {
  static const bool value = [] {
    const char* env = getenv("GRMX_TC_VARIANT");
    return env != nullptr && strcmp(env, "sync") == 0;
  }();
  return value;
}

int launch_scan_tcgen05(const ScanParams& p, cudaStream_t stream) {
  const bool simple = p.K == 64 && p.H == 64 && p.T % kChunk == 0 && !p.reverse && !p.first_step_no_decay;
  if (scan_tcgen05_pipe_supported(p) && !(simple && prefer_sync_variant())) {
    return launch_scan_tcgen05_selfcut(p, stream);
  }
  if (p.K == 64 && p.H == 64) return launch<64, 64>(p, stream);
  return fail(GRMX_ERR_UNSUPPORTED, "tcgen05 scan: no kernel for d_k=%lld d_v=%lld", (long long)p.K,
              (long long)p.H);
}

}  // namespace grmx
