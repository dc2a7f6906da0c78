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

#include <mutex>

#include "scan.cuh"

namespace grmx {
namespace {

constexpr int kChunk = 128;     // tokens per chunk == MMA M for the token-row products
constexpr int kThreads = 128;   // one warpgroup: thread t <-> TMEM lane t
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;      // S, later O1   (128 columns)
constexpr uint32_t kColO2 = 128;   // O2            (d_v columns)
constexpr uint32_t kColM = 256;    // state         (d_k columns, d_v lanes)
constexpr uint32_t kWaitLimit = 1u << 22;

// ---------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the
// barrier did not flip within the limit or another thread already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Bounded wait that ignores the abort flag: used on the way out to let copies land.
__device__ __forceinline__ bool mbar_wait_quiet(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
      "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
      "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
      "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
      "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
      "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
      "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
      "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- shared-memory matrix descriptors (sm_100 format, 128-byte swizzle) ----
// bits [0,14) start address >> 4; [16,30) leading byte offset >> 4; [32,46) stride byte
// offset >> 4; [46,48) version = 1; [61,64) layout type, 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B.
// bits [4,6) D format (1 = f32); [7,10) A format (1 = bf16); [10,13) B format;
// [15] A major (1 = MN); [16] B major; [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

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

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

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
bool make_map(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t D) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(T) * D * 2};
  const cuuint32_t box[3] = {64, kChunk, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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
  if (!make_map(&map_q, p.queries, p.B, p.T, K) || !make_map(&map_k, p.keys, p.B, p.T, K) ||
      !make_map(&map_v, p.values, p.B, p.T, V)) {
    return fail(GRMX_ERR_LAUNCH, "tcgen05 scan: cuTensorMapEncodeTiled failed");
  }
  linear_scan_tc_kernel<K, V><<<static_cast<unsigned>(p.B), kThreads, Plan::kAlloc, stream>>>(
      map_q, map_k, map_v, p, device_error_word_ptr());
  return check_launch("linear_scan_tcgen05");
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

}  // namespace

bool scan_tcgen05_supported(const ScanParams& p, int io_dtype, int state_dtype, const char** why) {
  if (io_dtype != GRMX_BF16 || state_dtype != GRMX_F32) {
    *why = "needs bf16 tokens and an fp32 state";
    return false;
  }
  if (!(p.K == 64 && p.H == 64)) {
    *why = "d_k and d_v must both be 64";
    return false;
  }
  if (p.T < kChunk || p.T % kChunk != 0) {
    *why = "T must be a positive multiple of 128";
    return false;
  }
  if (p.reverse || p.first_step_no_decay) {
    *why = "reverse scans and decay-free first steps run on the fp32 path";
    return false;
  }
  if (p.B > 0x7fffffffLL || p.T > 0x7fffffffLL) {
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

int launch_scan_tcgen05(const ScanParams& p, cudaStream_t stream) {
  if (p.K == 64 && p.H == 64) return launch<64, 64>(p, stream);
  return fail(GRMX_ERR_UNSUPPORTED, "tcgen05 scan: no kernel for d_k=%lld d_v=%lld", (long long)p.K,
              (long long)p.H);
}

}  // namespace grmx
