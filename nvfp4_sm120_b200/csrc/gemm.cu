// Block-scaled NVFP4 GEMM for B200 (sm_100a): D[M,N] = (A.sfA)(B.sfB)^T * ptsA * ptsB.
//
// tcgen05.mma kind::mxf4nvf4 with 1x16 E4M3 block scales (scale_vec::4X), fp32 accumulators in
// tensor memory.  Per CTA: one 128 x 256 output tile; K is walked in slices of 256 elements
// (= one 128-byte swizzled row per operand row).  Warp roles:
//   warp 0      TMA producer: A and B slices by tensor-map copies into 128B-swizzled shared
//               memory, the matching scale-factor tiles by plain bulk copies (the 128x4-tiled
//               scale layout makes the scales of one slice contiguous per 128 rows)
//   warp 1      allocates tensor memory and issues the MMAs (one elected lane)
//   warps 2..5  during the main loop: move the scale factors of each landed stage from shared
//               memory to tensor memory through registers (tcgen05.st; measured here, the
//               tcgen05.cp route costs ~110 cycles per 512-byte tile and serialises with the MMAs);
//               afterwards the epilogue: tcgen05.ld the accumulators, multiply by ptsA*ptsB,
//               store bf16/fp32
// All waits are bounded: a wait that gives up writes a code to *status, raises a CTA-wide abort
// flag, and the kernel drains and frees its tensor memory before returning.
#include <cuda.h>
#include "common.cuh"
#include "nvfp4_b200.h"

namespace nvfp4 {
namespace gemm {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 256;                 // elements per K slice = 128 bytes per row
constexpr int kStages = 4;
constexpr int kABytes = kTileM * 128;       // 16 KiB
constexpr int kBBytes = kTileN * 128;       // 32 KiB
constexpr int kSfaBytes = 4 * 512;          // 128 rows x 16 scales
constexpr int kSfbBytes = 2 * 4 * 512;      // 256 rows x 16 scales
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 55296
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;                  // row tiles per rasterization group
constexpr int kSfColsPerStage = 16 + 32;    // SFA 4 columns per K=64 block, SFB 8
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // a wait that lasts 2 s gives up

enum : int { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3 };

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up (or another thread already raised the abort flag).
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 consecutive 32-bit columns of this warp's 32 TMEM lanes, from registers
__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand rows of 128 bytes with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::mxf4nvf4: A/B format E2M1 (code 1), E4M3 scales (0), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24, dense K = 64.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Params {
  const uint8_t* a_sf;
  const uint8_t* b_sf;
  const float* a_pts;
  const float* b_pts;
  void* d;
  int64_t M, N, K, ldd;
  int out_f32;
  int32_t* status;
};

__device__ __forceinline__ void raise(volatile int* abort_flag, int32_t* status, int code) {
  *abort_flag = 1;
  if (status != nullptr) atomicCAS(status, 0, code);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                 // 1024-byte alignment for the swizzle
  uint8_t* smem = smem_raw + (base - raw);
  // layout: [stage][A | B | SFA | SFB] ... then barriers
  const uint32_t bar_base = base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                  // TMA landed
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };      // MMAs have read the stage
  auto sf_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };     // scale factors are in TMEM
  const uint32_t acc_bar = bar_base + 8u * (3 * kStages);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kStages * kStageBytes + 8 * (3 * kStages + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kStages * kStageBytes + 8 * (3 * kStages + 1) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grouped rasterization: consecutive CTAs walk kGroupM row tiles before the next column tile, so
  // that one wave of CTAs touches a near-square patch of A and B (both stay L2 resident)
  const uint32_t tiles_n = (uint32_t)((p.N + kTileN - 1) / kTileN), tiles_m = (uint32_t)((p.M + kTileM - 1) / kTileM);
  const uint32_t per_group = kGroupM * tiles_n;
  const uint32_t group = blockIdx.x / per_group, first_m = group * kGroupM;
  const uint32_t gsize = min((uint32_t)kGroupM, tiles_m - first_m);
  const uint32_t in_group = blockIdx.x - group * per_group;
  const int64_t m0 = (int64_t)(first_m + in_group % gsize) * kTileM, n0 = (int64_t)(in_group / gsize) * kTileN;
  const int num_kt = (int)((p.K + kTileK - 1) / kTileK);
  const int64_t sf_col_tiles = (p.K / 16 + 3) / 4;               // 512-byte tiles per 128-row group

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(sf_bar(s), 4); }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf0 = tmem_base + kTileN;                  // scale factors behind the accumulator

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const bool second_sfb = (n0 + 128) < p.N;                  // rows 128..255 of the B tile exist
      int issued = 0;
      for (int kt = 0; kt < num_kt; ++kt) {
        const int s = kt % kStages;
        if (kt >= kStages && !mbar_wait(empty_bar(s), ((kt / kStages) - 1) & 1, abort_flag)) {
          raise(abort_flag, p.status, kErrProducerWait);
          break;
        }
        const int64_t k_left = p.K - (int64_t)kt * kTileK;
        const int nkb = k_left >= kTileK ? 4 : (int)((k_left + 63) / 64);
        const uint32_t sf_bytes = (uint32_t)nkb * 512u;
        const uint32_t stage = base + s * kStageBytes;
        mbar_expect_tx(full_bar(s), kABytes + kBBytes + sf_bytes * (second_sfb ? 3u : 2u));
        tma_load_2d(stage, &map_a, kt * 128, (int)m0, full_bar(s));
        tma_load_2d(stage + kABytes, &map_b, kt * 128, (int)n0, full_bar(s));
        const uint8_t* sfa = p.a_sf + ((m0 >> 7) * sf_col_tiles + (int64_t)kt * 4) * 512;
        const uint8_t* sfb = p.b_sf + ((n0 >> 7) * sf_col_tiles + (int64_t)kt * 4) * 512;
        bulk_load(stage + kABytes + kBBytes, sfa, sf_bytes, full_bar(s));
        bulk_load(stage + kABytes + kBBytes + kSfaBytes, sfb, sf_bytes, full_bar(s));
        if (second_sfb)
          bulk_load(stage + kABytes + kBBytes + kSfaBytes + 2048, sfb + sf_col_tiles * 512, sf_bytes, full_bar(s));
        ++issued;
      }
      if (*abort_flag != 0) {
        // give copies already in flight a bounded chance to land before shared memory goes away
        const int first = issued > kStages ? issued - kStages : 0;
        for (int kt = first; kt < issued; ++kt)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(full_bar(kt % kStages), (kt / kStages) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kTileM, kTileN);
      bool ok = true;
      for (int kt = 0; kt < num_kt && ok; ++kt) {
        const int s = kt % kStages;
        if (!mbar_wait(sf_bar(s), (kt / kStages) & 1, abort_flag)) {     // implies the TMA data landed
          raise(abort_flag, p.status, kErrMmaWait);
          ok = false;
          break;
        }
        tc_fence_after();
        const int64_t k_left = p.K - (int64_t)kt * kTileK;
        const int nkb = k_left >= kTileK ? 4 : (int)((k_left + 63) / 64);
        const uint32_t stage = base + s * kStageBytes;
        const uint32_t t_sfa = tmem_sf0 + s * kSfColsPerStage, t_sfb = t_sfa + 16;
        const uint64_t da = make_desc_sw128(stage), db = make_desc_sw128(stage + kABytes);
        for (int kb = 0; kb < nkb; ++kb) {
          // 64 elements = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
          tc_mma_nvf4(tmem_base, da + 2u * kb, db + 2u * kb, idesc, t_sfa + 4 * kb, t_sfb + 8 * kb,
                      (kt > 0 || kb > 0) ? 1u : 0u);
        }
        tc_commit(empty_bar(s));          // frees the stage once these MMAs have read it
      }
      if (ok) tc_commit(acc_bar);         // accumulator complete
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;                                   // TMEM lanes 32*quad .. +31
    bool ok = true;
    // During the main loop these four warps move the scale factors of every landed stage from
    // shared memory into tensor memory.  The MMA wants, in every 32-lane quarter, lane l / 32-bit
    // column c of a K=64 block to hold the four E4M3 scales of row 32c + l: exactly 16 bytes per
    // lane of the 512-byte tile the quantizer wrote, so one 128-bit shared load per tile and lane
    // feeds four columns, and each warp writes the copy of its own quarter (tcgen05.st).
    for (int kt = 0; kt < num_kt && ok; ++kt) {
      const int s = kt % kStages;
      if (lane == 0) ok = mbar_wait(full_bar(s), (kt / kStages) & 1, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) { if (lane == 0) raise(abort_flag, p.status, kErrEpilogueWait); break; }
      const uint8_t* sf_s = smem + s * kStageBytes + kABytes + kBBytes + lane * 16;
      const uint32_t t_sf = tmem_sf0 + s * kSfColsPerStage + ((uint32_t)(quad * 32) << 16);
      uint32_t r[16];
      // SFA: columns 0..15 = K blocks 0..3
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        const uint4 v = *reinterpret_cast<const uint4*>(sf_s + 512 * kb);
        r[4 * kb] = v.x; r[4 * kb + 1] = v.y; r[4 * kb + 2] = v.z; r[4 * kb + 3] = v.w;
      }
      tc_st_32x32b_x16(t_sf, r);
      // SFB: per K block 8 columns, rows 0..127 then rows 128..255 of the B tile
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int kb = 2 * half + (q >> 1), tile = q & 1;
          const uint4 v = *reinterpret_cast<const uint4*>(sf_s + kSfaBytes + 2048 * tile + 512 * kb);
          r[4 * q] = v.x; r[4 * q + 1] = v.y; r[4 * q + 2] = v.z; r[4 * q + 3] = v.w;
        }
        tc_st_32x32b_x16(t_sf + 16 + 16 * half, r);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sf_bar(s));
    }
    if (ok && lane == 0) {
      ok = mbar_wait(acc_bar, 0, abort_flag);
      if (!ok) raise(abort_flag, p.status, kErrEpilogueWait);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (ok) {
      tc_fence_after();
      const float alpha = __ldg(p.a_pts) * __ldg(p.b_pts);
      const int64_t row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < kTileN; c0 += 32) {
        if (n0 + c0 >= p.N) break;                               // uniform across the warp
        uint32_t r[32];
        tc_ld_32x32b_x32(taddr + c0, r);
        tc_wait_ld();
        if (row < p.M) {
          const int64_t col = n0 + c0;
          const bool full = (col + 32 <= p.N);
          if (p.out_f32) {
            float* out = static_cast<float*>(p.d) + row * p.ldd + col;
            if (full && ((p.ldd & 3) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(out + j) =
                    make_float4(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha,
                                __uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) out[j] = __uint_as_float(r[j]) * alpha;
            }
          } else {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.d) + row * p.ldd + col;
            if (full && ((p.ldd & 7) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * q]) * alpha,
                                                           __uint_as_float(r[j + 2 * q + 1]) * alpha);
                  w[q] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(out + j) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) out[j] = __float2bfloat16_rn(__uint_as_float(r[j]) * alpha);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// packed E2M1 operand [rows, K/2] bytes, K-major -> 2-D byte tensor map, box 128 bytes x box_rows
static bool make_operand_map(CUtensorMap* map, const uint8_t* ptr, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)(k / 2), (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(k / 2)};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemm
}  // namespace nvfp4

extern "C" int nvfp4_gemm(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts, const uint8_t* b_q,
                          const uint8_t* b_sf, const float* b_pts, void* d, int out_dtype, int64_t M, int64_t N,
                          int64_t K, int64_t ldd, int32_t* status, void* stream_) {
  using namespace nvfp4::gemm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a_q || !a_sf || !a_pts || !b_q || !b_sf || !b_pts || !d) return NVFP4_E_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (K & 31) != 0 || ldd < N) return NVFP4_E_SHAPE;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return NVFP4_E_SHAPE;
  if (out_dtype != NVFP4_OUT_BF16 && out_dtype != NVFP4_OUT_F32) return NVFP4_E_MODE;
  auto mis = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (mis(a_q, 16) || mis(b_q, 16) || mis(a_sf, 16) || mis(b_sf, 16) || mis(d, 16)) return NVFP4_E_ALIGN;
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, a_q, M, K, kTileM) || !make_operand_map(&map_b, b_q, N, K, kTileN))
    return NVFP4_E_DRIVER;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_E_LAUNCH;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return NVFP4_E_LAUNCH;
    attr_set[dev] = true;
  }
  Params p{a_sf, b_sf, a_pts, b_pts, d, M, N, K, ldd, out_dtype == NVFP4_OUT_F32 ? 1 : 0, status};
  const int64_t n_tiles = ((N + kTileN - 1) / kTileN) * ((M + kTileM - 1) / kTileM);
  if (n_tiles > 0x7fffffffLL) return NVFP4_E_SHAPE;
  dim3 grid((unsigned)n_tiles);
  gemm_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}
