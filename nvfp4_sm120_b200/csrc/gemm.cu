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
// gemm_pair.cu holds the persistent cta_group::2 kernel (256 x 256 per CTA pair), gemm_api.cu the C entry point.
#include <atomic>

#include "gemm_common.cuh"

namespace nvfp4 {
namespace gemm {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kStages = 4;
constexpr int kABytes = kTileM * 128;       // 16 KiB
constexpr int kBBytes = kTileN * 128;       // 32 KiB
constexpr int kSfaBytes = 4 * 512;          // 128 rows x 16 scales
constexpr int kSfbBytes = 2 * 4 * 512;      // 256 rows x 16 scales
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 55296
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int kThreads = 192;
constexpr int kSfColsPerStage = 16 + 32;    // SFA 4 columns per K=64 block, SFB 8

__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_d, const Params p) {
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
  const uint32_t tile_id = blockIdx.x / (uint32_t)p.splits, split = blockIdx.x % (uint32_t)p.splits;
  const uint32_t group = tile_id / per_group, first_m = group * kGroupM;
  const uint32_t gsize = min((uint32_t)kGroupM, tiles_m - first_m);
  const uint32_t in_group = tile_id - group * per_group;
  const int64_t m0 = (int64_t)(first_m + in_group % gsize) * kTileM, n0 = (int64_t)(in_group / gsize) * kTileN;
  // this CTA's share of the K slices (all of them unless K is split)
  const int total_kt = (int)((p.K + kTileK - 1) / kTileK);
  const int per_split = (total_kt + p.splits - 1) / p.splits;
  const int kt0 = (int)split * per_split;
  const int num_kt = min(total_kt, kt0 + per_split) - kt0;
  if (num_kt <= 0) return;                                       // whole CTA, before any barrier
  const int64_t sf_col_tiles = (p.K / 16 + 3) / 4;               // 512-byte tiles per 128-row group

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(sf_bar(s), 4); }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    set_wait_limit(abort_flag, p.wait_limit_ns);
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
        const int64_t k_left = p.K - (int64_t)(kt0 + kt) * kTileK;
        const int nkb = k_left >= kTileK ? 4 : (int)((k_left + 63) / 64);
        const uint32_t sf_bytes = (uint32_t)nkb * 512u;
        const uint32_t stage = base + s * kStageBytes;
        mbar_expect_tx(full_bar(s), kABytes + kBBytes + sf_bytes * (second_sfb ? 3u : 2u));
        tma_load_2d(stage, &map_a, (kt0 + kt) * 128, (int)m0, full_bar(s));
        tma_load_2d(stage + kABytes, &map_b, (kt0 + kt) * 128, (int)n0, full_bar(s));
        const uint8_t* sfa = p.a_sf + ((m0 >> 7) * sf_col_tiles + (int64_t)(kt0 + kt) * 4) * 512;
        const uint8_t* sfb = p.b_sf + ((n0 >> 7) * sf_col_tiles + (int64_t)(kt0 + kt) * 4) * 512;
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
      // K slices that hold all four K=64 blocks (every one except possibly the last of the matrix)
      const int whole_kt = (int)min((int64_t)num_kt, max((int64_t)0, p.K / kTileK - kt0));
      int s = 0;
      uint32_t parity = 0;
      for (int kt = 0; kt < num_kt; ++kt) {
        if (!mbar_wait(sf_bar(s), parity, abort_flag)) {                 // implies the TMA data landed
          raise(abort_flag, p.status, kErrMmaWait);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t stage = base + s * kStageBytes;
        const uint32_t t_sfa = tmem_sf0 + s * kSfColsPerStage, t_sfb = t_sfa + 16;
        const uint64_t da = make_desc_sw128(stage), db = make_desc_sw128(stage + kABytes);
        // 64 elements = 32 bytes further along K inside the swizzled row: +2 in 16-byte units.
        // The four instructions go out back to back: the tensor pipe only stays busy while the next
        // one is already queued, so nothing else sits between them.
        if (kt < whole_kt) {
          tc_mma_nvf4(tmem_base, da, db, idesc, t_sfa, t_sfb, kt > 0 ? 1u : 0u);
          tc_mma_nvf4(tmem_base, da + 2u, db + 2u, idesc, t_sfa + 4, t_sfb + 8, 1u);
          tc_mma_nvf4(tmem_base, da + 4u, db + 4u, idesc, t_sfa + 8, t_sfb + 16, 1u);
          tc_mma_nvf4(tmem_base, da + 6u, db + 6u, idesc, t_sfa + 12, t_sfb + 24, 1u);
        } else {
          const int nkb = (int)((p.K - (int64_t)(kt0 + kt) * kTileK + 63) / 64);
          for (int kb = 0; kb < nkb; ++kb)
            tc_mma_nvf4(tmem_base, da + 2u * kb, db + 2u * kb, idesc, t_sfa + 4 * kb, t_sfb + 8 * kb,
                        (kt > 0 || kb > 0) ? 1u : 0u);
        }
        tc_commit(empty_bar(s));          // frees the stage once these MMAs have read it
        if (++s == kStages) { s = 0; parity ^= 1u; }
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
      if (lane == 0 && !(p.drop_first_scale_arrival && kt == 0)) mbar_arrive(sf_bar(s));
    }
    if (ok && lane == 0) {
      ok = mbar_wait(acc_bar, 0, abort_flag);
      if (!ok) raise(abort_flag, p.status, kErrEpilogueWait);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    uint32_t mbits = 0u;
    if (ok) {
      tc_fence_after();
      const float alpha = __ldg(p.a_pts) * __ldg(p.b_pts);
      const int64_t row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      if (p.tma_store) {
        // every MMA has finished and every TMA load has landed, so the stages are free: 32 KiB per warp
        drain_through_tma(p, &map_d, taddr, smem + (warp - 2) * 32768, m0 + quad * 32, n0, 0, kTileN, alpha, lane,
                          mbits);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < kTileN; c0 += 32) {
          if (n0 + c0 >= p.N) break;                             // uniform across the warp
          uint32_t r[32];
          tc_ld_32x32b_x32(taddr + c0, r);
          tc_wait_ld();
          if (p.d_amax_out != nullptr) track_amax(p, r, alpha, row, n0 + c0, mbits);
          if (row < p.M) store_row_chunk(p, row, n0 + c0, r, alpha);
        }
      }
    }
    flush_amax(p, mbits, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace gemm
}  // namespace nvfp4

namespace nvfp4 { namespace gemm {
// launch of the one-CTA kernel (arguments already validated)
int launch_1cta(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const Params& p,
                cudaStream_t stream) {
  static std::atomic<bool> attr_set[64];        // setting the attribute twice is harmless; the flag is atomic
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_E_LAUNCH;
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return NVFP4_E_LAUNCH;
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int64_t n_tiles = ((p.N + kTileN - 1) / kTileN) * ((p.M + kTileM - 1) / kTileM);
  if (n_tiles * p.splits > 0x7fffffffLL) return NVFP4_E_SHAPE;
  gemm_kernel<<<dim3((unsigned)(n_tiles * p.splits)), kThreads, kSmemBytes, stream>>>(map_a, map_b, map_d, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}
}}  // namespace nvfp4::gemm
