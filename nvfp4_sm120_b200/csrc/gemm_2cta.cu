// Two-CTA block-scaled NVFP4 GEMM for B200 (sm_100a): a pair of CTAs on neighbouring SMs (a
// cluster of 2) computes one 256 x 256 output tile with tcgen05.mma cta_group::2.
//
// Why pairs: per K slice of 256 a one-CTA 128 x 256 tile has to bring 48 KiB of operands from the L2
// into shared memory for 512 cycles of MMA work, and the L2 -> SM path delivers about 64 bytes per
// clock; in a pair each CTA holds only half of the B rows (32 KiB per slice for the same flops).
// This file is the one-tile-per-cluster form; gemm_pair.cu is the persistent form of the same
// kernel, which nvfp4_gemm picks by default.
//
// Per CTA (rank r in the pair) and K slice of 256 elements:
//   TMA tensor copies: A rows [m0 + 128 r, +128), B rows [n0 + 128 r, +128)  -> 128B-swizzled smem,
//     completing on the LEADER's (rank 0) "full" barrier (cta_group::2 form, no multicast);
//   bulk copies: scale tiles of its own A rows and of all 256 B rows -> smem, on a local barrier;
//   warps 2..9 (two sets of four, alternating K slices): scale factors smem -> registers -> tensor
//     memory (tcgen05.st), then arrive on the leader's "scales ready" barrier (remote for rank 1);
//   leader's warp 1, one lane: waits for both, issues four MMAs (M 256 = 128 per CTA, N 256, K 64),
//     then commits to the "empty" barrier of BOTH CTAs (two commits, one local, one remote).
// Each CTA's warps 2..9 finally drain their own 128 accumulator rows.  All waits are bounded; the
// kernel ends with a cluster barrier before the paired tensor-memory free.
#include "gemm_common.cuh"

namespace nvfp4 {
namespace gemm2 {

using namespace nvfp4::gemm;

constexpr int kTileN = 256;
constexpr int kStages = 5;
constexpr int kABytes = 128 * 128;          // this CTA's 128 A rows
constexpr int kBBytes = 128 * 128;          // this CTA's 128 of the 256 B rows
constexpr int kSfaBytes = 4 * 512;
constexpr int kSfbBytes = 2 * 4 * 512;
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;      // 38912
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr int kThreads = 320;             // producer, MMA issuer, and two sets of four scale/epilogue warps
constexpr int kSfColsPerStage = 48;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Remote arrive, relaxed: the tensor-memory stores it announces are already complete
// (tcgen05.wait::st precedes it), and a release at cluster scope costs ~1100 cycles here.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const __grid_constant__ CUtensorMap map_d, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                 // same offset in both CTAs of the pair
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar_base = base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                    // leader: A/B of both CTAs landed
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };        // MMAs have read the stage
  auto sfull_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };    // this CTA's scale tiles landed
  auto sready_bar = [&](int s) { return bar_base + 8u * (3 * kStages + s); };   // leader: scales in TMEM, both CTAs
  const uint32_t acc_bar = bar_base + 8u * (4 * kStages);
  const int misc = kStages * kStageBytes + 8 * (4 * kStages + 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // rasterization over PAIRS of row tiles (256 rows), kGroupM / 2 pairs per group
  const uint32_t tiles_n = (uint32_t)((p.N + kTileN - 1) / kTileN), pairs_m = (uint32_t)((p.M + 255) / 256);
  constexpr uint32_t kGroupPairs = kGroupM / 2;
  const uint32_t pid = blockIdx.x >> 1;
  const uint32_t per_group = kGroupPairs * tiles_n;
  const uint32_t group = pid / per_group, first = group * kGroupPairs;
  const uint32_t gsize = min(kGroupPairs, pairs_m - first);
  const uint32_t in_group = pid - group * per_group;
  const int64_t m0 = (int64_t)(first + in_group % gsize) * 256 + (int64_t)rank * 128;
  const int64_t n0 = (int64_t)(in_group / gsize) * kTileN;
  const int num_kt = (int)((p.K + kTileK - 1) / kTileK);
  const int64_t sf_col_tiles = (p.K / 16 + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(sfull_bar(s), 1); mbar_init(sready_bar(s), 8);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf0 = tmem_base + kTileN;

  if (warp == 0) {
    // ------------------------------ producer (one per CTA) ------------------------------
    if (lane == 0) {
      const bool have_sfa = m0 < p.M;                            // padded pair: no such rows in the scale buffer
      const bool second_sfb = (n0 + 128) < p.N;
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
        const uint32_t leader_full = map_to_cta(full_bar(s), 0);
        if (leader) mbar_expect_tx(full_bar(s), 2u * (kABytes + kBBytes));
        tma_load_2d_pair(stage, &map_a, kt * 128, (int)m0, leader_full);
        tma_load_2d_pair(stage + kABytes, &map_b, kt * 128, (int)(n0 + rank * 128), leader_full);
        mbar_expect_tx(sfull_bar(s), sf_bytes * ((have_sfa ? 1u : 0u) + 1u + (second_sfb ? 1u : 0u)));
        const uint8_t* sfa = p.a_sf + ((m0 >> 7) * sf_col_tiles + (int64_t)kt * 4) * 512;
        const uint8_t* sfb = p.b_sf + ((n0 >> 7) * sf_col_tiles + (int64_t)kt * 4) * 512;
        if (have_sfa) bulk_load(stage + kABytes + kBBytes, sfa, sf_bytes, sfull_bar(s));
        bulk_load(stage + kABytes + kBBytes + kSfaBytes, sfb, sf_bytes, sfull_bar(s));
        if (second_sfb)
          bulk_load(stage + kABytes + kBBytes + kSfaBytes + 2048, sfb + sf_col_tiles * 512, sf_bytes, sfull_bar(s));
        ++issued;
      }
      if (*abort_flag != 0) {
        const int first_kt = issued > kStages ? issued - kStages : 0;
        for (int kt = first_kt; kt < issued; ++kt)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(sfull_bar(kt % kStages), (kt / kStages) & 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(256, kTileN);
      bool ok = true;
      const int whole_kt = (int)min((int64_t)num_kt, p.K / kTileK);     // K slices with all four K=64 blocks
      const uint32_t partner_empty0 = map_to_cta(empty_bar(0), 1);
      int s = 0;
      uint32_t par = 0;
      for (int kt = 0; kt < num_kt; ++kt) {
        // one wait per K slice: the leader's scale warps arrive only after the operand tiles of both
        // CTAs have landed, so "scales ready" covers "data landed"
        if (!mbar_wait(sready_bar(s), par, abort_flag)) {
          raise(abort_flag, p.status, kErrMmaWait);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t stage = base + s * kStageBytes;
        const uint32_t t_sfa = tmem_sf0 + s * kSfColsPerStage, t_sfb = t_sfa + 16;
        const uint64_t da = make_desc_sw128(stage), db = make_desc_sw128(stage + kABytes);
        if (kt < whole_kt) {                                  // back to back, nothing in between
          tc_mma_nvf4_pair(tmem_base, da, db, idesc, t_sfa, t_sfb, kt > 0 ? 1u : 0u);
          tc_mma_nvf4_pair(tmem_base, da + 2u, db + 2u, idesc, t_sfa + 4, t_sfb + 8, 1u);
          tc_mma_nvf4_pair(tmem_base, da + 4u, db + 4u, idesc, t_sfa + 8, t_sfb + 16, 1u);
          tc_mma_nvf4_pair(tmem_base, da + 6u, db + 6u, idesc, t_sfa + 12, t_sfb + 24, 1u);
        } else {
          const int nkb = (int)((p.K - (int64_t)kt * kTileK + 63) / 64);
          for (int kb = 0; kb < nkb; ++kb)
            tc_mma_nvf4_pair(tmem_base, da + 2u * kb, db + 2u * kb, idesc, t_sfa + 4 * kb, t_sfb + 8 * kb,
                             (kt > 0 || kb > 0) ? 1u : 0u);
        }
        tc_commit_pair(empty_bar(s));                       // frees the stage here ...
        tc_commit_pair(partner_empty0 + 8u * s);            // ... and in the partner CTA
        if (++s == kStages) { s = 0; par ^= 1u; }
      }
      if (ok) {
        tc_commit_pair(acc_bar);
        tc_commit_pair(map_to_cta(acc_bar, 1));
      }
    }
  } else {
    // ------------------------------ scale factors, then epilogue ------------------------------
    const int quad = warp & 3;                    // tensor-memory lanes 32 * quad .. + 31
    const int set = (warp - 2) >> 2;              // the two sets of four warps take alternate K slices
    bool ok = true;
    const uint32_t leader_ready0 = map_to_cta(sready_bar(0), 0);
    for (int kt = set; kt < num_kt && ok; kt += 2) {
      const int s = kt % kStages;
      if (lane == 0) {
        ok = mbar_wait(sfull_bar(s), (kt / kStages) & 1, abort_flag);
        if (ok && leader) ok = mbar_wait(full_bar(s), (kt / kStages) & 1, abort_flag);   // see the MMA issuer
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) { if (lane == 0) raise(abort_flag, p.status, kErrScaleWait); break; }
      const uint8_t* sf_s = smem + s * kStageBytes + kABytes + kBBytes + lane * 16;
      const uint32_t t_sf = tmem_sf0 + s * kSfColsPerStage + ((uint32_t)(quad * 32) << 16);
      uint32_t r[16];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        const uint4 v = *reinterpret_cast<const uint4*>(sf_s + 512 * kb);
        r[4 * kb] = v.x; r[4 * kb + 1] = v.y; r[4 * kb + 2] = v.z; r[4 * kb + 3] = v.w;
      }
      tc_st_32x32b_x16(t_sf, r);
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
      if (lane == 0) { if (leader) mbar_arrive(sready_bar(s)); else mbar_arrive_cluster(leader_ready0 + 8u * s); }
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
      if (p.tma_store) {
        // every MMA of the pair has finished and every load has landed: the stages are free, 16 KiB per warp
        drain_through_tma(p, &map_d, taddr, smem + (warp - 2) * 16384, m0 + quad * 32, n0, 128 * set, 128 * set + 128,
                          alpha, lane);
      } else {
#pragma unroll 1
        for (int c0 = 128 * set; c0 < 128 * set + 128; c0 += 32) {   // each set drains half of the columns
          if (n0 + c0 >= p.N) break;
          uint32_t r[32];
          tc_ld_32x32b_x32(taddr + c0, r);
          tc_wait_ld();
          if (row < p.M) store_row_chunk(p, row, n0 + c0, r, alpha);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA frees tensor memory while the partner may still use the pair
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

int launch_2cta(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const Params& p,
                cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_E_LAUNCH;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return NVFP4_E_LAUNCH;
    attr_set[dev] = true;
  }
  const int64_t n_ctas = 2 * ((p.N + kTileN - 1) / kTileN) * ((p.M + 255) / 256);
  if (n_ctas > 0x7fffffffLL) return NVFP4_E_SHAPE;
  gemm2_kernel<<<dim3((unsigned)n_ctas), kThreads, kSmemBytes, stream>>>(map_a, map_b, map_d, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

}  // namespace gemm2
}  // namespace nvfp4
