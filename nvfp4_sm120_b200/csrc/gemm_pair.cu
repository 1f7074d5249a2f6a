// Persistent two-CTA block-scaled NVFP4 GEMM for B200 (sm_100a).
//
// One cluster of two CTAs per pair of SMs stays resident and walks over 256 x 256 output tiles
// (tile = cluster index + i * number of clusters, grouped rasterization).  The roles of a CTA:
//   warp 0      producer: TMA tensor copies of its 128 A rows and its 128 of the 256 B rows
//               (cta_group::2 form, completing on the leader's barrier; no multicast) and bulk
//               copies of the scale tiles, into a ring of five stages that runs on across tiles;
//   warp 1      (leader CTA only) issues tcgen05.mma cta_group::2, M 256 = 128 per CTA, N 256, K 64:
//               four per K slice, back to back, one barrier wait per slice;
//   warps 2-5   scale factors shared memory -> registers -> tensor memory (one warp per 32-lane quarter);
//   warps 6-13  epilogue: tensor memory -> registers -> swizzled shared memory -> TMA store.
// Because the ring never drains, the loads of the next tile are in flight while the epilogue warps
// empty the accumulator; the MMA issuer only waits for "accumulator read" before the next tile, so
// the launch, barrier set-up, tensor-memory allocation and pipeline fill are paid once per SM pair,
// not once per tile.  All waits are bounded (they raise the status word and every role leaves its
// loops); the kernel ends with a cluster barrier before the paired tensor-memory free.
#include <atomic>

#include "gemm_common.cuh"

namespace nvfp4 {
namespace gemm3 {

using namespace nvfp4::gemm;

constexpr int kTileN = 256;
constexpr int kStages = 5;
constexpr int kABytes = 128 * 128;          // this CTA's 128 A rows
constexpr int kBBytes = 128 * 128;          // this CTA's 128 of the 256 B rows
constexpr int kSfaBytes = 4 * 512;
constexpr int kSfbBytes = 2 * 4 * 512;
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;      // 38912
constexpr int kOutBytes = 8 * 4096;         // per epilogue warp one box of 32 rows x 128 bytes
constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024 + 256;
constexpr int kSfSets = 1;                  // groups of four scale-factor warps taking the K slices in turn
constexpr int kEpiWarp0 = 2 + 4 * kSfSets;  // first epilogue warp
constexpr int kThreads = (kEpiWarp0 + 8) * 32;
constexpr int kSfColsPerStage = 48;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Remote arrive, relaxed: what it announces (tcgen05.st / tcgen05.ld) has already completed
// (tcgen05.wait precedes it); a release at cluster scope costs about 1100 cycles here.
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

// tile index -> first row of the pair and first column (grouped rasterization over pairs of row tiles)
struct TileMap {
  uint32_t tiles_n, pairs_m, per_group;
  __device__ TileMap(const Params& p)
      : tiles_n((uint32_t)((p.N + kTileN - 1) / kTileN)), pairs_m((uint32_t)((p.M + 255) / 256)),
        per_group((kGroupM / 2) * tiles_n) {}
  __device__ uint32_t total() const { return tiles_n * pairs_m; }
  __device__ void locate(uint32_t tile, int64_t& pair_m0, int64_t& n0) const {
    const uint32_t group = tile / per_group, first = group * (kGroupM / 2);
    const uint32_t gsize = min((uint32_t)(kGroupM / 2), pairs_m - first);
    const uint32_t in_group = tile - group * per_group;
    pair_m0 = (int64_t)(first + in_group % gsize) * 256;
    n0 = (int64_t)(in_group / gsize) * kTileN;
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const __grid_constant__ CUtensorMap map_d, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                 // same offset in both CTAs of the pair
  uint8_t* smem = smem_raw + (base - raw);
  uint8_t* out_stage = smem + kStages * kStageBytes;            // epilogue boxes (1024-byte aligned)
  const uint32_t bar_base = base + kStages * kStageBytes + kOutBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                    // leader: A/B of both CTAs landed
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };        // MMAs have read the stage
  auto sfull_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };    // this CTA's scale tiles landed
  auto sready_bar = [&](int s) { return bar_base + 8u * (3 * kStages + s); };   // leader: scales in TMEM, both CTAs
  const uint32_t acc_full = bar_base + 8u * (4 * kStages);                      // accumulator complete (both CTAs)
  const uint32_t acc_empty = bar_base + 8u * (4 * kStages + 1);                 // leader: accumulator read, both CTAs
  const int misc = kStages * kStageBytes + kOutBytes + 8 * (4 * kStages + 2);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const TileMap tm(p);
  const uint32_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1, total = tm.total();
  const int my_tiles = cluster_id < total ? (int)((total - cluster_id + n_clusters - 1) / n_clusters) : 0;
  const int num_kt = (int)((p.K + kTileK - 1) / kTileK);
  const int64_t sf_col_tiles = (p.K / 16 + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(sfull_bar(s), 1); mbar_init(sready_bar(s), 8);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 16);
    *abort_flag = 0;
    set_wait_limit(abort_flag, p.wait_limit_ns);
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
      int s = 0, issued = 0;
      uint32_t pass = 0;                                          // parity of the current pass over the ring
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        int64_t pair_m0, n0;
        tm.locate(cluster_id + (uint32_t)i * n_clusters, pair_m0, n0);
        const int64_t m0 = pair_m0 + (int64_t)rank * 128;
        const bool have_sfa = m0 < p.M;                           // padded pair: no such rows in the scale buffer
        const bool second_sfb = (n0 + 128) < p.N;
        const uint8_t* sfa_row = p.a_sf + (m0 >> 7) * sf_col_tiles * 512;
        const uint8_t* sfb_row = p.b_sf + (n0 >> 7) * sf_col_tiles * 512;
        for (int kt = 0; kt < num_kt; ++kt) {
          if (issued >= kStages && !mbar_wait(empty_bar(s), pass ^ 1u, abort_flag)) {
            raise(abort_flag, p.status, kErrProducerWait);
            ok = false;
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
          const int64_t off = (int64_t)kt * 4 * 512;
          if (have_sfa) bulk_load(stage + kABytes + kBBytes, sfa_row + off, sf_bytes, sfull_bar(s));
          bulk_load(stage + kABytes + kBBytes + kSfaBytes, sfb_row + off, sf_bytes, sfull_bar(s));
          if (second_sfb)
            bulk_load(stage + kABytes + kBBytes + kSfaBytes + 2048, sfb_row + sf_col_tiles * 512 + off, sf_bytes,
                      sfull_bar(s));
          ++issued;
          if (++s == kStages) { s = 0; pass ^= 1u; }
        }
      }
      if (*abort_flag != 0) {
        // give copies already in flight a bounded chance to land before shared memory goes away
        const int first_g = issued > kStages ? issued - kStages : 0;
        for (int g = first_g; g < issued; ++g) {
          for (uint32_t n = 0; n < (1u << 16) && !mbar_try_wait(sfull_bar(g % kStages), (g / kStages) & 1); ++n) {}
          if (leader)
            for (uint32_t n = 0; n < (1u << 16) && !mbar_try_wait(full_bar(g % kStages), (g / kStages) & 1); ++n) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(256, kTileN);
      const int whole_kt = (int)min((int64_t)num_kt, p.K / kTileK);     // K slices with all four K=64 blocks
      const uint32_t partner_empty0 = map_to_cta(empty_bar(0), 1);
      const uint32_t partner_acc_full = map_to_cta(acc_full, 1);
      int s = 0;
      uint32_t par = 0;
      bool ok = true;
      for (int i = 0; i < my_tiles && ok; ++i) {
        if (i > 0) {                                            // the epilogue warps have read the accumulator
          if (!mbar_wait(acc_empty, (uint32_t)(i - 1) & 1u, abort_flag)) {
            raise(abort_flag, p.status, kErrMmaWait);
            break;
          }
          tc_fence_after();
        }
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
          tc_commit_pair(acc_full);
          tc_commit_pair(partner_acc_full);
        }
      }
    }
  } else if (warp < kEpiWarp0) {
    // ------------------------------ scale factors ------------------------------
    // Lane l / 32-bit column c of a K=64 block must hold, in every 32-lane quarter of tensor memory,
    // the four E4M3 scales of row 32c + l: exactly 16 bytes per lane of the 512-byte tile the
    // quantizer wrote, so one 128-bit shared load per tile and lane feeds four columns, and each
    // warp writes the copy of its own quarter.  The two sets take alternate K slices.
    const int quad = warp & 3;
    const int set = (warp - 2) >> 2;
    const uint32_t leader_ready0 = map_to_cta(sready_bar(0), 0);
    const int64_t total_g = (int64_t)my_tiles * num_kt;
    bool ok = true;
    for (int64_t g = set; g < total_g && ok; g += kSfSets) {
      const int s = (int)(g % kStages);
      const uint32_t par = (uint32_t)(g / kStages) & 1u;
      if (lane == 0) {
        ok = mbar_wait(sfull_bar(s), par, abort_flag);
        if (ok && leader) ok = mbar_wait(full_bar(s), par, abort_flag);   // see the MMA issuer
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
      if (lane == 0 && !(p.drop_first_scale_arrival && g == 0)) {
        if (leader) mbar_arrive(sready_bar(s)); else mbar_arrive_cluster(leader_ready0 + 8u * s);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // Two warps per 32-lane quarter of tensor memory, 128 accumulator columns each.  For bf16 output a
    // warp pulls its 32 x 128 slab into registers as packed bf16 (64 registers), signals "accumulator
    // read" -- the MMA issuer starts the next tile about 600 cycles after the last MMA of this one --
    // and only then writes the slab out at leisure, under the next tile's main loop: swizzled
    // 32 x 128-byte box in shared memory -> TMA store, which writes whole lines and clips at the
    // matrix edge.  fp32 output (128 registers would not fit) goes box by box and signals after its
    // last tensor-memory load.
    const int quad = warp & 3;
    const int c_base = 128 * ((warp - kEpiWarp0) >> 2);
    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + c_base;
    uint8_t* box = out_stage + (warp - kEpiWarp0) * 4096;
    const uint32_t box_u32 = smem_u32(box);
    uint8_t* rowp = box + lane * 128;
    const uint32_t leader_acc_empty = map_to_cta(acc_empty, 0);
    const float alpha = __ldg(p.a_pts) * __ldg(p.b_pts);
    const uint32_t sw = (uint32_t)lane & 7u;
    bool ok = true;
    uint32_t mbits = 0u;                                          // running max|D| (see track_amax)
    auto release_accumulator = [&]() {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { if (leader) mbar_arrive(acc_empty); else mbar_arrive_cluster(leader_acc_empty); }
    };
    auto send_box = [&](int64_t x, int64_t y) {                   // the box is written: hand it to the TMA unit
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> TMA reads
      __syncwarp();
      if (lane == 0) tma_store_2d(&map_d, box_u32, (int)x, (int)y);
    };
    auto box_free = [&]() {                                       // its last store has read the box
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
    };
    for (int i = 0; i < my_tiles; ++i) {
      int64_t pair_m0, n0;
      tm.locate(cluster_id + (uint32_t)i * n_clusters, pair_m0, n0);
      const int64_t row0 = pair_m0 + (int64_t)rank * 128 + quad * 32;
      const int64_t col0 = n0 + c_base;
      if (lane == 0) ok = mbar_wait_relaxed(acc_full, (uint32_t)i & 1u, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) { if (lane == 0) raise(abort_flag, p.status, kErrEpilogueWait); break; }
      tc_fence_after();
      if (row0 >= p.M || col0 >= p.N) {                           // padding only: nothing to read
        release_accumulator();
        continue;
      }
      if (p.tma_store && !p.out_f32) {
        uint32_t packed[64];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tc_ld_32x32b_x32(taddr + 32 * ch, r);
          tc_wait_ld();
          if (p.d_amax_out != nullptr) track_amax(p, r, alpha, row0 + lane, col0 + 32 * ch, mbits);
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * q]) * alpha, __uint_as_float(r[2 * q + 1]) * alpha);
            packed[16 * ch + q] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        release_accumulator();
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          if (col0 + 64 * b >= p.N) break;                        // uniform across the warp
          box_free();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + (((uint32_t)j ^ sw) << 4)) =
                make_uint4(packed[32 * b + 4 * j], packed[32 * b + 4 * j + 1], packed[32 * b + 4 * j + 2], packed[32 * b + 4 * j + 3]);
          send_box(col0 + 64 * b, row0);
        }
      } else {
        const int64_t n_left = p.N - col0;
        const int chunks = n_left >= 128 ? 4 : (int)((n_left + 31) / 32);
#pragma unroll 1
        for (int ch = 0; ch < chunks; ++ch) {
          uint32_t r[32];
          tc_ld_32x32b_x32(taddr + 32 * ch, r);
          tc_wait_ld();
          if (ch == chunks - 1) release_accumulator();
          if (p.d_amax_out != nullptr) track_amax(p, r, alpha, row0 + lane, col0 + 32 * ch, mbits);
          if (!p.tma_store) {
            if (row0 + lane < p.M) store_row_chunk(p, row0 + lane, col0 + 32 * ch, r, alpha);
            continue;
          }
          box_free();                                             // fp32: a box is 32 columns
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(rowp + (((uint32_t)j ^ sw) << 4)) =
                make_float4(__uint_as_float(r[4 * j]) * alpha, __uint_as_float(r[4 * j + 1]) * alpha,
                            __uint_as_float(r[4 * j + 2]) * alpha, __uint_as_float(r[4 * j + 3]) * alpha);
          send_box(col0 + 32 * ch, row0);
        }
      }
    }
    box_free();                                                   // before shared memory goes away
    flush_amax(p, mbits, lane);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA frees tensor memory while the partner may still use the pair
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const Params& p,
                cudaStream_t stream) {
  static std::atomic<int> sm_count[64];         // 0 = not looked up yet; a second look-up is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_E_LAUNCH;
  int sms = sm_count[dev].load(std::memory_order_acquire);
  if (sms == 0) {
    if (cudaFuncSetAttribute(gemm3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return NVFP4_E_LAUNCH;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
      return NVFP4_E_LAUNCH;
    sm_count[dev].store(sms, std::memory_order_release);
  }
  const int64_t tiles = ((p.N + kTileN - 1) / kTileN) * ((p.M + 255) / 256);
  if (tiles > 0x3fffffffLL) return NVFP4_E_SHAPE;
  const int64_t clusters = tiles < sms / 2 ? tiles : sms / 2;    // one resident pair per two SMs
  gemm3_kernel<<<dim3((unsigned)(2 * clusters)), kThreads, kSmemBytes, stream>>>(map_a, map_b, map_d, p);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

}  // namespace gemm3
}  // namespace nvfp4
