// Single-launch NVFP4 quantizer, tile form (sm_100a): blocks along the columns of a row-major bf16
// matrix, work cut into tiles of 128 rows x 64 columns = 512 blocks of 16 = exactly one 512-byte
// tile of the swizzled scale layout.
//
// Why tiles: the quantize phase is bound by how many 32-byte sectors the SM hands to the L2, not by
// arithmetic.  With a lane per consecutive block of one row, a warp's 32 scale bytes land in eight
// different 512-byte scale tiles (eight partly written sectors per store instruction, as many as
// the packed data itself).  Here a warp owns rows {2w, 2w+1} + 32 g (g = 0..3) of a tile and four
// blocks of each, so its 32 scale bytes are ONE contiguous 32-byte sector and its 256 data bytes are
// eight full sectors: 9 sector writes per 32 blocks instead of 16, and padding rows / columns of the
// scale buffer are written as zeros on the way (no separate clearing pass).
//
// Data movement: every tile is brought into shared memory by one TMA tensor copy (box 64 x 128
// elements, 128-byte swizzle, out-of-range rows and columns read as zero) into a ring of five 16 KiB
// slots per half CTA (two halves of 16 warps work on two tiles at a time).  The swizzle makes the two
// 128-bit shared loads of a lane conflict-free, and every per-lane address (shared offsets, output
// row, scale byte) is a loop invariant: a tile costs a thread a handful of pointer bumps.
//   phase 1  (two-phase kernel) all tiles of the half CTA's range stream through the ring for the
//            per-tensor maximum; each block's maximum is kept (2 bytes) for phase 2; the last five
//            tiles stay in the ring.
//   barrier  red.max + arrival counter in the workspace, bounded wait (see quantize_common.cuh).
//   phase 2  the resident tiles are quantized first; every slot that frees up is refilled from the
//            L2 with the next tile of the head of the range, so the loads run ahead of the math.
// With the maximum given (KNOWN) the kernel is phase 2 alone over all tiles, straight from HBM.
// Arithmetic and Philox counters are those of the other quantizer kernels: the bytes are identical.
#include <cuda.h>

#include "quantize_common.cuh"

namespace nvfp4 {
namespace tiled {

using namespace nvfp4::fused;

constexpr int kThreads = 1024;
constexpr int kHalfThreads = 512;
constexpr int kTileRows = 128;
constexpr int kTileCols = 64;                              // elements: four blocks of 16
constexpr int kTileBytes = kTileRows * kTileCols * 2;      // 16 KiB
constexpr int kPairBytes = 2 * kTileBytes;                 // a ring slot holds two consecutive tiles
constexpr int kSlots = 3;                                  // ring depth per half CTA, in pairs
constexpr int kTabTiles = 16;                              // per half CTA: block maxima of its first 16 tiles
constexpr int kRingBytes = 2 * kSlots * kPairBytes;        // 192 KiB
constexpr int kTabBytes = 2 * kTabTiles * kHalfThreads * 2;   // 32 KiB
constexpr int kMiscOff = kRingBytes + kTabBytes;
constexpr int kSmemBytes = kMiscOff + 1024 /* tables, barriers */ + 1024 /* alignment slack */;

enum : int { kErrBarrier = 1, kErrCopy = 2 };

struct Params {
  uint32_t rows, bpr;            // rows of x, 16-element blocks per row
  uint32_t ntc, ntiles;          // column tiles per row of tiles, tiles in all
  uint32_t ctr_pitch, ctr_base;  // Philox counter of block (row, kb) = row * ctr_pitch + ctr_base + kb
  uint64_t q_pitch;              // bytes per row of qdata (cols / 2)
  const float* signs16;
  PhiloxKeys keys;
  uint64_t offset;
  uint8_t* qdata;
  uint8_t* scales;
  float* pts_out;
  Workspace* ws;
  const float* amax_in;
  unsigned long long wait_limit_ns;
  uint32_t extra_arrivals;       // test hook: surplus arrivals the grid barrier expects (normally 0)
};

__device__ __forceinline__ void tma_tile_load(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Bounded wait on an mbarrier phase; false when it gave up or the CTA is already aborting.
__device__ __forceinline__ bool wait_phase(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                           unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t n = 1;; ++n) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((n & 127u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_ns() - t0 > limit_ns) return false;
    }
  }
}

// Where this lane's block of the current tile goes: running pointers into the two outputs, the block's
// Philox counter and whether the block lies inside the matrix.  step() moves to the next tile in range
// order with additions only (a row of tiles ends every ntc tiles).
struct Cursor {
  uint8_t* q;            // this lane's 8 bytes of packed codes
  uint8_t* s;            // this lane's scale byte
  uint32_t i;            // block index row * bpr + k/16 (the Philox counter)
  uint32_t ct, rt;
  bool inside;
};
struct CursorConst {
  uint32_t ntc, rows, bpr, row_t, kb, ctr_pitch, ctr_base;
  uint64_t q_wrap;       // from the last tile of a row of tiles to the first of the next: 128 rows down, back to column 0
  uint32_t i_wrap;
};
__device__ __forceinline__ void cursor_set(Cursor& c, const CursorConst& k, uint32_t tile, uint8_t* qdata, uint64_t q_pitch,
                                           uint64_t q_lane, uint8_t* scales, uint32_t sc_lane) {
  c.rt = tile / k.ntc;
  c.ct = tile - c.rt * k.ntc;
  c.q = qdata + (uint64_t)c.rt * (128u * q_pitch) + c.ct * 32u + q_lane;
  c.s = scales + (uint64_t)tile * 512u + sc_lane;
  c.i = (c.rt * 128u + k.row_t) * k.ctr_pitch + k.ctr_base + c.ct * 4u + k.kb;
  c.inside = c.rt * 128u + k.row_t < k.rows && c.ct * 4u + k.kb < k.bpr;
}
__device__ __forceinline__ void cursor_step(Cursor& c, const CursorConst& k) {
  c.q += 32; c.s += 512; c.i += 4u;
  if (++c.ct == k.ntc) {
    c.ct = 0; ++c.rt;
    c.q += k.q_wrap; c.i += k.i_wrap;
  }
  c.inside = c.rt * 128u + k.row_t < k.rows && c.ct * 4u + k.kb < k.bpr;
}

template <bool SR, bool RHT, bool KNOWN>
__global__ void __launch_bounds__(kThreads, 1)
quant_tiled_kernel(const __grid_constant__ CUtensorMap map_x, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);          // the swizzle wants 1024-byte alignment
  float* recip_tab = reinterpret_cast<float*>(smem + kMiscOff);          // 128 floats
  float* red = reinterpret_cast<float*>(smem + kMiscOff + 512);          // 32 floats
  float* sgs = reinterpret_cast<float*>(smem + kMiscOff + 640);          // 16 floats
  const uint32_t bars = smem_u32(smem + kMiscOff + 704);                 // full[2][kSlots]: a pair has landed
  const uint32_t counts = smem_u32(smem + kMiscOff + 704 + 8 * 2 * kSlots);   // done[2][kSlots]: warps finished with a slot
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + kMiscOff + 704 + 8 * 2 * kSlots + 4 * 2 * kSlots);

  const uint32_t tid = threadIdx.x, half = tid >> 9, tih = tid & 511u, lane = tid & 31u, wsub = tih >> 5;
  const uint32_t full0 = bars + 8u * (half * kSlots), done0 = counts + 4u * (half * kSlots);
  const uint32_t ring = smem_u32(smem) + half * (kSlots * kPairBytes);
  uint16_t* tab = reinterpret_cast<uint16_t*>(smem + kRingBytes) + half * (kTabTiles * kHalfThreads) + tih;

  // this half CTA's contiguous range of tiles, walked in pairs
  const uint64_t halves = 2ull * gridDim.x, hid = 2ull * blockIdx.x + half;
  const uint32_t t0 = (uint32_t)(hid * p.ntiles / halves), t1 = (uint32_t)((hid + 1) * p.ntiles / halves);
  const uint32_t nt = t1 - t0, np = (nt + 1u) >> 1;
  const uint32_t resident = KNOWN ? 0u : min(np, (uint32_t)kSlots);      // pairs phase 1 leaves in the ring
  const uint32_t head = np - resident;                                   // pairs phase 2 fetches (again)

  if (tid == 0) {
    for (uint32_t b = 0; b < 2u * kSlots; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars + 8u * b));
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(counts + 4u * b), "r"(0u) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *cta_abort = 0;
  }
  if (RHT && tid < 16) sgs[tid] = __ldg(p.signs16 + tid);
  const bool stamper = blockIdx.x == 0 && tid == 0 && p.ws != nullptr;
  unsigned long long t_start = 0;
  if (stamper) { t_start = global_ns(); p.ws->start = t_start; p.ws->last_end = 0ull; }
  unsigned int epoch = 0;
  if (tid == 0 && !KNOWN) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(&p.ws->epoch) : "memory");
  __syncthreads();

  // ---- per-lane invariants ------------------------------------------------------------------
  // lane -> (block kb of four, row pair h, row group g): rows {2 wsub + h + 32 g} of a tile
  const uint32_t kb = lane & 3u, hrow = (lane >> 2) & 1u, grp = lane >> 3;
  const uint32_t row_t = 2u * wsub + hrow + 32u * grp;
  const uint32_t off0 = row_t * 128u + (((2u * kb) ^ (row_t & 7u)) << 4);        // 128-byte swizzle: 16-byte chunk c
  const uint32_t off1 = row_t * 128u + (((2u * kb + 1u) ^ (row_t & 7u)) << 4);   // of row r sits at c ^ (r & 7)
  const uint32_t sc_lane = (2u * wsub + hrow) * 16u + grp * 4u + kb;             // byte inside the 512-byte scale tile
  const uint64_t q_lane = (uint64_t)row_t * p.q_pitch + kb * 8u;
  const CursorConst cc{p.ntc, p.rows, p.bpr, row_t, kb, p.ctr_pitch, p.ctr_base,
                       128ull * p.q_pitch - 32ull * p.ntc, 128u * p.ctr_pitch - 4u * p.ntc};
  uint32_t sm[8];                 // sign-bit masks of the packed bf16 pairs (bit 15: even, bit 31: odd)
#pragma unroll
  for (int j = 0; j < 8; ++j)
    sm[j] = RHT ? ((sgs[2 * j] < 0.0f ? 0x8000u : 0u) | (sgs[2 * j + 1] < 0.0f ? 0x80000000u : 0u)) : 0u;

  // Fill number f of this half's ring goes to slot f % kSlots and completes phase (f / kSlots) & 1 of
  // its barrier.  Phase 1 uses fills 0 .. np-1 (pair f of the range); phase 2 fetches the head of the
  // range again as fills np .. (pair f - np).  KNOWN has no phase 1: its fills are the pairs in order.
  auto issue_fill = [&](uint32_t f) {
    const uint32_t pair = (KNOWN || f < np) ? f : f - np;
    const uint32_t ta = t0 + 2u * pair;
    const bool two = ta + 1u < t1;
    const uint32_t rt = ta / p.ntc, ct = ta - rt * p.ntc;
    const uint32_t s = f % kSlots, bar = full0 + 8u * s, dst = ring + s * kPairBytes;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 ::"r"(bar), "r"((uint32_t)(two ? kPairBytes : kTileBytes)) : "memory");
    tma_tile_load(dst, &map_x, (int)(ct * kTileCols), (int)(rt * kTileRows), bar);
    if (two) {
      const bool wrap = ct + 1u == p.ntc;
      tma_tile_load(dst + kTileBytes, &map_x, (int)(wrap ? 0u : (ct + 1u) * kTileCols),
                    (int)((wrap ? rt + 1u : rt) * kTileRows), bar);
    }
  };
  auto load_block = [&](uint32_t addr, uint32_t (&w)[8]) {
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr + off0));
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(addr + off1));
  };
  // This warp has read slot s.  The warp that finishes LAST with the slot (sixteen share it) puts
  // fill `next_f` into it; nobody waits for a slot to become free.  The acq_rel increment orders
  // every warp's reads of the slot before the last one's copy into it.
  auto release_and_refill = [&](uint32_t s, uint32_t next_f) {
    __syncwarp();
    if (lane == 0) {
      uint32_t before;
      asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(before) : "r"(done0 + 4u * s) : "memory");
      if (before == 15u) {
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(done0 + 4u * s), "r"(0u) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic reads of the slot before the async write
        issue_fill(next_f);
      }
    }
  };
  auto fail = [&](int code) {
    *cta_abort = 1;
    if (p.ws != nullptr) p.ws->error = code;
  };

  if (tih == 0) {
    const uint32_t n0 = min(np, (uint32_t)kSlots);
    for (uint32_t f = 0; f < n0; ++f) issue_fill(f);
  }

  // ------------------------------- phase 1: per-tensor maximum -------------------------------
  float amax;
  if (!KNOWN) {
    float m = 0.0f;
    uint32_t s = 0, par = 0;
    uint16_t* tp = tab;                              // this lane's slot in the table of block maxima
    for (uint32_t c = 0; c < np; ++c) {
      if (!wait_phase(full0 + 8u * s, par, cta_abort, p.wait_limit_ns)) { fail(kErrCopy); break; }
      uint32_t w[2][8];
      const uint32_t addr = ring + s * kPairBytes;
      load_block(addr, w[0]);
      load_block(addr + kTileBytes, w[1]);               // the unused half of a last odd pair holds stale bytes
      const bool two = 2u * c + 1u < nt;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float a;
        if (RHT) {
          float v[16];
          expand<true>(w[e], sm, v);
          a = 0.0f;
#pragma unroll
          for (int j = 0; j < 16; ++j) a = fmaxf(a, fabsf(v[j]));
          a *= 0.25f;
        } else {
          a = amax_packed8(w[e]);
          if (c < (uint32_t)(kTabTiles / 2)) tp[e * kHalfThreads] = (uint16_t)(__float_as_uint(a) >> 16);
        }
        if (e == 0 || two) m = fmaxf(m, a);
      }
      tp += 2 * kHalfThreads;
      if (c + kSlots < np) release_and_refill(s, c + kSlots);      // not one of the last pairs: the slot takes pair c + kSlots
      if (++s == kSlots) { s = 0; par ^= 1u; }
    }
    if (stamper) p.ws->after[0] = (unsigned int)(global_ns() - t_start);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    if (lane == 0) red[tid >> 5] = m;
    __syncthreads();
    if (stamper) p.ws->after[1] = (unsigned int)(global_ns() - t_start);

    // ------------------------------- grid barrier -------------------------------
    if (tid < 32) {
      float mm = red[tid];
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 8));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 4));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 2));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 1));
      if (tid == 0) {
        const unsigned int slot = epoch & 1u;
        unsigned int* amax_word = reinterpret_cast<unsigned int*>(&p.ws->amax[slot]);
        // non-negative floats order like their bit patterns; the release on the arrival publishes the
        // maximum before it
        asm volatile("red.relaxed.gpu.global.max.u32 [%0], %1;" ::"l"(amax_word), "r"(__float_as_uint(mm)) : "memory");
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(&p.ws->arrived[slot]), "r"(1u) : "memory");
        const unsigned long long tb = global_ns();
        unsigned int seen;
        uint32_t spins = 0;
        do {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&p.ws->arrived[slot]) : "memory");
          if (seen >= gridDim.x + p.extra_arrivals) break;
          if ((++spins & 63u) == 0u && global_ns() - tb > p.wait_limit_ns) { fail(kErrBarrier); break; }
        } while (true);
        unsigned int amax_bits;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(amax_bits) : "l"(amax_word) : "memory");
        red[0] = __uint_as_float(amax_bits);                       // to the whole CTA through shared memory
        if (blockIdx.x == 0 && *cta_abort == 0) {
          // every CTA has read `epoch` (it did so before it arrived): prepare the next launch
          p.ws->amax[slot ^ 1u] = 0.0f;
          p.ws->arrived[slot ^ 1u] = 0u;
          p.ws->epoch = epoch + 1u;
        }
      }
    }
    __syncthreads();
    if (*cta_abort != 0) return;                  // every copy of phase 1 has landed or been given up on
    if (stamper) p.ws->after[2] = (unsigned int)(global_ns() - t_start);
    amax = red[0];
  } else {
    amax = __ldg(p.amax_in);
  }

  // ------------------------------- phase 2: quantize -------------------------------
  Scale sc;
  sc.pts = __fdiv_rn(fmaxf(amax, kAmaxFloor), kGlobalDiv);
  sc.inv_pts = __fdiv_rn(1.0f, sc.pts);
  sc.c = __fdiv_rn(1.0f, kF4Max * sc.pts);
  if (blockIdx.x == 0 && tid == 0 && p.pts_out != nullptr) *p.pts_out = sc.pts;
  if (tid < 128) recip_tab[tid] = __fdiv_rn(sc.inv_pts, e4m3_to_f32(tid));
  __syncthreads();

  // One pair of tiles from a ring slot: this lane's block (row row_t, block kb) of each.  k = position
  // of the pair's first tile in the half's range (block maxima of positions < kTabTiles are in the
  // table at tp); cur = where the first tile's block goes, left at the tile after the pair.
  auto quantize_pair = [&](uint32_t slot_addr, uint32_t k, const uint16_t* tp, Cursor& cur) {
    uint32_t w[2][8];
    load_block(slot_addr, w[0]);
    load_block(slot_addr + kTileBytes, w[1]);
    const bool two = k + 1u < nt;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      if (e == 1 && !two) break;
      float v[16];
      float amax_b;
      if (RHT) {
        expand<true>(w[e], sm, v);
        amax_b = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax_b = fmaxf(amax_b, fabsf(v[j]));
        amax_b *= 0.25f;                                   // H = butterfly / 4, an exact scaling
      } else {
        expand<false>(w[e], sm, v);
        amax_b = (!KNOWN && k < (uint32_t)kTabTiles) ? __uint_as_float((uint32_t)tp[e * kHalfThreads] << 16)
                                                     : amax_packed8(w[e]);
      }
      const uint32_t sf = block_scale_byte(amax_b, sc);
      const float recip = RHT ? recip_tab[sf] * 0.25f : recip_tab[sf];
      float d[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (RHT) mul2_poszero(v[2 * j], v[2 * j + 1], recip, d[2 * j], d[2 * j + 1]);
        else mul2(v[2 * j], v[2 * j + 1], recip, d[2 * j], d[2 * j + 1]);
      }
      uint32_t lo, hi;
      if (SR) {
        const Philox4 r = philox_rounds(cur.i, 0u, (uint32_t)p.offset, (uint32_t)(p.offset >> 32), p.keys);
        lo = e2m1x4_rs(d[0], d[1], d[2], d[3], r.x) | (e2m1x4_rs(d[4], d[5], d[6], d[7], r.y) << 16);
        hi = e2m1x4_rs(d[8], d[9], d[10], d[11], r.z) | (e2m1x4_rs(d[12], d[13], d[14], d[15], r.w) << 16);
      } else {
        lo = e2m1x8_rn(d);
        hi = e2m1x8_rn(d + 8);
      }
      if (cur.inside) *reinterpret_cast<uint2*>(cur.q) = make_uint2(lo, hi);
      // the scale tile is written whole: padding rows and columns read as zero
      *cur.s = cur.inside ? (uint8_t)sf : (uint8_t)0;
      cursor_step(cur, cc);
    }
  };

  const uint32_t first_fetch = KNOWN ? 0u : np;           // fill number of the first pair phase 2 fetches
  // (a) the pairs phase 1 left in the ring, in range order; each freed slot takes the next head pair
  {
    Cursor cur;
    cursor_set(cur, cc, t0 + 2u * head, p.qdata, p.q_pitch, q_lane, p.scales, sc_lane);
    const uint16_t* tp = tab + 2u * head * kHalfThreads;
    for (uint32_t j = 0; j < resident; ++j) {
      const uint32_t f = head + j, s = f % kSlots;          // it arrived as fill head + j of phase 1
      quantize_pair(ring + s * kPairBytes, 2u * f, tp, cur);
      tp += 2 * kHalfThreads;
      if (j < head) release_and_refill(s, f + kSlots);      // head pair j comes next into this slot (np = head + kSlots)
    }
  }
  // (b) the head of the range, fetched (again) through the ring
  {
    Cursor cur;
    cursor_set(cur, cc, t0, p.qdata, p.q_pitch, q_lane, p.scales, sc_lane);
    const uint16_t* tp = tab;
    uint32_t s = first_fetch % kSlots, par = (first_fetch / kSlots) & 1u;
    for (uint32_t q = 0; q < head; ++q) {
      if (!wait_phase(full0 + 8u * s, par, cta_abort, p.wait_limit_ns)) { fail(kErrCopy); break; }
      quantize_pair(ring + s * kPairBytes, 2u * q, tp, cur);
      tp += 2 * kHalfThreads;
      const uint32_t nq = q + kSlots;                       // the head pair this slot takes next
      if (nq < head) release_and_refill(s, first_fetch + nq);
      if (++s == kSlots) { s = 0; par ^= 1u; }
    }
  }
  if (tid == 0 && p.ws != nullptr) {                               // diagnostics only, nothing waits for them
    const unsigned long long t_end = global_ns();
    if (stamper) p.ws->after[3] = (unsigned int)(t_end - t_start);
    atomicMax(&p.ws->last_end, t_end);
  }
}

}  // namespace tiled
}  // namespace nvfp4

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
#include <mutex>

#include "gemm_common.cuh"      // encode_fn(): the driver's tensor-map encoder, looked up once

namespace nvfp4 {
namespace tiled {

namespace {
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int coop_ctas = 0;            // CTAs of the two-phase kernel the device keeps resident at once
};
std::mutex g_mutex;
DeviceInfo g_info[64];

const void* kernel_fn(bool sr, bool rht, bool known) {
#define NVFP4_TILED_FN(K_) \
  (sr ? (rht ? (const void*)quant_tiled_kernel<true, true, K_> : (const void*)quant_tiled_kernel<true, false, K_>) \
      : (rht ? (const void*)quant_tiled_kernel<false, true, K_> : (const void*)quant_tiled_kernel<false, false, K_>))
  return known ? NVFP4_TILED_FN(true) : NVFP4_TILED_FN(false);
#undef NVFP4_TILED_FN
}

int device_info(DeviceInfo& out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NVFP4_E_LAUNCH;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_info[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sm_count < 1)
      return NVFP4_E_LAUNCH;
    for (int sr = 0; sr < 2; ++sr)
      for (int rht = 0; rht < 2; ++rht)
        for (int known = 0; known < 2; ++known)
          if (cudaFuncSetAttribute(kernel_fn(sr, rht, known), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
              cudaSuccess) {
            cudaGetLastError();
            return NVFP4_E_LAUNCH;
          }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel_fn(true, true, false), kThreads, kSmemBytes) !=
        cudaSuccess) {
      cudaGetLastError();
      return NVFP4_E_LAUNCH;
    }
    d.coop_ctas = per_sm * d.sm_count;
    d.ready = true;
  }
  out = d;
  return NVFP4_OK;
}
}  // namespace

// amax_in == nullptr: the two-phase kernel (cooperative launch: its grid barrier needs every CTA
// resident) with the caller's workspace; otherwise one quantize pass with the given maximum, a plain
// launch.  Arguments have been validated by the caller (quantize_fused.cu).
int launch(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht, const float* signs16,
           uint64_t seed, uint64_t offset, uint8_t* qdata, uint8_t* scales, float* pts_out, void* workspace,
           const float* amax_in, unsigned long long wait_limit_ns, uint32_t extra_arrivals, uint64_t counter_pitch,
           uint64_t counter_base, cudaStream_t stream) {
  DeviceInfo info;
  const int irc = device_info(info);
  if (irc != NVFP4_OK) return irc;
  const bool known = amax_in != nullptr;
  if (!known && info.coop_ctas < 1) return NVFP4_E_LAUNCH;
  gemm::EncodeTiledFn encode = gemm::encode_fn();
  if (encode == nullptr) return NVFP4_E_DRIVER;
  CUtensorMap map;
  {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2u};
    cuuint32_t box[2] = {(cuuint32_t)kTileCols, (cuuint32_t)kTileRows};
    cuuint32_t estr[2] = {1u, 1u};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return NVFP4_E_DRIVER;
  }
  Params p;
  p.rows = (uint32_t)rows;
  p.bpr = (uint32_t)(cols / 16);
  p.ntc = (uint32_t)((cols + kTileCols - 1) / kTileCols);
  const uint64_t ntiles = (uint64_t)((rows + kTileRows - 1) / kTileRows) * p.ntc;
  if (ntiles >= (1ull << 31)) return NVFP4_E_LIMIT;
  p.ntiles = (uint32_t)ntiles;
  p.ctr_pitch = (uint32_t)counter_pitch;
  p.ctr_base = (uint32_t)counter_base;
  p.q_pitch = (uint64_t)(cols / 2);
  p.signs16 = signs16;
  for (int r = 0; r < 10; ++r) {
    p.keys.k[r][0] = (uint32_t)seed + (uint32_t)r * 0x9E3779B9u;
    p.keys.k[r][1] = (uint32_t)(seed >> 32) + (uint32_t)r * 0xBB67AE85u;
  }
  p.offset = offset;
  p.qdata = qdata;
  p.scales = scales;
  p.pts_out = pts_out;
  p.ws = static_cast<Workspace*>(workspace);
  p.amax_in = amax_in;
  p.wait_limit_ns = wait_limit_ns != 0 ? wait_limit_ns : kWaitLimitNs;
  p.extra_arrivals = extra_arrivals;
  uint32_t grid = (uint32_t)(known ? info.sm_count : (info.coop_ctas < info.sm_count ? info.coop_ctas : info.sm_count));
  const uint32_t want = (p.ntiles + 1u) / 2u;             // a tile per half CTA before more CTAs are used
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  const void* fn = kernel_fn(mode == NVFP4_ROUND_STOCHASTIC, rht != 0, known);
  void* args[] = {&map, &p};
  const cudaError_t e = known ? cudaLaunchKernel(fn, dim3(grid), dim3(kThreads), args, kSmemBytes, stream)
                              : cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), args, kSmemBytes, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();          // a refused launch must not show up as the next call's error
    return NVFP4_E_LAUNCH;
  }
  return NVFP4_OK;
}

}  // namespace tiled
}  // namespace nvfp4
