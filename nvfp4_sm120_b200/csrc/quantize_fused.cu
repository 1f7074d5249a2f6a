// Single-launch NVFP4 quantizer for a row-major bf16 matrix, blocks along the columns (sm_100a).
//
// One persistent cooperative kernel, one CTA per SM, does what the two-launch path does:
//   phase 1  every CTA takes a contiguous range of 16-element blocks.  The tail of the range is
//            pulled into shared memory with bulk async copies (it stays there for phase 2), the
//            head is streamed with 128-bit loads; both feed the per-tensor |x| maximum (taken
//            after the Hadamard transform when that is on).
//   barrier  atomicMax into the workspace word, then a grid-wide arrive/wait on a counter
//            (bounded: a wait that lasts 2 s records an error in the workspace and returns).
//   phase 2  pts = amax / 2688 on the device; the blocks are quantized from shared memory
//            (no second HBM read) and, for the streamed head, from global memory, which the L2
//            still holds.  E4M3 scale bytes go straight to the 128x4-tiled layout.
// Arithmetic is the reference's (nvfp4_gemm.py:36-45).  Two exact shortcuts keep the kernel
// memory-bound: the block scale (amax_b/6)/pts is first formed as one multiply and accepted only
// when its E4M3 rounding provably equals that of the two true divisions (else those are done),
// and (1/pts)/scale comes from a 128-entry table built per CTA with true divisions.
#include <atomic>
#include <cstddef>
#include <cstdlib>
#include <mutex>

#include "quantize_common.cuh"

namespace nvfp4 {
namespace fused {

constexpr int kThreads = 1024;
constexpr int kChunkBytes = 16384;                 // one bulk copy
constexpr int kMaxChunks = 12;                     // 192 KiB of the range stay in shared memory
constexpr int kStashBytes = kChunkBytes * kMaxChunks;
constexpr int kTabBlocks = 16384;                  // block maxima of phase 1 kept for phase 2 (2 B each)
constexpr int kMiscOff = kStashBytes + 2 * kTabBlocks;
constexpr int kSmemBytes = kMiscOff + 1024;        // + reciprocal table, barrier, reduction scratch
constexpr int kBatch = 4;                          // blocks per thread in flight, amax pass
constexpr int kBatch2 = 2;                         // same, quantize pass (register budget: 64)

// KNOWN: the per-tensor maximum comes in (amax_in), so the kernel is the quantize pass alone; that
// variant runs 512 threads with 128 registers (the pass then streams from HBM and
// needs the bytes in flight: two register buffers of three blocks per thread in turn).
template <bool SR, bool RHT, bool KNOWN, int THREADS, int B2>
__global__ void __launch_bounds__(THREADS, 1)
quant_fused_kernel(const uint16_t* __restrict__ x, uint32_t rows, uint32_t blk_per_row, int64_t ld,
                   FastDiv div_bpr, const float* __restrict__ signs16, PhiloxKeys keys, uint64_t offset,
                   uint8_t* __restrict__ qdata, uint8_t* __restrict__ scales, float* __restrict__ pts_out,
                   Workspace* __restrict__ ws, uint32_t blocks_per_cta, int contiguous,
                   const float* __restrict__ amax_in, unsigned long long wait_limit_ns, uint32_t extra_arrivals) {
  // wait_limit_ns: after this long a bounded wait gives up.  extra_arrivals (test hook, normally 0):
  // the grid barrier expects that many arrivals more than there are CTAs, so it can only run out.
  // KNOWN: the caller knows the per-tensor maximum (a fused producer, or an all-reduce over a
  // sharded tensor): no first pass, no grid barrier, no workspace; one streaming quantize pass.
  constexpr bool known = KNOWN;
  extern __shared__ __align__(128) uint8_t smem[];
  uint16_t* amax_tab = reinterpret_cast<uint16_t*>(smem + kStashBytes);       // bf16 bits, no RHT only
  float* recip_tab = reinterpret_cast<float*>(smem + kMiscOff);               // 128 floats
  float* red = reinterpret_cast<float*>(smem + kMiscOff + 512);               // 32 floats
  float* sgs = reinterpret_cast<float*>(smem + kMiscOff + 640);               // 16 floats
  const uint32_t bar = smem_u32(smem + kMiscOff + 704);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + kMiscOff + 712);

  const uint32_t total = rows * blk_per_row;
  const uint32_t b0 = min(total, blockIdx.x * blocks_per_cta);
  const uint32_t b1 = min(total, b0 + blocks_per_cta);
  // tail of the range that lives in shared memory (contiguous inputs only)
  uint32_t stash_blocks = (contiguous && !known) ? min(b1 - b0, (uint32_t)(kStashBytes / 32)) : 0u;
  const uint32_t s0 = b1 - stash_blocks;                                      // first stashed block
  const uint32_t tid = threadIdx.x;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *cta_abort = 0;
    if (stash_blocks > 0) {
      const uint32_t bytes = stash_blocks * 32u;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      const uint8_t* src = reinterpret_cast<const uint8_t*>(x) + (size_t)s0 * 32;
      for (uint32_t o = 0; o < bytes; o += kChunkBytes) {
        const uint32_t n = min((uint32_t)kChunkBytes, bytes - o);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(smem + o)), "l"(src + o), "r"(n), "r"(bar) : "memory");
      }
    }
  }
  if (RHT && tid < 16) sgs[tid] = __ldg(signs16 + tid);
  const bool stamper = blockIdx.x == 0 && tid == 0 && ws != nullptr;
  unsigned long long t_start = 0;
  if (stamper) { t_start = global_ns(); ws->start = t_start; ws->last_end = 0ull; }
  // which of the two barrier slots this launch uses (needed only at the barrier: the load has all of
  // phase 1 to come back)
  unsigned int epoch = 0;
  if (tid == 0 && !known) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(&ws->epoch) : "memory");
  __syncthreads();
  uint32_t sm[8];                 // sign-bit masks of the packed bf16 pairs (bit 15: even, bit 31: odd)
#pragma unroll
  for (int j = 0; j < 8; ++j)
    sm[j] = RHT ? ((sgs[2 * j] < 0.0f ? 0x8000u : 0u) | (sgs[2 * j + 1] < 0.0f ? 0x80000000u : 0u)) : 0u;

  // ------------------------------- phase 1: per-tensor maximum -------------------------------
  float m = 0.0f;
  auto load_global = [&](uint32_t i, uint32_t (&w)[8]) {
    const uint32_t r = fast_div(i, div_bpr);
    const uint32_t kb = i - r * blk_per_row;
    const uint4* p = reinterpret_cast<const uint4*>(x + (int64_t)r * ld + (int64_t)kb * 16);
    const uint4 a = __ldg(p), b = __ldg(p + 1);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  };
  auto load_stash = [&](uint32_t i, uint32_t (&w)[8]) {
    const uint4* p = reinterpret_cast<const uint4*>(smem + (size_t)(i - s0) * 32);
    const uint4 a = p[0], b = p[1];
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  };
  auto block_max = [&](uint32_t i, const uint32_t (&w)[8]) {
    if (RHT) {
      float v[16];
      expand<true>(w, sm, v);
      float a = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; ++j) a = fmaxf(a, fabsf(v[j]));
      return a * 0.25f;
    }
    const float a = amax_packed8(w);
    if (i - b0 < (uint32_t)kTabBlocks) amax_tab[i - b0] = (uint16_t)(__float_as_uint(a) >> 16);
    return a;
  };
  // the streamed head, kBatch blocks per thread in flight before any of them is consumed
  for (uint32_t i = b0 + tid; i < s0 && !known; i += kBatch * THREADS) {
    uint32_t w[kBatch][8];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const uint32_t iu = min(i + u * THREADS, s0 - 1);     // clamped duplicates cost no extra traffic
      load_global(iu, w[u]);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) m = fmaxf(m, block_max(min(i + u * THREADS, s0 - 1), w[u]));
  }
  if (stamper) ws->after[0] = (unsigned int)(global_ns() - t_start);
  if (stash_blocks > 0) {
    bool landed = mbar_try_wait(bar, 0);
    if (!landed) {
      const unsigned long long t0 = global_ns();
      while (!(landed = mbar_try_wait(bar, 0))) {
        if (global_ns() - t0 > wait_limit_ns) break;
      }
    }
    if (!landed) { *cta_abort = 1; ws->error = 2; }
    for (uint32_t i = s0 + tid; i < b1; i += THREADS) {
      uint32_t w[8];
      load_stash(i, w);
      m = fmaxf(m, block_max(i, w));
    }
  }
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  if (stamper) ws->after[1] = (unsigned int)(global_ns() - t_start);

  // The first blocks of the quantize pass do not depend on the maximum: their loads (L2 hits by now)
  // go out before the barrier and are in registers when it opens.
  uint32_t pre[B2][8];
  const uint32_t i_first = b0 + tid;
  if (i_first < s0) {
#pragma unroll
    for (int u = 0; u < B2; ++u) load_global(min(i_first + u * THREADS, s0 - 1), pre[u]);
  }

  // ------------------------------- grid barrier -------------------------------
  if (known) {
    if (tid == 0) red[0] = __ldg(amax_in);
  } else if (tid < 32) {
    float mm = red[tid];
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 8));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 4));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 2));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 1));
    if (tid == 0) {
      const unsigned int slot = epoch & 1u;
      unsigned int* amax_word = reinterpret_cast<unsigned int*>(&ws->amax[slot]);
      // non-negative floats order like their bit patterns; the release on the arrival publishes the
      // maximum before it
      asm volatile("red.relaxed.gpu.global.max.u32 [%0], %1;" ::"l"(amax_word), "r"(__float_as_uint(mm)) : "memory");
      asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(&ws->arrived[slot]), "r"(1u) : "memory");
      const unsigned long long t0 = global_ns();
      unsigned int seen;
      uint32_t spins = 0;
      do {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&ws->arrived[slot]) : "memory");
        if (seen >= gridDim.x + extra_arrivals) break;
        if ((++spins & 63u) == 0u && global_ns() - t0 > wait_limit_ns) { *cta_abort = 1; ws->error = 1; break; }
      } while (true);
      unsigned int amax_bits;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(amax_bits) : "l"(amax_word) : "memory");
      red[0] = __uint_as_float(amax_bits);                       // to the whole CTA through shared memory
      if (blockIdx.x == 0 && *cta_abort == 0) {
        // every CTA has read `epoch` (it did so before it arrived): prepare the next launch
        ws->amax[slot ^ 1u] = 0.0f;
        ws->arrived[slot ^ 1u] = 0u;
        ws->epoch = epoch + 1u;
      }
    }
  }
  __syncthreads();
  if (*cta_abort != 0) return;
  if (stamper) ws->after[2] = (unsigned int)(global_ns() - t_start);

  // ------------------------------- phase 2: quantize -------------------------------
  Scale sc;
  {
    const float amax = red[0];
    sc.pts = __fdiv_rn(fmaxf(amax, kAmaxFloor), kGlobalDiv);
    sc.inv_pts = __fdiv_rn(1.0f, sc.pts);
    sc.c = __fdiv_rn(1.0f, kF4Max * sc.pts);
  }
  if (blockIdx.x == 0 && tid == 0 && pts_out != nullptr) *pts_out = sc.pts;
  if (tid < 128) recip_tab[tid] = __fdiv_rn(sc.inv_pts, e4m3_to_f32(tid));
  __syncthreads();
  const uint32_t col_tiles = (blk_per_row + 3) >> 2;

  auto quantize = [&](uint32_t i, const uint32_t (&w)[8]) {
    float v[16];
    float amax_b;
    if (RHT) {
      expand<true>(w, sm, v);
      amax_b = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; ++j) amax_b = fmaxf(amax_b, fabsf(v[j]));
      amax_b *= 0.25f;                                   // H = butterfly / 4, an exact scaling
    } else {
      expand<false>(w, sm, v);
      amax_b = (!known && i - b0 < (uint32_t)kTabBlocks) ? __uint_as_float((uint32_t)amax_tab[i - b0] << 16)
                                                         : amax_packed8(w);
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
      const Philox4 r = philox_rounds(i, 0u, (uint32_t)offset, (uint32_t)(offset >> 32), keys);
      lo = e2m1x4_rs(d[0], d[1], d[2], d[3], r.x) | (e2m1x4_rs(d[4], d[5], d[6], d[7], r.y) << 16);
      hi = e2m1x4_rs(d[8], d[9], d[10], d[11], r.z) | (e2m1x4_rs(d[12], d[13], d[14], d[15], r.w) << 16);
    } else {
      lo = e2m1x8_rn(d);
      hi = e2m1x8_rn(d + 8);
    }
    const uint32_t r = fast_div(i, div_bpr);
    const uint32_t kb = i - r * blk_per_row;
    *reinterpret_cast<uint2*>(qdata + (size_t)i * 8) = make_uint2(lo, hi);
    const uint32_t tile = (r >> 7) * col_tiles + (kb >> 2);
    scales[(size_t)tile * 512 + ((r & 31u) << 4) + (((r >> 5) & 3u) << 2) + (kb & 3u)] = (uint8_t)sf;
  };
  // the streamed head (first batch already loaded), then the stashed tail
  auto load_batch = [&](uint32_t i, uint32_t (&w)[B2][8]) {
#pragma unroll
    for (int u = 0; u < B2; ++u) load_global(min(i + u * THREADS, s0 - 1), w[u]);
  };
  auto quantize_batch = [&](uint32_t i, const uint32_t (&w)[B2][8]) {
#pragma unroll
    for (int u = 0; u < B2; ++u)
      if (i + u * THREADS < s0) quantize(i + u * THREADS, w[u]);
  };
  if (KNOWN) {
    // out of HBM: the loads of the next batch are in flight while this one is encoded (two register
    // buffers in turn; this variant has the registers for it)
    uint32_t nxt[B2][8];
    uint32_t i = i_first;
    while (i < s0) {
      uint32_t in = i + B2 * THREADS;
      if (in < s0) load_batch(in, nxt);
      quantize_batch(i, pre);
      i = in;
      if (i >= s0) break;
      in = i + B2 * THREADS;
      if (in < s0) load_batch(in, pre);
      quantize_batch(i, nxt);
      i = in;
    }
  } else {
    if (i_first < s0) quantize_batch(i_first, pre);
    for (uint32_t i = i_first + B2 * THREADS; i < s0; i += B2 * THREADS) {
      uint32_t w[B2][8];
      load_batch(i, w);
      quantize_batch(i, w);
    }
  }
  for (uint32_t i = s0 + tid; i < b1; i += THREADS) {
    uint32_t w[8];
    load_stash(i, w);
    quantize(i, w);
  }
  if (tid == 0 && ws != nullptr) {                               // diagnostics only, nothing waits for them
    const unsigned long long t_end = global_ns();
    if (stamper) ws->after[3] = (unsigned int)(t_end - t_start);
    atomicMax(&ws->last_end, t_end);
  }
}

static FastDiv make_fast_div(uint32_t d) {
  // Granlund-Montgomery for 31-bit dividends: with l = ceil(log2 d), mul = ceil(2^(31+l) / d) fits
  // 32 bits and n / d == mulhi(n, mul) >> (l - 1) for every n < 2^31.
  FastDiv f{0, 0, d};
  if (d == 1) return f;
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;
  f.mul = (uint32_t)(((1ull << (31 + l)) + d - 1) / d);
  f.shift = l - 1;
  return f;
}

}  // namespace fused
}  // namespace nvfp4

using namespace nvfp4;
using namespace nvfp4::fused;

extern "C" size_t nvfp4_quantize_fused_workspace_bytes(void) { return sizeof(Workspace); }

namespace {

constexpr int kThreadsKnown = 512, kBatchKnown = 3;
constexpr int kMaxDevices = 64;

// Per-device launch facts, looked up once under a lock (the entry points may be called from several
// host threads): SM count, the shared-memory attribute of every instantiation, and how many CTAs of
// the two-phase kernel the device keeps resident (its grid barrier needs all of them at once).
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int coop_ctas = 0;          // resident CTAs of the two-phase kernel over the whole device
};
std::mutex g_info_mutex;
DeviceInfo g_info[kMaxDevices];
// test hooks (nvfp4_test_hooks): wait limit of the next launches, surplus arrivals the barrier expects
std::atomic<unsigned long long> g_wait_ns{0};
std::atomic<unsigned int> g_extra_arrivals{0};

const void* fused_fn(bool sr, bool rht, bool known) {
#define NVFP4_FUSED_FN(K_, T_, B_) \
  (sr ? (rht ? (const void*)quant_fused_kernel<true, true, K_, T_, B_> : (const void*)quant_fused_kernel<true, false, K_, T_, B_>) \
      : (rht ? (const void*)quant_fused_kernel<false, true, K_, T_, B_> : (const void*)quant_fused_kernel<false, false, K_, T_, B_>))
  return known ? NVFP4_FUSED_FN(true, kThreadsKnown, kBatchKnown) : NVFP4_FUSED_FN(false, kThreads, kBatch2);
#undef NVFP4_FUSED_FN
}

int device_info(DeviceInfo& out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NVFP4_E_LAUNCH;
  std::lock_guard<std::mutex> lock(g_info_mutex);
  DeviceInfo& d = g_info[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sm_count < 1)
      return NVFP4_E_LAUNCH;
    for (int sr = 0; sr < 2; ++sr)
      for (int rht = 0; rht < 2; ++rht)
        for (int known = 0; known < 2; ++known)
          if (cudaFuncSetAttribute(fused_fn(sr, rht, known), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
              cudaSuccess) {
            cudaGetLastError();
            return NVFP4_E_LAUNCH;
          }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_fn(true, true, false), kThreads, kSmemBytes) !=
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
// resident) with the caller's workspace; otherwise one quantize pass with the given per-tensor
// maximum, a plain launch with no barrier and no workspace (it may share the device with other work).
namespace nvfp4 { namespace tiled {
int launch(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht, const float* signs16,
           uint64_t seed, uint64_t offset, uint8_t* qdata, uint8_t* scales, float* pts_out, void* workspace,
           const float* amax_in, unsigned long long wait_limit_ns, uint32_t extra_arrivals, uint64_t counter_pitch,
           uint64_t counter_base, cudaStream_t stream);
}}

static int launch_fused(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht,
                        const float* signs16, uint64_t seed, uint64_t offset, uint8_t* qdata, uint8_t* scales,
                        float* pts_out, void* workspace, const float* amax_in, cudaStream_t stream,
                        uint64_t counter_pitch = 0, uint64_t counter_base = 0) {
  // counter_pitch / counter_base: Philox counter of block (row, kb) = row * pitch + base + kb (a column
  // shard of a larger tensor numbers its blocks as the whole tensor does); 0 / 0 = the block's own index
  if (counter_pitch == 0) counter_pitch = (uint64_t)(cols / 16);
  const bool whole = counter_pitch == (uint64_t)(cols / 16) && counter_base == 0;
  // Kernel choice.  With the maximum given, the tile-form kernel (quantize_tiled.cu) is the faster one
  // (15.9 / 20.5 / 23.7 us against 19.8 / 22.2 / 24.6 us at 8192 x 4096 in the three modes); for the
  // two-phase launch the range-form kernel below is (26.6 / 30.1 / 35.5 us against 26.4 / 31.6 / 37.3).
  // NVFP4_QUANT_TILED = 0 / 1 forces one of them for both cases (measurements, tests).
  static const int force_tiled = []() { const char* e = getenv("NVFP4_QUANT_TILED"); return e == nullptr ? -1 : atoi(e); }();
  const bool use_tiled = (force_tiled < 0 ? amax_in != nullptr : force_tiled != 0) || !whole;
  if (use_tiled)
    return nvfp4::tiled::launch(x, rows, cols, ld, mode, rht, signs16, seed, offset, qdata, scales, pts_out, workspace,
                                amax_in, g_wait_ns.load(std::memory_order_relaxed),
                                g_extra_arrivals.load(std::memory_order_relaxed), counter_pitch, counter_base, stream);
  DeviceInfo info;
  const int irc = device_info(info);
  if (irc != NVFP4_OK) return irc;
  const bool sr = mode == NVFP4_ROUND_STOCHASTIC;
  const bool known = amax_in != nullptr;
  if (!known && info.coop_ctas < 1) return NVFP4_E_LAUNCH;
  const void* fn = fused_fn(sr, rht != 0, known);
  const int64_t sm = (rows + 127) / 128 * 128, sk = (cols / 16 + 3) / 4 * 4;
  if (sm != rows || sk != cols / 16) {
    if (cudaMemsetAsync(scales, 0, (size_t)(sm * sk), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  }

  uint32_t rows32 = (uint32_t)rows, bpr = (uint32_t)(cols / 16);
  const uint32_t total = rows32 * bpr;
  uint32_t grid = (uint32_t)(known ? info.sm_count : (info.coop_ctas < info.sm_count ? info.coop_ctas : info.sm_count));
  const uint32_t min_per_cta = 2048;                       // do not spread tiny tensors over all SMs
  if ((uint64_t)grid * min_per_cta > total) grid = (total + min_per_cta - 1) / min_per_cta;
  if (grid < 1) grid = 1;
  uint32_t per = (total + grid - 1) / grid;
  per = (per + 31u) & ~31u;                                // whole warps of blocks, 1 KiB-aligned ranges
  FastDiv fd = make_fast_div(bpr);
  int contiguous = (ld == cols) ? 1 : 0;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  Workspace* ws = static_cast<Workspace*>(workspace);
  PhiloxKeys keys;
  for (int r = 0; r < 10; ++r) {
    keys.k[r][0] = (uint32_t)seed + (uint32_t)r * 0x9E3779B9u;
    keys.k[r][1] = (uint32_t)(seed >> 32) + (uint32_t)r * 0xBB67AE85u;
  }
  unsigned long long wait_ns = g_wait_ns.load(std::memory_order_relaxed);
  if (wait_ns == 0) wait_ns = kWaitLimitNs;
  uint32_t extra = g_extra_arrivals.load(std::memory_order_relaxed);
  void* args[] = {&xp, &rows32, &bpr, &ld, &fd, &signs16, &keys, &offset, &qdata, &scales, &pts_out, &ws, &per,
                  &contiguous, &amax_in, &wait_ns, &extra};
  const cudaError_t e = known ? cudaLaunchKernel(fn, dim3(grid), dim3(kThreadsKnown), args, kSmemBytes, stream)
                              : cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), args, kSmemBytes, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();          // a refused launch must not show up as the next call's error
    return NVFP4_E_LAUNCH;
  }
  return NVFP4_OK;
}

namespace nvfp4 { namespace gemm { void set_test_hooks(unsigned long long wait_ns, int drop_arrival); } }

extern "C" int nvfp4_test_hooks(uint64_t wait_limit_ns, int quantizer_extra_arrivals, int gemm_drop_first_scale_arrival) {
  if (quantizer_extra_arrivals < 0 || quantizer_extra_arrivals > 1024) return NVFP4_E_MODE;
  g_wait_ns.store(wait_limit_ns, std::memory_order_relaxed);
  g_extra_arrivals.store((unsigned int)quantizer_extra_arrivals, std::memory_order_relaxed);
  nvfp4::gemm::set_test_hooks(wait_limit_ns, gemm_drop_first_scale_arrival != 0 ? 1 : 0);
  return NVFP4_OK;
}

static int check_fused_args(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht,
                            const float* signs16, const uint8_t* qdata, const uint8_t* scales) {
  if (!x || !qdata || !scales || (rht && !signs16)) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || (cols & 15) != 0) return NVFP4_E_SHAPE;
  if (rows * (cols / 16) >= (1ll << 31)) return NVFP4_E_LIMIT;
  if (mode != NVFP4_ROUND_NEAREST && mode != NVFP4_ROUND_STOCHASTIC) return NVFP4_E_MODE;
  auto mis = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (mis(x, 16) || (ld & 7) != 0 || mis(qdata, 16) || mis(scales, 16)) return NVFP4_E_ALIGN;
  return NVFP4_OK;
}

extern "C" int nvfp4_quantize_fused_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode,
                                         int rht, const float* signs16, uint64_t seed, uint64_t offset,
                                         uint8_t* qdata, uint8_t* scales, float* pts_out, void* workspace,
                                         size_t workspace_bytes, void* stream_) {
  if (!workspace) return NVFP4_E_NULL;
  if (workspace_bytes < sizeof(Workspace)) return NVFP4_E_WORKSPACE;
  const int rc = check_fused_args(x, rows, cols, ld, mode, rht, signs16, qdata, scales);
  if (rc != NVFP4_OK) return rc;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return NVFP4_E_ALIGN;
  return launch_fused(x, rows, cols, ld, mode, rht, signs16, seed, offset, qdata, scales, pts_out, workspace, nullptr,
                      static_cast<cudaStream_t>(stream_));
}

namespace nvfp4 { namespace fused {
// For nvfp4_quantize_bf16 (row-wise output, maximum given): the same kernel as one streaming pass.
// Returns NVFP4_E_LIMIT when this kernel does not take the case (the caller then uses its plain
// kernel).
int quantize_rows_known_amax(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht,
                             const float* signs16, const float* amax, uint64_t seed, uint64_t offset,
                             uint64_t counter_pitch, uint64_t counter_base,
                             uint8_t* qdata, uint8_t* scales, float* pts_out, cudaStream_t stream) {
  const int rc = check_fused_args(x, rows, cols, ld, mode, rht, signs16, qdata, scales);
  if (rc != NVFP4_OK) return rc;
  // the tile kernel keeps the counter in 32 bits: larger global indices go to the plain kernel
  if ((uint64_t)rows * counter_pitch + counter_base >= (1ull << 32)) return NVFP4_E_LIMIT;
  return launch_fused(x, rows, cols, ld, mode, rht, signs16, seed, offset, qdata, scales, pts_out, nullptr, amax,
                      stream, counter_pitch, counter_base);
}
}}

// ---------------------------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// Some users of this library reach it from places where a device allocation is not an option: a C
// or FFI binding running inside a host runtime that handed all of HBM to its own pool at start-up,
// or a callback in which the implicit synchronisation of cudaMalloc is not acceptable.  For them
// the 64-byte scratch of the single-launch quantizer lives in this file-scope device array instead
// of a caller-provided workspace.  Every GPU that loads the library holds these 256 bytes until the
// process exits.  All calls on a device share the array: calls that overlap on the GPU (different
// streams) race on it; calls on one stream do not.
static __device__ __align__(256) unsigned char g_static_scratch[256];

// Largest tensor the no-allocation entry point accepts: 2^31 - 1 blocks of 16 elements (the same
// bound the single-launch kernel has); the scratch itself does not grow with the tensor.
static constexpr long long kStaticMaxBlocks = (1ll << 31) - 1;

static std::mutex g_static_mutex;
static void* g_static_ptr[kMaxDevices] = {};

// Device address of the array on the current device.  The array's name is only a host-side handle
// here, so the address has to be asked for (once per device, with that device current) before it
// can be given to a kernel or a copy.
static int static_scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NVFP4_E_LAUNCH;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return NVFP4_E_LAUNCH;
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return NVFP4_OK;
}

extern "C" int nvfp4_quantize_static_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht,
                                          const float* signs16, uint64_t seed, uint64_t offset, uint8_t* qdata,
                                          uint8_t* scales, float* pts_out, void* stream_) {
  if (rows <= 0 || cols <= 0 || (cols & 15) != 0) return NVFP4_E_SHAPE;
  if (rows > kStaticMaxBlocks || (cols / 16) > kStaticMaxBlocks / rows) return NVFP4_E_LIMIT;
  void* ptr = nullptr;
  const int rc = static_scratch_address(&ptr);
  if (rc != NVFP4_OK) return rc;
  // The array keeps whatever the previous call (or one that gave up) left.  The two barrier slots
  // (the first 16 bytes) must start at zero and are cleared on the stream first; with both slots
  // clean the launch counter may hold anything.  The error word behind them is NOT cleared: it stays
  // set until nvfp4_quantize_static_status reads and clears it.  This is a memset, not an allocation.
  if (cudaMemsetAsync(ptr, 0, 16, static_cast<cudaStream_t>(stream_)) != cudaSuccess) return NVFP4_E_LAUNCH;
  return nvfp4_quantize_fused_bf16(x, rows, cols, ld, mode, rht, signs16, seed, offset, qdata, scales, pts_out, ptr,
                                   sizeof(Workspace), stream_);
}

extern "C" int nvfp4_quantize_static_status(int32_t* host_out, int clear, void* stream_) {
  if (host_out == nullptr) return NVFP4_E_NULL;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  void* ptr = nullptr;
  const int rc = static_scratch_address(&ptr);
  if (rc != NVFP4_OK) return rc;
  unsigned char* word = static_cast<unsigned char*>(ptr) + offsetof(Workspace, error);
  if (cudaMemcpyAsync(host_out, word, sizeof(int32_t), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      (clear && cudaMemsetAsync(word, 0, sizeof(int32_t), stream) != cudaSuccess) ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    cudaGetLastError();
    return NVFP4_E_LAUNCH;
  }
  return NVFP4_OK;
}
