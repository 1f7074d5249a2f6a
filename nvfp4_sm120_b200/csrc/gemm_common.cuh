// Pieces shared by the one-CTA and the two-CTA NVFP4 GEMM kernels: PTX wrappers (mbarrier, TMA,
// tcgen05), descriptors, the parameter block and the host-side tensor-map encoding.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "nvfp4_b200.h"

namespace nvfp4 {
namespace gemm {

constexpr int kTileK = 256;                 // elements per K slice = 128 bytes per operand row
constexpr int kTmemCols = 512;
constexpr int kGroupM = 32;                 // row tiles per rasterization group (32 measured 1-3 % above 16, 8 below)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // a wait that lasts 2 s gives up (the default)

enum : int { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3, kErrScaleWait = 4 };

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
// The CTA keeps its abort flag (int) and, 8 bytes behind it, the wait limit in nanoseconds (the
// launch's Params::wait_limit_ns, written by thread 0 before the first wait) in shared memory.
__device__ __forceinline__ unsigned long long wait_limit_of(volatile int* abort_flag) {
  return *reinterpret_cast<volatile unsigned long long*>(const_cast<int*>(abort_flag) + 2);
}
__device__ __forceinline__ void set_wait_limit(volatile int* abort_flag, unsigned long long ns) {
  *reinterpret_cast<volatile unsigned long long*>(const_cast<int*>(abort_flag) + 2) = ns != 0 ? ns : kWaitLimitNs;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns(), limit = wait_limit_of(abort_flag);
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_ns() - t0 > limit) return false;
    }
  }
}
// The same for a long wait whose end is not urgent: sleeps between polls so that the waiting lane
// does not take issue slots from the warps of its scheduler that feed the tensor pipe.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns(), limit = wait_limit_of(abort_flag);
  for (uint32_t i = 1;; ++i) {
    __nanosleep(64);
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_ns() - t0 > limit) return false;
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
  int splits;        // > 1: K is split over `splits` CTAs per tile, which add their partial sums into
                     // a zeroed fp32 output with atomics (one-CTA kernel only)
  int tma_store;     // the output goes through shared memory and TMA stores (needs a 16-byte row pitch)
  unsigned long long wait_limit_ns;   // every bounded wait gives up after this long (0 = kWaitLimitNs)
  int drop_first_scale_arrival;       // test hook: the scale warps never announce K slice 0, so the MMA
                                      // issuer's first wait runs out and the kernel takes its abort path
  // NVFP4 output (out_fp4 != 0): d is the packed E2M1 buffer [M, N/2]; the bf16 rounding of every
  // output row is quantized in blocks of 16 along N with the per-tensor maximum *d_amax given
  uint8_t* d_sf;                      // swizzled E4M3 scales of the [M, N] operand
  const float* d_amax;
  int out_fp4;
  // optional: the kernel leaves max|D| over the stored output (after its rounding to the output type) in
  // this zeroed fp32 word, so that a quantizer reading D next needs no pass of its own to find it
  float* d_amax_out;
};

__device__ __forceinline__ void raise(volatile int* abort_flag, int32_t* status, int code) {
  *abort_flag = 1;
  if (status != nullptr) atomicCAS(status, 0, code);
}


// Running maximum of |D| over the elements this thread stores, kept as the bit pattern of a
// non-negative float (unsigned order = numeric order, and a NaN stays on top).  32 accumulator columns
// of one output row per call; rows and columns outside the matrix do not count.
__device__ __forceinline__ void track_amax(const Params& p, const uint32_t (&r)[32], float alpha, int64_t row,
                                           int64_t col, uint32_t& mbits) {
  if (row >= p.M) return;
  const int64_t left = p.N - col;
  const int n = left < 32 ? (int)left : 32;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float v = __uint_as_float(r[j]) * alpha;
    if (!p.out_f32) v = __bfloat162float(__float2bfloat16_rn(v));
    const uint32_t b = __float_as_uint(v) & 0x7fffffffu;
    if (j < n) mbits = max(mbits, b);
  }
}
// one atomic per warp and kernel
__device__ __forceinline__ void flush_amax(const Params& p, uint32_t mbits, int lane) {
  if (p.d_amax_out == nullptr) return;
  const uint32_t m = __reduce_max_sync(0xffffffffu, mbits);
  if (lane == 0 && m != 0u) atomicMax(reinterpret_cast<unsigned int*>(p.d_amax_out), m);
}

// 32 consecutive accumulator columns of one output row: scale by alpha, convert, store
// (vector stores when the chunk is whole and the leading dimension allows it).
// 16 consecutive values of one output row -> 8 bytes of E2M1 codes and the block's E4M3 scale byte, with
// the quantizer's own operations (nvfp4_gemm.py:36-45: true divisions, clamp, RNE) applied to the bf16
// rounding of the values, i.e. what quantizing the stored bf16 output with this maximum would give.
__device__ __forceinline__ void quantize_out_block(const uint32_t* acc, float alpha, float pts, float inv_pts,
                                                   uint32_t& lo, uint32_t& hi, uint32_t& sf) {
  float v[16];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[j]) * alpha));
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const float sbs = fminf(fmaxf(__fdiv_rn(__fdiv_rn(amax, kF4Max), pts), kE4M3Eps), kE4M3Max);
  sf = f32_to_e4m3(sbs);
  const float recip = __fdiv_rn(inv_pts, e4m3_to_f32(sf));
  lo = e2m1x2_rn(v[0] * recip, v[1] * recip) | (e2m1x2_rn(v[2] * recip, v[3] * recip) << 8) |
       (e2m1x2_rn(v[4] * recip, v[5] * recip) << 16) | (e2m1x2_rn(v[6] * recip, v[7] * recip) << 24);
  hi = e2m1x2_rn(v[8] * recip, v[9] * recip) | (e2m1x2_rn(v[10] * recip, v[11] * recip) << 8) |
       (e2m1x2_rn(v[12] * recip, v[13] * recip) << 16) | (e2m1x2_rn(v[14] * recip, v[15] * recip) << 24);
}

__device__ __forceinline__ void store_row_chunk(const Params& p, int64_t row, int64_t col, const uint32_t (&r)[32],
                                                float alpha) {
  const bool full = (col + 32 <= p.N);
  if (p.out_fp4) {                                      // N is a multiple of 16: a block is whole or absent
    const float pts = __fdiv_rn(fmaxf(__ldg(p.d_amax), kAmaxFloor), kGlobalDiv);
    const float inv_pts = __fdiv_rn(1.0f, pts);
    uint8_t* q = static_cast<uint8_t*>(p.d) + row * (p.N >> 1) + (col >> 1);
    const int64_t col_tiles = ((p.N >> 4) + 3) >> 2;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      if (col + 16 * b < p.N) {
        uint32_t sf;
        quantize_out_block(&r[16 * b], alpha, pts, inv_pts, w[2 * b], w[2 * b + 1], sf);
        p.d_sf[sf_offset(row, (col >> 4) + b, col_tiles)] = (uint8_t)sf;
      }
    }
    // a row of N / 2 bytes starts on an 8-byte boundary (N % 16 == 0), not always on a 16-byte one
    *reinterpret_cast<uint2*>(q) = make_uint2(w[0], w[1]);
    if (full) *reinterpret_cast<uint2*>(q + 8) = make_uint2(w[2], w[3]);
    return;
  }
  if (p.splits > 1) {                                   // split-K partial sum (fp32 output only)
    float* out = static_cast<float*>(p.d) + row * p.ldd + col;
    if (full && ((p.ldd & 3) == 0)) {                   // four floats per reduction instruction
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(out + j), "f"(__uint_as_float(r[j]) * alpha), "f"(__uint_as_float(r[j + 1]) * alpha),
                       "f"(__uint_as_float(r[j + 2]) * alpha), "f"(__uint_as_float(r[j + 3]) * alpha) : "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col + j < p.N) atomicAdd(out + j, __uint_as_float(r[j]) * alpha);
    }
    return;
  }
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


// ---- epilogue through shared memory and TMA stores -------------------------------------------
// A lane owns one accumulator row, so direct stores touch 32 different rows per instruction and the
// load/store unit spends one cycle per 32-byte sector.  Instead each warp lays 32 rows x 128 bytes
// out in shared memory in the 128-byte swizzle (conflict-free: the eight lanes of a quarter warp hit
// eight different 16-byte slots) and one lane hands the box to the TMA unit, which writes whole
// lines and clips at the matrix edge.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Drains accumulator columns [c_begin, c_end) (multiples of 64) of this warp's 32 TMEM lanes =
// output rows row0 .. row0 + 31.  `buf` is this warp's staging area: 4 KiB per box, a box being 64
// bf16 or 32 fp32 columns, 1024-byte aligned, not reused (so nothing waits until the end).
__device__ __forceinline__ void drain_through_tma(const Params& p, const CUtensorMap* map_d, uint32_t taddr,
                                                  uint8_t* buf, int64_t row0, int64_t n0, int c_begin, int c_end,
                                                  float alpha, int lane, uint32_t& mbits) {
  if (row0 >= p.M) return;                               // padded rows of a pair: nothing to write
  const uint32_t sw = (uint32_t)lane & 7u;
  int box = 0;
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    if (n0 + c0 >= p.N) break;                           // uniform across the warp
    uint32_t r[32];
    tc_ld_32x32b_x32(taddr + c0, r);
    tc_wait_ld();
    if (p.d_amax_out != nullptr) track_amax(p, r, alpha, row0 + lane, n0 + c0, mbits);
    uint8_t* rowp = buf + box * 4096 + lane * 128;
    bool box_done = true;
    int x = (int)(n0 + c0);
    if (p.out_f32) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(rowp + (((uint32_t)j ^ sw) << 4)) =
            make_float4(__uint_as_float(r[4 * j]) * alpha, __uint_as_float(r[4 * j + 1]) * alpha,
                        __uint_as_float(r[4 * j + 2]) * alpha, __uint_as_float(r[4 * j + 3]) * alpha);
    } else {
      const int half = ((c0 - c_begin) >> 5) & 1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * q]) * alpha,
                                                   __uint_as_float(r[8 * j + 2 * q + 1]) * alpha);
          w[q] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(rowp + (((uint32_t)(4 * half + j) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      box_done = half == 1 || c0 + 32 >= c_end || n0 + c0 + 32 >= p.N;
      x -= 32 * half;
    }
    if (box_done) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> TMA reads
      __syncwarp();
      if (lane == 0) tma_store_2d(map_d, smem_u32(buf + box * 4096), x, (int)row0);
      ++box;
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // before shared memory goes away
  __syncwarp();
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  // looked up once; the initialisation of a function-local static is thread-safe
  static const EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(sym);
    return nullptr;
  }();
  return fn;
}

// packed E2M1 operand [rows, K/2] bytes, K-major -> 2-D byte tensor map, box 128 bytes x box_rows
inline bool make_operand_map(CUtensorMap* map, const uint8_t* ptr, int64_t rows, int64_t k, int box_rows) {
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


// row-major output [M, ldd] -> 2-D tensor map for the epilogue's stores: boxes of 32 rows x 128 bytes
inline bool make_output_map(CUtensorMap* map, void* d, int64_t M, int64_t N, int64_t ldd, bool f32) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t elem = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)ldd * elem};
  cuuint32_t box[2] = {f32 ? 32u : 64u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  return fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemm
}  // namespace nvfp4
