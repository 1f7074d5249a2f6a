// Per-tensor amax and the fused NVFP4 quantizer for B200 (sm_100a).
//
// One pass computes, per 16-element block: [random-sign Hadamard] -> block amax -> E4M3 block
// scale -> E2M1 codes (round-to-nearest-even, or hardware stochastic rounding fed by a Philox
// stream) -> packed nibbles, and writes the scale byte straight to its place in the 128x4-tiled
// layout the tcgen05 block-scaled MMA reads.  The arithmetic follows the reference's pure-torch
// quantizer operation by operation (nvfp4_gemm.py:36-45): true fp32 divisions, no fast-math.
#include "quantize_common.cuh"

namespace nvfp4 {

using fused::PhiloxKeys;

// ---------------------------------------------------------------------------------------
// shared per-block arithmetic: that of the single-launch kernels (quantize_common.cuh) -- the block
// scale byte by the checked one-multiply shortcut, (1 / pts) / scale from a 128-entry table made with
// true divisions, Philox with host-made round keys -- so the bytes are the same and a block costs
// about 80 instructions less than with three true divisions and in-kernel key updates.
// ---------------------------------------------------------------------------------------
struct GlobalScale {
  fused::Scale sc;          // pts = amax / 2688, 1 / pts, 1 / (6 pts)
  const float* recip;       // shared memory: recip[b] = (1 / pts) / e4m3(b)
  float pts;
};

// Every thread of the CTA calls this (it holds a barrier); `tab` is 128 floats of shared memory.
__device__ __forceinline__ GlobalScale global_scale(const float* __restrict__ amax, float* tab) {
  GlobalScale g;
  g.sc.pts = __fdiv_rn(fmaxf(__ldg(amax), kAmaxFloor), kGlobalDiv);
  g.sc.inv_pts = __fdiv_rn(1.0f, g.sc.pts);
  g.sc.c = __fdiv_rn(1.0f, kF4Max * g.sc.pts);
  g.pts = g.sc.pts;
  g.recip = tab;
  if (threadIdx.x < 128) tab[threadIdx.x] = __fdiv_rn(g.sc.inv_pts, e4m3_to_f32(threadIdx.x));
  __syncthreads();
  return g;
}

inline PhiloxKeys make_philox_keys(uint64_t seed) {
  PhiloxKeys keys;
  for (int r = 0; r < 10; ++r) {
    keys.k[r][0] = (uint32_t)seed + (uint32_t)r * 0x9E3779B9u;
    keys.k[r][1] = (uint32_t)(seed >> 32) + (uint32_t)r * 0xBB67AE85u;
  }
  return keys;
}

// v[16] (already Hadamard-transformed if wanted) -> 8 bytes of codes (lo, hi) and the E4M3 byte.
__device__ __forceinline__ float block_amax16(const float (&v)[16]) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  return amax;
}

// amax: the maximum the block scale is derived from -- the block's own (1 x 16 scaling), or that of
// the 16 x 16 tile around it (2-D weight scaling, nvfp4_validate.py:68-82)
template <bool SR>
__device__ __forceinline__ void encode_block_scaled(const float (&v)[16], float amax, const GlobalScale& g,
                                                    uint64_t blk_index, const PhiloxKeys& keys, uint64_t offset,
                                                    uint32_t& lo, uint32_t& hi, uint32_t& sf_byte) {
  sf_byte = fused::block_scale_byte(amax, g.sc);                   // nvfp4_gemm.py:39-40
  const float recip = g.recip[sf_byte];                            // :41
  // the clamp to +-6 of :42 is the saturation of the conversions below
  if (SR) {
    const Philox4 r = fused::philox_rounds((uint32_t)blk_index, (uint32_t)(blk_index >> 32),
                                           (uint32_t)offset, (uint32_t)(offset >> 32), keys);
    const uint32_t q0 = e2m1x4_rs(v[0] * recip, v[1] * recip, v[2] * recip, v[3] * recip, r.x);
    const uint32_t q1 = e2m1x4_rs(v[4] * recip, v[5] * recip, v[6] * recip, v[7] * recip, r.y);
    const uint32_t q2 = e2m1x4_rs(v[8] * recip, v[9] * recip, v[10] * recip, v[11] * recip, r.z);
    const uint32_t q3 = e2m1x4_rs(v[12] * recip, v[13] * recip, v[14] * recip, v[15] * recip, r.w);
    lo = q0 | (q1 << 16);
    hi = q2 | (q3 << 16);
  } else {
    float d[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) d[j] = v[j] * recip;
    lo = fused::e2m1x8_rn(d);
    hi = fused::e2m1x8_rn(d + 8);
  }
}

template <bool SR>
__device__ __forceinline__ void encode_block(const float (&v)[16], const GlobalScale& g,
                                             uint64_t blk_index, const PhiloxKeys& keys, uint64_t offset,
                                             uint32_t& lo, uint32_t& hi, uint32_t& sf_byte) {
  encode_block_scaled<SR>(v, block_amax16(v), g, blk_index, keys, offset, lo, hi, sf_byte);
}

__device__ __forceinline__ void load_signs(const float* __restrict__ signs16, float (&sg)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 s = __ldg(reinterpret_cast<const float4*>(signs16) + i);
    sg[4 * i] = s.x; sg[4 * i + 1] = s.y; sg[4 * i + 2] = s.z; sg[4 * i + 3] = s.w;
  }
}

__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  // non-negative floats order like their bit patterns
  atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Maximum of a non-negative per-thread value over the CTA, then ONE atomic per CTA: same-address atomics
// from every warp serialise in the L2 (19 000 of them cost 25 us, more than reading 64 MiB does).
// Every thread of the CTA calls this; `slot` selects one of two independent reductions.
__device__ __forceinline__ void cta_max_to(float* addr, float v, int slot = 0) {
  __shared__ float part[2][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (lane == 0) part[slot][warp] = v;
  __syncthreads();
  if (warp == 0) {
    float m = lane < nwarps ? part[slot][lane] : 0.0f;
    m = warp_max(m);
    if (lane == 0 && !(m == 0.0f)) atomic_max_nonneg(addr, m);
  }
}

// ---------------------------------------------------------------------------------------
// amax kernels
// ---------------------------------------------------------------------------------------
// plain |x| maximum: 16-byte loads, max taken on the bf16 bit patterns (sign cleared)
__global__ void __launch_bounds__(512) amax_plain_kernel(const uint16_t* __restrict__ x, int64_t rows,
                                                         int vec_per_row, int64_t ld,
                                                         float* __restrict__ amax) {
  const int64_t total = rows * vec_per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  uint32_t m = 0;
  auto fold = [&](const uint4& q) {
    const uint32_t k = 0x7fff7fffu;
    const uint32_t a = __vimax3_u16x2(q.x & k, q.y & k, q.z & k);
    m = __vimax3_u16x2(a, q.w & k, m);                 // both 16-bit halves of m carry a running maximum
  };
  const bool flat = ld == (int64_t)vec_per_row * 8;      // contiguous rows: no division per load
  auto load = [&](int64_t i) {
    if (flat) return __ldg(reinterpret_cast<const uint4*>(x) + i);
    const int64_t r = i / vec_per_row;
    const int cv = (int)(i - r * vec_per_row);
    return __ldg(reinterpret_cast<const uint4*>(x + r * ld) + cv);
  };
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // four 16-byte loads per thread in flight: one per thread leaves the memory system half idle
  for (; i + 3 * stride < total; i += 4 * stride) {
    const uint4 q0 = load(i), q1 = load(i + stride), q2 = load(i + 2 * stride), q3 = load(i + 3 * stride);
    fold(q0); fold(q1); fold(q2); fold(q3);
  }
  for (; i < total; i += stride) fold(load(i));
  m = max(m & 0xffffu, m >> 16);
  cta_max_to(amax, __uint_as_float(m << 16));
}

// maximum after the Hadamard transform, blocks along the columns: one thread per block
__global__ void __launch_bounds__(256) amax_rht_rows_kernel(const uint16_t* __restrict__ x,
                                                            int64_t rows, int blk_per_row, int64_t ld,
                                                            const float* __restrict__ signs16,
                                                            float* __restrict__ amax) {
  float sg[16];
  load_signs(signs16, sg);
  const int64_t total = rows * blk_per_row;
  float m = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / blk_per_row;
    const int kb = (int)(i - r * blk_per_row);
    const uint4* p = reinterpret_cast<const uint4*>(x + r * ld + (int64_t)kb * 16);
    const uint4 a = __ldg(p), b = __ldg(p + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = bf16_lo(w[j]) * sg[2 * j];
      v[2 * j + 1] = bf16_hi(w[j]) * sg[2 * j + 1];
    }
    hadamard16_inplace(v);
#pragma unroll
    for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(v[j]));
  }
  cta_max_to(amax, m);
}

// ---------------------------------------------------------------------------------------
// quantizer, blocks along the columns (output describes x itself)
// ---------------------------------------------------------------------------------------
template <bool SR, bool RHT>
__global__ void __launch_bounds__(256) quant_rows_kernel(const uint16_t* __restrict__ x, int64_t rows,
                                                         int blk_per_row, int64_t ld,
                                                         const float* __restrict__ signs16,
                                                         const float* __restrict__ amax,
                                                         const PhiloxKeys keys, uint64_t offset,
                                                         uint8_t* __restrict__ qdata,
                                                         uint8_t* __restrict__ scales,
                                                         float* __restrict__ pts_out,
                                                         uint64_t ctr_pitch, uint64_t ctr_base) {
  // Philox counter of block (row, kb) = row * ctr_pitch + ctr_base + kb: the block's index in the
  // whole tensor when x is a column shard of it (pitch = blocks per row of the whole tensor)
  __shared__ float recip_tab[128];
  const GlobalScale g = global_scale(amax, recip_tab);
  if (blockIdx.x == 0 && threadIdx.x == 0 && pts_out != nullptr) *pts_out = g.pts;
  float sg[16];
  if (RHT) load_signs(signs16, sg);
  const int64_t total = rows * blk_per_row;
  const int64_t col_tiles = (blk_per_row + 3) >> 2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / blk_per_row;
    const int kb = (int)(i - r * blk_per_row);
    const uint4* p = reinterpret_cast<const uint4*>(x + r * ld + (int64_t)kb * 16);
    const uint4 a = __ldg(p), b = __ldg(p + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = bf16_lo(w[j]);
      v[2 * j + 1] = bf16_hi(w[j]);
    }
    if (RHT) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= sg[j];
      hadamard16_inplace(v);
    }
    uint32_t lo, hi, sf;
    encode_block<SR>(v, g, (uint64_t)r * ctr_pitch + ctr_base + (uint64_t)kb, keys, offset, lo, hi, sf);
    *reinterpret_cast<uint2*>(qdata + i * 8) = make_uint2(lo, hi);
    scales[sf_offset(r, kb, col_tiles)] = (uint8_t)sf;
  }
}

// ---------------------------------------------------------------------------------------
// transposing variants: blocks along the ROWS of x; the output describes x^T [cols, rows].
// A thread owns two adjacent columns and up to 64 consecutive rows (four 16-row blocks), so
// that a warp reads 128 contiguous bytes per row and each thread writes 32 contiguous output
// bytes per column.
// ---------------------------------------------------------------------------------------
// The 16-point butterfly of two adjacent columns at once: (v0[i], v1[i]) ride in the two lanes of the
// packed fp32 add / sub / fma, half the instructions of two scalar butterflies and the same bits
// (same operations in the same order as hadamard16_inplace, exact zeros made +0).
__device__ __forceinline__ void hadamard16_pair(float (&v0)[16], float (&v1)[16]) {
#pragma unroll
  for (int s = 1; s < 16; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & s) == 0) fused::addsub2(v0[i], v1[i], v0[i | s], v1[i | s]);
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) fused::mul2_poszero(v0[i], v1[i], 0.25f, v0[i], v1[i]);
}

// sign-bit masks of the 16 rows for a packed bf16 pair (both halves of a word belong to one row)
__device__ __forceinline__ void sign_masks(const float (&sg)[16], uint32_t (&sm)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) sm[i] = sg[i] < 0.0f ? 0x80008000u : 0u;
}

template <bool RHT>
__device__ __forceinline__ void load_col_pair_block(const uint16_t* __restrict__ x, int64_t ld,
                                                    int64_t r0, int64_t c, const uint32_t (&sm)[16],
                                                    float (&v0)[16], float (&v1)[16]) {
  const uint32_t* p = reinterpret_cast<const uint32_t*>(x + r0 * ld + c);
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = __ldg(p + (size_t)i * (size_t)(ld >> 1));
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t u = RHT ? (w[i] ^ sm[i]) : w[i];      // times +-1 = a flip of the sign bit
    v0[i] = bf16_lo(u);
    v1[i] = bf16_hi(u);
  }
  if (RHT) hadamard16_pair(v0, v1);
}

__global__ void __launch_bounds__(256) amax_rht_cols_kernel(const uint16_t* __restrict__ x, int64_t rows,
                                                            int64_t cols, int64_t ld,
                                                            const float* __restrict__ signs16,
                                                            float* __restrict__ amax) {
  float sg[16];
  load_signs(signs16, sg);
  uint32_t sm[16];
  sign_masks(sg, sm);
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  const int64_t r_base = (int64_t)blockIdx.y * 64;
  float m = 0.0f;
  if (c < cols) {
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const int64_t r0 = r_base + 16 * j;
      if (r0 >= rows) break;
      float v0[16], v1[16];
      load_col_pair_block<true>(x, ld, r0, c, sm, v0, v1);
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
    }
  }
  cta_max_to(amax, m);
}

template <bool SR, bool RHT>
__global__ void __launch_bounds__(256) quant_cols_kernel(const uint16_t* __restrict__ x, int64_t rows,
                                                         int64_t cols, int64_t ld,
                                                         const float* __restrict__ signs16,
                                                         const float* __restrict__ amax,
                                                         const PhiloxKeys keys, uint64_t offset,
                                                         uint8_t* __restrict__ qdata,
                                                         uint8_t* __restrict__ scales,
                                                         float* __restrict__ pts_out,
                                                         uint64_t ctr_pitch, uint64_t ctr_base) {
  // Philox counter of output block (column c, row block kb) = c * ctr_pitch + ctr_base + kb
  __shared__ float recip_tab[128];
  const GlobalScale g = global_scale(amax, recip_tab);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && pts_out != nullptr) *pts_out = g.pts;
  uint32_t sm[16];
  if (RHT) {
    float sg[16];
    load_signs(signs16, sg);
    sign_masks(sg, sm);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) sm[i] = 0u;
  }
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= cols) return;
  const int64_t r_base = (int64_t)blockIdx.y * 64;
  const int64_t blk_per_orow = rows >> 4;            // blocks per OUTPUT row (K = rows)
  const int64_t col_tiles = (blk_per_orow + 3) >> 2;
  const int64_t out_ld = rows >> 1;                  // bytes per output row
  uint32_t q[2][8];
  uint32_t sfw[2] = {0u, 0u};
  int nvalid = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r0 = r_base + 16 * j;
    if (r0 < rows) {
      float v0[16], v1[16];
      load_col_pair_block<RHT>(x, ld, r0, c, sm, v0, v1);
      const uint64_t kb = (uint64_t)(r0 >> 4);
      uint32_t sf0, sf1;
      encode_block<SR>(v0, g, (uint64_t)c * ctr_pitch + ctr_base + kb, keys, offset, q[0][2 * j], q[0][2 * j + 1], sf0);
      encode_block<SR>(v1, g, (uint64_t)(c + 1) * ctr_pitch + ctr_base + kb, keys, offset, q[1][2 * j], q[1][2 * j + 1], sf1);
      sfw[0] |= sf0 << (8 * j);
      sfw[1] |= sf1 << (8 * j);
      nvalid = j + 1;
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint8_t* orow = qdata + (c + h) * out_ld + (r_base >> 1);
    const size_t so = sf_offset(c + h, r_base >> 4, col_tiles);
    if (nvalid == 4 && (out_ld & 15) == 0) {
      reinterpret_cast<uint4*>(orow)[0] = make_uint4(q[h][0], q[h][1], q[h][2], q[h][3]);
      reinterpret_cast<uint4*>(orow)[1] = make_uint4(q[h][4], q[h][5], q[h][6], q[h][7]);
      *reinterpret_cast<uint32_t*>(scales + so) = sfw[h];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < nvalid) {
          *reinterpret_cast<uint2*>(orow + 8 * j) = make_uint2(q[h][2 * j], q[h][2 * j + 1]);
          scales[so + j] = (uint8_t)(sfw[h] >> (8 * j));
        }
      }
    }
  }
}


// ---------------------------------------------------------------------------------------
// Wide form of the column MAXIMUM kernels for 16-byte rows (cols % 8 == 0).  The narrow kernels above read
// 128 contiguous bytes of a row per warp instruction; here a CTA takes tiles of 16 rows x 512 columns
// the way the activation kernels do (csrc/swiglu.cu): thread t and step k load the eight columns
// 8 * (t % 64) of row 4k + t / 64 with one 16-byte load (a warp moves 512 contiguous bytes of a row),
// the tile goes to padded shared memory, and thread t then reads its two columns of all 16 rows from
// there (consecutive lanes, consecutive banks), with the next tile's loads in flight.  Measured on a
// B200 at 4096 x 4096: both maxima 14.9 us against 17.1 us.  The same staging for the quantizer itself
// was slower (116 us against 89.5 us at 4096 x 28672, RHT + stochastic): its long encode phase leaves
// only the four prefetch loads per thread in flight, so quant_cols_kernel keeps its direct loads.
// ---------------------------------------------------------------------------------------
constexpr int kWideCols = 512;
constexpr int kWidePitch = kWideCols / 2 + 4;            // 32-bit words per tile row, padded

struct WideTile {
  int64_t c0, r_base, c;        // first column of the CTA, first row of its 64, this thread's column pair
  int cc, lr;                   // load role: eight columns at cc, row 4k + lr of a tile
  bool col_in, mine;
};
__device__ __forceinline__ WideTile wide_tile(int64_t cols) {
  WideTile t;
  t.c0 = (int64_t)blockIdx.x * kWideCols;
  t.r_base = (int64_t)blockIdx.y * 64;
  t.cc = (threadIdx.x & 63) * 8;
  t.lr = threadIdx.x >> 6;
  t.col_in = t.c0 + t.cc < cols;
  t.c = t.c0 + 2 * (int64_t)threadIdx.x;
  t.mine = t.c < cols;
  return t;
}
__device__ __forceinline__ void wide_fetch(const uint16_t* __restrict__ x, int64_t rows, int64_t ld, const WideTile& t,
                                           int j, uint4 (&d)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t r = t.r_base + 16 * j + 4 * k + t.lr;
    d[k] = (t.col_in && r < rows) ? __ldg(reinterpret_cast<const uint4*>(x + r * ld + t.c0 + t.cc))
                                  : make_uint4(0u, 0u, 0u, 0u);
  }
}
__device__ __forceinline__ void wide_stage(uint32_t* tile, const WideTile& t, const uint4 (&d)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(&tile[(4 * k + t.lr) * kWidePitch + (t.cc >> 1)]) = d[k];
}

// BOTH: maxima2[0] = plain maximum as well (else only maxima2[0] = maximum after the transform)
template <bool BOTH>
__global__ void __launch_bounds__(256) amax_cols_wide_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols,
                                                             int64_t ld, const float* __restrict__ signs16,
                                                             float* __restrict__ out) {
  __shared__ __align__(16) uint32_t tile[16 * kWidePitch];
  float sg[16];
  load_signs(signs16, sg);
  uint32_t sm[16];
  sign_masks(sg, sm);
  const WideTile t = wide_tile(cols);
  float m = 0.0f;
  uint32_t mp = 0u;
  uint4 nxt[4];
  wide_fetch(x, rows, ld, t, 0, nxt);
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    if (t.r_base + 16 * j >= rows) break;                  // uniform over the CTA
    wide_stage(tile, t, nxt);
    if (BOTH) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t kk = 0x7fff7fffu;
        mp = __vimax3_u16x2(mp, nxt[k].x & kk, nxt[k].y & kk);
        mp = __vimax3_u16x2(mp, nxt[k].z & kk, nxt[k].w & kk);
      }
    }
    if (j + 1 < 4) wide_fetch(x, rows, ld, t, j + 1, nxt);
    __syncthreads();
    if (t.mine) {
      float v0[16], v1[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t u = tile[i * kWidePitch + threadIdx.x] ^ sm[i];
        v0[i] = bf16_lo(u);
        v1[i] = bf16_hi(u);
      }
      hadamard16_pair(v0, v1);
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
    }
    __syncthreads();
  }
  if (BOTH) {
    mp = max(mp & 0xffffu, mp >> 16);
    cta_max_to(out, __uint_as_float(mp << 16), 0);
    cta_max_to(out + 1, m, 1);
  } else {
    cta_max_to(out, m);
  }
}

// ---------------------------------------------------------------------------------------
// weights: both layouts from one read.  A CTA takes a 64 x 64 tile of w [rows, cols]; thread
// (row t / 4, segment t % 4) loads the 16 elements of row-wise block (row, segment) and leaves them in
// a padded shared tile, from which thread (column t % 64, row block t / 64) reads the 16 elements of
// column-wise block (column, row block).  Round to nearest only (weights).  TWO_D: one scale per
// 16 x 16 tile, shared by the row-wise and the column-wise blocks that cross it, so that both
// quantized layouts hold the same values (the reference simulator's weight scaling,
// nvfp4_validate.py:68-82); otherwise every block has its own 1 x 16 scale, as quant_nvfp4 gives.
// ---------------------------------------------------------------------------------------
template <bool TWO_D>
__global__ void __launch_bounds__(256) quant_weight_dual_kernel(const uint16_t* __restrict__ w, int64_t rows, int64_t cols,
                                                                int64_t ld, const float* __restrict__ amax,
                                                                uint8_t* __restrict__ q_rows, uint8_t* __restrict__ sf_rows,
                                                                uint8_t* __restrict__ q_cols, uint8_t* __restrict__ sf_cols,
                                                                float* __restrict__ pts_out) {
  __shared__ uint16_t tile[64][66];          // 33 words per row: a column walk touches 16 different banks
  __shared__ float bmax[64][4];              // row-wise block maxima of the tile
  __shared__ float tmax[4][4];               // 16 x 16 tile maxima
  __shared__ float recip_tab[128];
  const GlobalScale g = global_scale(amax, recip_tab);
  const PhiloxKeys keys{};                   // round to nearest: unused
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && pts_out != nullptr) *pts_out = g.pts;
  const int t = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  // ---- load: row-wise block (r, seg) ----
  const int r = t >> 2, seg = t & 3;
  const int64_t gr = r0 + r, gc = c0 + seg * 16;
  const bool have = gr < rows && gc < cols;          // rows and cols are multiples of 16: a block is whole or absent
  uint32_t wv[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (have) {
    const uint4* p = reinterpret_cast<const uint4*>(w + gr * ld + gc);
    const uint4 a = __ldg(p), b = __ldg(p + 1);
    wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
  }
  float v[16];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[2 * j] = bf16_lo(wv[j]);
    v[2 * j + 1] = bf16_hi(wv[j]);
    *reinterpret_cast<uint32_t*>(&tile[r][seg * 16 + 2 * j]) = wv[j];
  }
  const float my_max = block_amax16(v);
  if (TWO_D) bmax[r][seg] = my_max;
  __syncthreads();
  if (TWO_D) {
    if (t < 16) {
      const int rb = t >> 2, cb = t & 3;
      float m = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, bmax[rb * 16 + i][cb]);
      tmax[rb][cb] = m;
    }
    __syncthreads();
  }
  // ---- row-wise output ----
  if (have) {
    uint32_t lo, hi, sf;
    encode_block_scaled<false>(v, TWO_D ? tmax[r >> 4][seg] : my_max, g, 0, keys, 0, lo, hi, sf);
    const int64_t kb = gc >> 4;
    *reinterpret_cast<uint2*>(q_rows + gr * (cols >> 1) + kb * 8) = make_uint2(lo, hi);
    sf_rows[sf_offset(gr, kb, ((cols >> 4) + 3) >> 2)] = (uint8_t)sf;
  }
  // ---- column-wise output: block (column c, row block rb) ----
  const int c = t & 63, rb = t >> 6;
  const int64_t oc = c0 + c, orow0 = r0 + rb * 16;
  if (oc < cols && orow0 < rows) {
    float u[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) u[i] = __uint_as_float((uint32_t)tile[rb * 16 + i][c] << 16);
    uint32_t lo, hi, sf;
    encode_block_scaled<false>(u, TWO_D ? tmax[rb][c >> 4] : block_amax16(u), g, 0, keys, 0, lo, hi, sf);
    const int64_t kb = orow0 >> 4;
    *reinterpret_cast<uint2*>(q_cols + oc * (rows >> 1) + kb * 8) = make_uint2(lo, hi);
    sf_cols[sf_offset(oc, kb, ((rows >> 4) + 3) >> 2)] = (uint8_t)sf;
  }
}


// ---------------------------------------------------------------------------------------
// activations and gradients: both layouts from one read.  Every operand of FP4Linear is needed
// twice: x row-wise for fprop and x^T (Hadamard along the tokens) for wgrad, dY row-wise
// (stochastic) for dgrad and dY^T (Hadamard + stochastic) for wgrad (nvfp4_train.py:36-55).  Same
// 64 x 64 tiling as the weight kernel above: thread (row t / 4, segment t % 4) encodes row-wise
// block (row, segment) with the plain maximum, then thread (column t % 64, row block t / 64) reads
// its 16 rows of one column from the shared tile, applies the random-sign Hadamard along the rows
// and encodes the column-wise block with the maximum of the transformed tensor.  Each layout has
// its own per-tensor maximum, seed and Philox counter (counter of a block = its index in the whole
// tensor of that layout: out_row * pitch + base + k_block), so the bytes are those of the two
// separate quantizations.
// ---------------------------------------------------------------------------------------
struct DualCounters { uint64_t pitch_r, base_r, pitch_c, base_c; };

template <bool SR_R, bool SR_C>
__global__ void __launch_bounds__(256) quant_act_dual_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols,
                                                             int64_t ld, const float* __restrict__ signs16,
                                                             const float* __restrict__ amax_r,
                                                             const float* __restrict__ amax_c, const PhiloxKeys keys_r,
                                                             const PhiloxKeys keys_c, uint64_t offset, DualCounters ctr,
                                                             uint8_t* __restrict__ q_rows, uint8_t* __restrict__ sf_rows,
                                                             float* __restrict__ pts_r, uint8_t* __restrict__ q_cols,
                                                             uint8_t* __restrict__ sf_cols, float* __restrict__ pts_c) {
  __shared__ uint16_t tile[64][66];          // 33 words per row: a column walk touches 16 different banks
  __shared__ float recip_r[128], recip_c[128];
  const GlobalScale g_r = global_scale(amax_r, recip_r), g_c = global_scale(amax_c, recip_c);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
    if (pts_r != nullptr) *pts_r = g_r.pts;
    if (pts_c != nullptr) *pts_c = g_c.pts;
  }
  const int t = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  const int r = t >> 2, seg = t & 3;
  const int64_t gr = r0 + r, gc = c0 + seg * 16;
  const bool have = gr < rows && gc < cols;          // rows and cols are multiples of 16: a block is whole or absent
  uint32_t wv[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (have) {
    const uint4* p = reinterpret_cast<const uint4*>(x + gr * ld + gc);
    const uint4 a = __ldg(p), b = __ldg(p + 1);
    wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) *reinterpret_cast<uint32_t*>(&tile[r][seg * 16 + 2 * j]) = wv[j];
  if (have) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = bf16_lo(wv[j]);
      v[2 * j + 1] = bf16_hi(wv[j]);
    }
    uint32_t lo, hi, sf;
    const int64_t kb = gc >> 4;
    encode_block<SR_R>(v, g_r, (uint64_t)gr * ctr.pitch_r + ctr.base_r + (uint64_t)kb, keys_r, offset, lo, hi, sf);
    *reinterpret_cast<uint2*>(q_rows + gr * (cols >> 1) + kb * 8) = make_uint2(lo, hi);
    sf_rows[sf_offset(gr, kb, ((cols >> 4) + 3) >> 2)] = (uint8_t)sf;
  }
  __syncthreads();
  const int c = t & 63, rb = t >> 6;
  const int64_t oc = c0 + c, orow0 = r0 + rb * 16;
  if (oc < cols && orow0 < rows) {
    float sg[16];
    load_signs(signs16, sg);
    float u[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) u[i] = __uint_as_float((uint32_t)tile[rb * 16 + i][c] << 16) * sg[i];
    hadamard16_inplace(u);
    uint32_t lo, hi, sf;
    const int64_t kb = orow0 >> 4;
    encode_block<SR_C>(u, g_c, (uint64_t)oc * ctr.pitch_c + ctr.base_c + (uint64_t)kb, keys_c, offset, lo, hi, sf);
    *reinterpret_cast<uint2*>(q_cols + oc * (rows >> 1) + kb * 8) = make_uint2(lo, hi);
    sf_cols[sf_offset(oc, kb, ((rows >> 4) + 3) >> 2)] = (uint8_t)sf;
  }
}

// plain maximum and maximum after the Hadamard transform along the rows, from one read
__global__ void __launch_bounds__(256) amax_both_cols_kernel(const uint16_t* __restrict__ x, int64_t rows,
                                                             int64_t cols, int64_t ld,
                                                             const float* __restrict__ signs16,
                                                             float* __restrict__ maxima2) {
  float sg[16];
  load_signs(signs16, sg);
  uint32_t sm[16];
  sign_masks(sg, sm);
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  const int64_t r_base = (int64_t)blockIdx.y * 64;
  float m = 0.0f;
  uint32_t mp = 0u;
  if (c < cols) {
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
      const int64_t r0 = r_base + 16 * j;
      if (r0 >= rows) break;
      const uint32_t* p = reinterpret_cast<const uint32_t*>(x + r0 * ld + c);
      float v0[16], v1[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t w = __ldg(p + (size_t)i * (size_t)(ld >> 1));
        mp = __vimax3_u16x2(mp, w & 0x7fff7fffu, 0u);          // both halves carry a running maximum
        const uint32_t u = w ^ sm[i];
        v0[i] = bf16_lo(u);
        v1[i] = bf16_hi(u);
      }
      hadamard16_pair(v0, v1);
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
    }
  }
  mp = max(mp & 0xffffu, mp >> 16);
  cta_max_to(maxima2, __uint_as_float(mp << 16), 0);
  cta_max_to(maxima2 + 1, m, 1);
}

static inline int grid_for(int64_t work_items, int threads, int max_blocks) {
  int64_t b = (work_items + threads - 1) / threads;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace nvfp4

using namespace nvfp4;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int nvfp4_amax_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int rht,
                               int transpose, const float* signs16, float* amax, int zero_first,
                               void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (x == nullptr || amax == nullptr || (rht && signs16 == nullptr)) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols) return NVFP4_E_SHAPE;
  if (!aligned16(x) || (ld & 7) != 0 || (rht && !aligned16(signs16))) return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(amax, 0, sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  if (!rht) {
    if ((cols & 7) != 0) return NVFP4_E_SHAPE;
    const int vpr = (int)(cols >> 3);
    amax_plain_kernel<<<grid_for(rows * vpr, 512 * 4, 148 * 8), 512, 0, stream>>>(xp, rows, vpr, ld, amax);
  } else if (!transpose) {
    if ((cols & 15) != 0) return NVFP4_E_SHAPE;
    const int bpr = (int)(cols >> 4);
    amax_rht_rows_kernel<<<grid_for(rows * bpr, 256 * 2, 148 * 16), 256, 0, stream>>>(xp, rows, bpr, ld, signs16, amax);
  } else {
    if ((rows & 15) != 0 || (cols & 1) != 0) return NVFP4_E_SHAPE;
    dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
    if (grid.y > 65535u) return NVFP4_E_SHAPE;
    if ((cols & 7) == 0) {
      const dim3 wgrid((unsigned)((cols + kWideCols - 1) / kWideCols), grid.y);
      amax_cols_wide_kernel<false><<<wgrid, 256, 0, stream>>>(xp, rows, cols, ld, signs16, amax);
    } else {
      amax_rht_cols_kernel<<<grid, 256, 0, stream>>>(xp, rows, cols, ld, signs16, amax);
    }
  }
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

namespace nvfp4 { namespace fused {
int quantize_rows_known_amax(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode, int rht,
                             const float* signs16, const float* amax, uint64_t seed, uint64_t offset,
                             uint64_t counter_pitch, uint64_t counter_base,
                             uint8_t* qdata, uint8_t* scales, float* pts_out, cudaStream_t stream);
}}

extern "C" int nvfp4_quantize_shard_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose,
                                         int mode, int rht, const float* signs16, const float* amax,
                                         uint64_t seed, uint64_t offset, uint64_t counter_pitch, uint64_t counter_base,
                                         uint8_t* qdata, uint8_t* scales, float* pts_out, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (x == nullptr || amax == nullptr || qdata == nullptr || scales == nullptr || (rht && signs16 == nullptr))
    return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols) return NVFP4_E_SHAPE;
  if (mode != NVFP4_ROUND_NEAREST && mode != NVFP4_ROUND_STOCHASTIC) return NVFP4_E_MODE;
  if (!aligned16(x) || (ld & 7) != 0 || (reinterpret_cast<uintptr_t>(qdata) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(scales) & 15u) != 0 || (rht && !aligned16(signs16)))
    return NVFP4_E_ALIGN;
  const int64_t out_rows = transpose ? cols : rows;
  const int64_t k = transpose ? rows : cols;
  if ((k & 15) != 0) return NVFP4_E_SHAPE;
  if (transpose && (cols & 1) != 0) return NVFP4_E_SHAPE;
  if (!transpose) {
    // row-wise output with the maximum given: one streaming pass of the single-launch kernel's
    // quantize phase (it declines only tensors of 2^31 blocks or more, which the plain kernel takes)
    const int rc = nvfp4::fused::quantize_rows_known_amax(x, rows, cols, ld, mode, rht, signs16, amax, seed, offset,
                                                          counter_pitch, counter_base, qdata, scales, pts_out, stream);
    if (rc != NVFP4_E_LIMIT) return rc;
  }
  // padding of the tiled scale buffer must read as zero (the reference pads with zeros)
  const int64_t sm = (out_rows + 127) / 128 * 128, sk = (k / 16 + 3) / 4 * 4;
  if (sm != out_rows || sk != k / 16) {
    if (cudaMemsetAsync(scales, 0, (size_t)(sm * sk), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  }
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const bool sr = mode == NVFP4_ROUND_STOCHASTIC;
  const PhiloxKeys keys = make_philox_keys(seed);
  if (!transpose) {
    const int bpr = (int)(cols >> 4);
    const int grid = grid_for(rows * bpr, 256, 1 << 30);
#define NVFP4_LAUNCH_ROWS(SR_, RHT_) \
    quant_rows_kernel<SR_, RHT_><<<grid, 256, 0, stream>>>(xp, rows, bpr, ld, signs16, amax, keys, offset, qdata, scales, pts_out, counter_pitch, counter_base)
    if (sr && rht) NVFP4_LAUNCH_ROWS(true, true);
    else if (sr) NVFP4_LAUNCH_ROWS(true, false);
    else if (rht) NVFP4_LAUNCH_ROWS(false, true);
    else NVFP4_LAUNCH_ROWS(false, false);
#undef NVFP4_LAUNCH_ROWS
  } else {
    dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
    if (grid.y > 65535u) return NVFP4_E_SHAPE;
#define NVFP4_LAUNCH_COLS(SR_, RHT_) \
    quant_cols_kernel<SR_, RHT_><<<grid, 256, 0, stream>>>(xp, rows, cols, ld, signs16, amax, keys, offset, qdata, scales, pts_out, counter_pitch, counter_base)
    if (sr && rht) NVFP4_LAUNCH_COLS(true, true);
    else if (sr) NVFP4_LAUNCH_COLS(true, false);
    else if (rht) NVFP4_LAUNCH_COLS(false, true);
    else NVFP4_LAUNCH_COLS(false, false);
#undef NVFP4_LAUNCH_COLS
  }
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}


extern "C" int nvfp4_quantize_weight_bf16(const void* w, int64_t rows, int64_t cols, int64_t ld, int two_d,
                                          const float* amax, uint8_t* qdata_rows, uint8_t* scales_rows,
                                          uint8_t* qdata_cols, uint8_t* scales_cols, float* pts_out, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!w || !amax || !qdata_rows || !scales_rows || !qdata_cols || !scales_cols) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || (rows & 15) != 0 || (cols & 15) != 0) return NVFP4_E_SHAPE;
  if (!aligned16(w) || (ld & 7) != 0 || !aligned16(qdata_rows) || !aligned16(qdata_cols) || !aligned16(scales_rows) ||
      !aligned16(scales_cols))
    return NVFP4_E_ALIGN;
  // padding of the tiled scale buffers must read as zero
  auto clear_if_padded = [&](uint8_t* sf, int64_t m, int64_t k) {
    const int64_t sm = (m + 127) / 128 * 128, sk = (k / 16 + 3) / 4 * 4;
    if (sm == m && sk == k / 16) return true;
    return cudaMemsetAsync(sf, 0, (size_t)(sm * sk), stream) == cudaSuccess;
  };
  if (!clear_if_padded(scales_rows, rows, cols) || !clear_if_padded(scales_cols, cols, rows)) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
  if (grid.y > 65535u) return NVFP4_E_LIMIT;
  const uint16_t* wp = static_cast<const uint16_t*>(w);
  if (two_d)
    quant_weight_dual_kernel<true><<<grid, 256, 0, stream>>>(wp, rows, cols, ld, amax, qdata_rows, scales_rows, qdata_cols,
                                                             scales_cols, pts_out);
  else
    quant_weight_dual_kernel<false><<<grid, 256, 0, stream>>>(wp, rows, cols, ld, amax, qdata_rows, scales_rows, qdata_cols,
                                                              scales_cols, pts_out);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}


extern "C" int nvfp4_amax_both_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, const float* signs16,
                                    float* maxima2, int zero_first, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !signs16 || !maxima2) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || (rows & 15) != 0 || (cols & 1) != 0) return NVFP4_E_SHAPE;
  if (!aligned16(x) || (ld & 7) != 0 || !aligned16(signs16)) return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(maxima2, 0, 2 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
  if (grid.y > 65535u) return NVFP4_E_LIMIT;
  if ((cols & 7) == 0) {
    const dim3 wgrid((unsigned)((cols + kWideCols - 1) / kWideCols), grid.y);
    amax_cols_wide_kernel<true><<<wgrid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), rows, cols, ld, signs16, maxima2);
  } else {
    amax_both_cols_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), rows, cols, ld, signs16, maxima2);
  }
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_quantize_dual_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode_rows,
                                        int mode_cols, const float* signs16, const float* amax_rows,
                                        const float* amax_cols, uint64_t seed_rows, uint64_t seed_cols, uint64_t offset,
                                        const uint64_t* counters4, uint8_t* qdata_rows, uint8_t* scales_rows,
                                        float* pts_rows, uint8_t* qdata_cols, uint8_t* scales_cols, float* pts_cols,
                                        void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !signs16 || !amax_rows || !amax_cols || !qdata_rows || !scales_rows || !qdata_cols || !scales_cols)
    return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || ld < cols || (rows & 15) != 0 || (cols & 15) != 0) return NVFP4_E_SHAPE;
  auto bad_mode = [](int m) { return m != NVFP4_ROUND_NEAREST && m != NVFP4_ROUND_STOCHASTIC; };
  if (bad_mode(mode_rows) || bad_mode(mode_cols)) return NVFP4_E_MODE;
  if (!aligned16(x) || (ld & 7) != 0 || !aligned16(qdata_rows) || !aligned16(qdata_cols) || !aligned16(scales_rows) ||
      !aligned16(scales_cols) || !aligned16(signs16))
    return NVFP4_E_ALIGN;
  DualCounters ctr{(uint64_t)(cols >> 4), 0, (uint64_t)(rows >> 4), 0};      // the tensor is whole
  if (counters4 != nullptr) ctr = DualCounters{counters4[0], counters4[1], counters4[2], counters4[3]};
  // the hardware draws from a 32-bit counter word pair; keep both layouts' counters inside 2^64 trivially,
  // and inside the documented 2^32 blocks per tensor
  if ((uint64_t)rows * ctr.pitch_r + ctr.base_r >= (1ull << 32) || (uint64_t)cols * ctr.pitch_c + ctr.base_c >= (1ull << 32))
    return NVFP4_E_LIMIT;
  auto clear_if_padded = [&](uint8_t* sf, int64_t m, int64_t k) {
    const int64_t sm = (m + 127) / 128 * 128, sk = (k / 16 + 3) / 4 * 4;
    if (sm == m && sk == k / 16) return true;
    return cudaMemsetAsync(sf, 0, (size_t)(sm * sk), stream) == cudaSuccess;
  };
  if (!clear_if_padded(scales_rows, rows, cols) || !clear_if_padded(scales_cols, cols, rows)) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
  if (grid.y > 65535u) return NVFP4_E_LIMIT;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const bool sr_r = mode_rows == NVFP4_ROUND_STOCHASTIC, sr_c = mode_cols == NVFP4_ROUND_STOCHASTIC;
  const PhiloxKeys keys_r = make_philox_keys(seed_rows), keys_c = make_philox_keys(seed_cols);
#define NVFP4_LAUNCH_DUAL(R_, C_) \
  quant_act_dual_kernel<R_, C_><<<grid, 256, 0, stream>>>(xp, rows, cols, ld, signs16, amax_rows, amax_cols, keys_r, \
      keys_c, offset, ctr, qdata_rows, scales_rows, pts_rows, qdata_cols, scales_cols, pts_cols)
  if (sr_r && sr_c) NVFP4_LAUNCH_DUAL(true, true);
  else if (sr_r) NVFP4_LAUNCH_DUAL(true, false);
  else if (sr_c) NVFP4_LAUNCH_DUAL(false, true);
  else NVFP4_LAUNCH_DUAL(false, false);
#undef NVFP4_LAUNCH_DUAL
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_quantize_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int transpose,
                                   int mode, int rht, const float* signs16, const float* amax,
                                   uint64_t seed, uint64_t offset, uint8_t* qdata, uint8_t* scales,
                                   float* pts_out, void* stream_) {
  // the tensor is whole: a block's counter is its index in x (or in x^T): out_row * (K / 16) + k / 16
  const uint64_t pitch = (uint64_t)((transpose ? rows : cols) / 16);
  return nvfp4_quantize_shard_bf16(x, rows, cols, ld, transpose, mode, rht, signs16, amax, seed, offset, pitch, 0,
                                   qdata, scales, pts_out, stream_);
}
