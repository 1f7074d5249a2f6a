// Producer fusion in front of the quantizer: SwiGLU (and its backward) as one pass that also leaves
// the per-tensor maxima the following NVFP4 quantizations need, so that those run as a single
// quantize pass (nvfp4_quantize_bf16 with the amax given) instead of amax pass + quantize pass.
//
//   forward   h  = silu(g) * u                                   -> h bf16, amax(h), amax(RHT_rows(h))
//   backward  dg = dh * u * sig(g) * (1 + g * (1 - sig(g)))      -> dg, du bf16 and both maxima of each
//             du = dh * silu(g)
//
// The arithmetic is fp32 and the result is rounded to bf16 once.  The maxima are taken over the
// ROUNDED values, with exactly the operations of amax_plain_kernel / amax_rht_cols_kernel
// (csrc/quantize.cu), so a quantizer given them produces the bytes it would produce after its own
// amax pass over the stored tensor.  "RHT_rows" is the 16-point random-sign Hadamard along the ROW
// (token) dimension in groups of 16 rows: the transform of the wgrad operands (the contraction of
// dW = dY^T X runs over tokens).
//
// A thread owns two adjacent columns and up to 64 consecutive rows (four 16-row blocks), so a warp
// reads and writes 128 contiguous bytes per row; the maxima leave a CTA as one atomic each.  HBM-bound: 6 bytes per element forward, 10 backward.
// The reference computes these with torch element-wise kernels (nvfp4_train.py:120-123 for the
// squared-ReLU MLP of its models); there is no fused counterpart in it.
#include "common.cuh"
#include "nvfp4_b200.h"

namespace nvfp4 {
namespace swiglu {

__device__ __forceinline__ void load_signs(const float* __restrict__ signs16, float (&sg)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 s = __ldg(reinterpret_cast<const float4*>(signs16) + i);
    sg[4 * i] = s.x; sg[4 * i + 1] = s.y; sg[4 * i + 2] = s.z; sg[4 * i + 3] = s.w;
  }
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));   // non-negative floats order like their bits
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// one atomic per CTA and address: same-address atomics from every warp would serialise in the L2
// (tens of thousands of them cost more than the whole pass)
template <int N>
__device__ __forceinline__ void cta_max_to_global(float (&m)[N], float* __restrict__ dst, const bool (&use)[N]) {
  __shared__ float part[N][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < N; ++k) {
    m[k] = warp_max(m[k]);
    if (lane == 0) part[k][warp] = m[k];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float v = lane < 8 ? part[k][lane] : 0.0f;
      v = warp_max(v);
      if (lane == 0 && use[k]) atomic_max_nonneg(dst + k, v);
    }
  }
}

constexpr int kRowBlocks = 4;     // 16-row blocks per thread: 64 rows per CTA

// max |v| and max |RHT(v)| of one 16-row block of two columns (already rounded to bf16)
__device__ __forceinline__ void block_maxima(const uint32_t (&w)[16], const float (&sg)[16], bool rht,
                                             float& m_plain, float& m_rht) {
  float v0[16], v1[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v0[i] = bf16_lo(w[i]);
    v1[i] = bf16_hi(w[i]);
    m_plain = fmaxf(m_plain, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
  }
  if (rht) {
#pragma unroll
    for (int i = 0; i < 16; ++i) { v0[i] *= sg[i]; v1[i] *= sg[i]; }
    hadamard16_inplace(v0);
    hadamard16_inplace(v1);
#pragma unroll
    for (int i = 0; i < 16; ++i) m_rht = fmaxf(m_rht, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
  }
}

// grid: (ceil(cols / 2 / 256), ceil(rows / 64)); maxima[0] = plain, maxima[1] = RHT along rows
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint16_t* __restrict__ gate,
                                                         const uint16_t* __restrict__ up, int64_t rows,
                                                         int64_t cols, int64_t ld_in, uint16_t* __restrict__ out,
                                                         int64_t ld_out, const float* __restrict__ signs16,
                                                         float* __restrict__ maxima) {
  const bool rht = signs16 != nullptr;
  float sg[16];
  if (rht) load_signs(signs16, sg);
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  float m[2] = {0.0f, 0.0f};
  if (c < cols) {
#pragma unroll 1
    for (int j = 0; j < kRowBlocks; ++j) {
      const int64_t r0 = ((int64_t)blockIdx.y * kRowBlocks + j) * 16;
      if (r0 >= rows) break;
      const int nrow = (int)min((int64_t)16, rows - r0);
      const uint32_t* pg = reinterpret_cast<const uint32_t*>(gate + r0 * ld_in + c);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(up + r0 * ld_in + c);
      uint32_t wg[16], wu[16], wh[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const bool in = i < nrow;
        wg[i] = in ? __ldg(pg + (size_t)i * (size_t)(ld_in >> 1)) : 0u;
        wu[i] = in ? __ldg(pu + (size_t)i * (size_t)(ld_in >> 1)) : 0u;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g0 = bf16_lo(wg[i]), g1 = bf16_hi(wg[i]);
        wh[i] = pack_bf16x2(g0 * sigmoidf(g0) * bf16_lo(wu[i]), g1 * sigmoidf(g1) * bf16_hi(wu[i]));
      }
      uint32_t* po = reinterpret_cast<uint32_t*>(out + r0 * ld_out + c);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i < nrow) po[(size_t)i * (size_t)(ld_out >> 1)] = wh[i];
      block_maxima(wh, sg, rht, m[0], m[1]);
    }
  }
  const bool use[2] = {true, rht};
  cta_max_to_global<2>(m, maxima, use);
}

// maxima[0], [1] = plain / RHT of dgate; maxima[2], [3] = plain / RHT of dup
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint16_t* __restrict__ gate,
                                                         const uint16_t* __restrict__ up,
                                                         const uint16_t* __restrict__ dh, int64_t rows,
                                                         int64_t cols, int64_t ld_in, int64_t ld_dh,
                                                         uint16_t* __restrict__ dgate,
                                                         uint16_t* __restrict__ dup, int64_t ld_out,
                                                         const float* __restrict__ signs16,
                                                         float* __restrict__ maxima) {
  const bool rht = signs16 != nullptr;
  float sg[16];
  if (rht) load_signs(signs16, sg);
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  float m[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (c < cols) {
#pragma unroll 1
    for (int j = 0; j < kRowBlocks; ++j) {
      const int64_t r0 = ((int64_t)blockIdx.y * kRowBlocks + j) * 16;
      if (r0 >= rows) break;
      const int nrow = (int)min((int64_t)16, rows - r0);
      const uint32_t* pg = reinterpret_cast<const uint32_t*>(gate + r0 * ld_in + c);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(up + r0 * ld_in + c);
      const uint32_t* pd = reinterpret_cast<const uint32_t*>(dh + r0 * ld_dh + c);
      uint32_t wg[16], wu[16], wd[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const bool in = i < nrow;
        const size_t off = (size_t)i * (size_t)(ld_in >> 1);
        wg[i] = in ? __ldg(pg + off) : 0u;
        wu[i] = in ? __ldg(pu + off) : 0u;
        wd[i] = in ? __ldg(pd + (size_t)i * (size_t)(ld_dh >> 1)) : 0u;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {                       // wg <- dgate, wu <- dup, in place
        float dgv[2], duv[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float g = h ? bf16_hi(wg[i]) : bf16_lo(wg[i]), u = h ? bf16_hi(wu[i]) : bf16_lo(wu[i]);
          const float d = h ? bf16_hi(wd[i]) : bf16_lo(wd[i]);
          const float sgm = sigmoidf(g);
          duv[h] = d * (g * sgm);
          dgv[h] = d * u * (sgm * (1.0f + g * (1.0f - sgm)));
        }
        wg[i] = pack_bf16x2(dgv[0], dgv[1]);
        wu[i] = pack_bf16x2(duv[0], duv[1]);
      }
      uint32_t* og = reinterpret_cast<uint32_t*>(dgate + r0 * ld_out + c);
      uint32_t* ou = reinterpret_cast<uint32_t*>(dup + r0 * ld_out + c);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i < nrow) {
          og[(size_t)i * (size_t)(ld_out >> 1)] = wg[i];
          ou[(size_t)i * (size_t)(ld_out >> 1)] = wu[i];
        }
      block_maxima(wg, sg, rht, m[0], m[1]);
      block_maxima(wu, sg, rht, m[2], m[3]);
    }
  }
  const bool use[4] = {true, rht, true, rht};
  cta_max_to_global<4>(m, maxima, use);
}

// ---- wide variants: row-contiguous 16-byte accesses, the 16-row column view through shared memory ----
// A CTA works on tiles of 16 rows x 512 columns.  Element-wise phase: thread t and step k own the
// eight columns 8 * (t % 64) of row 4 * k + t / 64, so a warp moves 512 contiguous bytes of a row per
// instruction; the rounded results also go to a shared tile.  Column phase: thread t reads its two
// columns of all 16 rows from the tile (consecutive lanes, consecutive banks) for the Hadamard maxima.
// The narrow kernels above stay for shapes without 16-byte rows.
constexpr int kTileCols = 512;
constexpr int kPitchWords = kTileCols / 2 + 4;            // 32-bit words per tile row, padded

__device__ __forceinline__ uint4 ldg16(const uint16_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void tile_rht_max(const uint32_t* tile, const float (&sg)[16], bool active, float& m_rht) {
  if (!active) return;
  float v0[16], v1[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t w = tile[i * kPitchWords + threadIdx.x];
    v0[i] = bf16_lo(w) * sg[i];
    v1[i] = bf16_hi(w) * sg[i];
  }
  hadamard16_inplace(v0);
  hadamard16_inplace(v1);
#pragma unroll
  for (int i = 0; i < 16; ++i) m_rht = fmaxf(m_rht, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
}

__global__ void __launch_bounds__(256) swiglu_fwd_wide_kernel(const uint16_t* __restrict__ gate,
                                                              const uint16_t* __restrict__ up, int64_t rows,
                                                              int64_t cols, int64_t ld_in, uint16_t* __restrict__ out,
                                                              int64_t ld_out, const float* __restrict__ signs16,
                                                              float* __restrict__ maxima) {
  __shared__ __align__(16) uint32_t tile[16 * kPitchWords];
  const bool rht = signs16 != nullptr;
  float sg[16];
  if (rht) load_signs(signs16, sg);
  const int64_t c0 = (int64_t)blockIdx.x * kTileCols;
  const int cc = (threadIdx.x & 63) * 8;
  const bool col_in = c0 + cc < cols;                       // cols is a multiple of 8 here
  float m[2] = {0.0f, 0.0f};
#pragma unroll 1
  for (int j = 0; j < kRowBlocks; ++j) {
    const int64_t r0 = ((int64_t)blockIdx.y * kRowBlocks + j) * 16;
    if (r0 >= rows) break;                                   // uniform across the CTA
    uint4 g4[4], u4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t r = r0 + 4 * k + (threadIdx.x >> 6);
      const bool in = col_in && r < rows;
      g4[k] = in ? ldg16(gate + r * ld_in + c0 + cc) : make_uint4(0, 0, 0, 0);
      u4[k] = in ? ldg16(up + r * ld_in + c0 + cc) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t gw[4] = {g4[k].x, g4[k].y, g4[k].z, g4[k].w}, uw[4] = {u4[k].x, u4[k].y, u4[k].z, u4[k].w};
      uint32_t hw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float a0 = bf16_lo(gw[q]), a1 = bf16_hi(gw[q]);
        hw[q] = pack_bf16x2(a0 * sigmoidf(a0) * bf16_lo(uw[q]), a1 * sigmoidf(a1) * bf16_hi(uw[q]));
        m[0] = fmaxf(m[0], fmaxf(fabsf(bf16_lo(hw[q])), fabsf(bf16_hi(hw[q]))));
      }
      const int rl = 4 * k + (threadIdx.x >> 6);
      const int64_t r = r0 + rl;
      const uint4 h4 = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      if (col_in && r < rows) *reinterpret_cast<uint4*>(out + r * ld_out + c0 + cc) = h4;
      if (rht) *reinterpret_cast<uint4*>(&tile[rl * kPitchWords + (cc >> 1)]) = h4;
    }
    if (rht) {
      __syncthreads();
      tile_rht_max(tile, sg, c0 + 2 * (int64_t)threadIdx.x < cols, m[1]);
      __syncthreads();
    }
  }
  const bool use[2] = {true, rht};
  cta_max_to_global<2>(m, maxima, use);
}

__global__ void __launch_bounds__(256) swiglu_bwd_wide_kernel(const uint16_t* __restrict__ gate,
                                                              const uint16_t* __restrict__ up,
                                                              const uint16_t* __restrict__ dh, int64_t rows,
                                                              int64_t cols, int64_t ld_in, int64_t ld_dh,
                                                              uint16_t* __restrict__ dgate, uint16_t* __restrict__ dup,
                                                              int64_t ld_out, const float* __restrict__ signs16,
                                                              float* __restrict__ maxima) {
  __shared__ __align__(16) uint32_t tile_g[16 * kPitchWords];
  __shared__ __align__(16) uint32_t tile_u[16 * kPitchWords];
  const bool rht = signs16 != nullptr;
  float sg[16];
  if (rht) load_signs(signs16, sg);
  const int64_t c0 = (int64_t)blockIdx.x * kTileCols;
  const int cc = (threadIdx.x & 63) * 8;
  const bool col_in = c0 + cc < cols;
  float m[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
  for (int j = 0; j < kRowBlocks; ++j) {
    const int64_t r0 = ((int64_t)blockIdx.y * kRowBlocks + j) * 16;
    if (r0 >= rows) break;
#pragma unroll 2
    for (int k = 0; k < 4; ++k) {
      const int rl = 4 * k + (threadIdx.x >> 6);
      const int64_t r = r0 + rl;
      const bool in = col_in && r < rows;
      const uint4 z = make_uint4(0, 0, 0, 0);
      const uint4 g4 = in ? ldg16(gate + r * ld_in + c0 + cc) : z, u4 = in ? ldg16(up + r * ld_in + c0 + cc) : z;
      const uint4 d4 = in ? ldg16(dh + r * ld_dh + c0 + cc) : z;
      const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
      uint32_t og[4], ou[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float dgv[2], duv[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float g = h ? bf16_hi(gw[q]) : bf16_lo(gw[q]), u = h ? bf16_hi(uw[q]) : bf16_lo(uw[q]);
          const float d = h ? bf16_hi(dw[q]) : bf16_lo(dw[q]);
          const float sgm = sigmoidf(g);
          duv[h] = d * (g * sgm);
          dgv[h] = d * u * (sgm * (1.0f + g * (1.0f - sgm)));
        }
        og[q] = pack_bf16x2(dgv[0], dgv[1]);
        ou[q] = pack_bf16x2(duv[0], duv[1]);
        m[0] = fmaxf(m[0], fmaxf(fabsf(bf16_lo(og[q])), fabsf(bf16_hi(og[q]))));
        m[2] = fmaxf(m[2], fmaxf(fabsf(bf16_lo(ou[q])), fabsf(bf16_hi(ou[q]))));
      }
      const uint4 og4 = make_uint4(og[0], og[1], og[2], og[3]), ou4 = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      if (in) {
        *reinterpret_cast<uint4*>(dgate + r * ld_out + c0 + cc) = og4;
        *reinterpret_cast<uint4*>(dup + r * ld_out + c0 + cc) = ou4;
      }
      if (rht) {
        *reinterpret_cast<uint4*>(&tile_g[rl * kPitchWords + (cc >> 1)]) = og4;
        *reinterpret_cast<uint4*>(&tile_u[rl * kPitchWords + (cc >> 1)]) = ou4;
      }
    }
    if (rht) {
      __syncthreads();
      const bool active = c0 + 2 * (int64_t)threadIdx.x < cols;
      tile_rht_max(tile_g, sg, active, m[1]);
      tile_rht_max(tile_u, sg, active, m[3]);
      __syncthreads();
    }
  }
  const bool use[4] = {true, rht, true, rht};
  cta_max_to_global<4>(m, maxima, use);
}

// Squared ReLU, the MLP activation of the reference's models (nvfp4_train.py:120-123,
// scaling/train_text.py:57-59): a = relu(x)^2 and da/dx = 2 relu(x), with the same two maxima of what
// is written.  Same tiling as the wide SwiGLU kernels; BWD reads x and the incoming gradient.
template <bool BWD>
__global__ void __launch_bounds__(256) relu2_wide_kernel(const uint16_t* __restrict__ x,
                                                         const uint16_t* __restrict__ dout, int64_t rows,
                                                         int64_t cols, int64_t ld_in, uint16_t* __restrict__ out,
                                                         int64_t ld_out, const float* __restrict__ signs16,
                                                         float* __restrict__ maxima) {
  __shared__ __align__(16) uint32_t tile[16 * kPitchWords];
  const bool rht = signs16 != nullptr;
  float sg[16];
  if (rht) load_signs(signs16, sg);
  const int64_t c0 = (int64_t)blockIdx.x * kTileCols;
  const int cc = (threadIdx.x & 63) * 8;
  const bool col_in = c0 + cc < cols;
  float m[2] = {0.0f, 0.0f};
#pragma unroll 1
  for (int j = 0; j < kRowBlocks; ++j) {
    const int64_t r0 = ((int64_t)blockIdx.y * kRowBlocks + j) * 16;
    if (r0 >= rows) break;
    uint4 x4[4], d4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t r = r0 + 4 * k + (threadIdx.x >> 6);
      const bool in = col_in && r < rows;
      x4[k] = in ? ldg16(x + r * ld_in + c0 + cc) : make_uint4(0, 0, 0, 0);
      if (BWD) d4[k] = in ? ldg16(dout + r * ld_in + c0 + cc) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t xw[4] = {x4[k].x, x4[k].y, x4[k].z, x4[k].w};
      const uint32_t dw[4] = {BWD ? d4[k].x : 0u, BWD ? d4[k].y : 0u, BWD ? d4[k].z : 0u, BWD ? d4[k].w : 0u};
      uint32_t hw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float r0f = fmaxf(bf16_lo(xw[q]), 0.0f), r1f = fmaxf(bf16_hi(xw[q]), 0.0f);
        hw[q] = BWD ? pack_bf16x2(2.0f * r0f * bf16_lo(dw[q]), 2.0f * r1f * bf16_hi(dw[q]))
                    : pack_bf16x2(r0f * r0f, r1f * r1f);
        m[0] = fmaxf(m[0], fmaxf(fabsf(bf16_lo(hw[q])), fabsf(bf16_hi(hw[q]))));
      }
      const int rl = 4 * k + (threadIdx.x >> 6);
      const int64_t r = r0 + rl;
      const uint4 h4 = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      if (col_in && r < rows) *reinterpret_cast<uint4*>(out + r * ld_out + c0 + cc) = h4;
      if (rht) *reinterpret_cast<uint4*>(&tile[rl * kPitchWords + (cc >> 1)]) = h4;
    }
    if (rht) {
      __syncthreads();
      tile_rht_max(tile, sg, c0 + 2 * (int64_t)threadIdx.x < cols, m[1]);
      __syncthreads();
    }
  }
  const bool use[2] = {true, rht};
  cta_max_to_global<2>(m, maxima, use);
}

// 16-byte rows everywhere: the wide kernels apply
static bool wide_ok(const void* a, const void* b, const void* c, const void* o1, const void* o2, int64_t cols,
                    int64_t ld_in, int64_t ld_out) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return (cols & 7) == 0 && (ld_in & 7) == 0 && (ld_out & 7) == 0 && al(a) && al(b) && al(c) && al(o1) && al(o2);
}

static int check(const void* a, const void* b, const void* c, const void* o1, const void* o2, int64_t rows,
                 int64_t cols, int64_t ld_in, int64_t ld_out, const float* signs16, const float* maxima) {
  if (!a || !b || !c || !o1 || !o2 || !maxima) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || (cols & 1) != 0 || ld_in < cols || ld_out < cols) return NVFP4_E_SHAPE;
  if (signs16 != nullptr && (rows & 15) != 0) return NVFP4_E_SHAPE;      // the row transform needs whole blocks
  if ((rows + 63) / 64 > 65535) return NVFP4_E_LIMIT;
  auto mis = [](const void* p, uintptr_t al) { return (reinterpret_cast<uintptr_t>(p) & (al - 1)) != 0; };
  if (mis(a, 4) || mis(b, 4) || mis(c, 4) || mis(o1, 4) || mis(o2, 4) || (ld_in & 1) != 0 || (ld_out & 1) != 0 ||
      mis(maxima, 4) || (signs16 != nullptr && mis(signs16, 16)))
    return NVFP4_E_ALIGN;
  return NVFP4_OK;
}

}  // namespace swiglu
}  // namespace nvfp4

using namespace nvfp4::swiglu;

extern "C" int nvfp4_swiglu_fwd_bf16(const void* gate, const void* up, int64_t rows, int64_t cols, int64_t ld_in,
                                     void* out, int64_t ld_out, const float* signs16, float* maxima2,
                                     int zero_first, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rc = check(gate, up, gate, out, out, rows, cols, ld_in, ld_out, signs16, maxima2);
  if (rc != NVFP4_OK) return rc;
  if (zero_first && cudaMemsetAsync(maxima2, 0, 2 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
  if (wide_ok(gate, up, gate, out, out, cols, ld_in, ld_out))
    swiglu_fwd_wide_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(gate),
                                                      static_cast<const uint16_t*>(up), rows, cols, ld_in,
                                                      static_cast<uint16_t*>(out), ld_out, signs16, maxima2);
  else
    swiglu_fwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(gate), static_cast<const uint16_t*>(up),
                                                 rows, cols, ld_in, static_cast<uint16_t*>(out), ld_out, signs16,
                                                 maxima2);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_swiglu_bwd_strided_bf16(const void* gate, const void* up, const void* dh, int64_t rows,
                                             int64_t cols, int64_t ld_in, int64_t ld_dout, void* dgate, void* dup,
                                             int64_t ld_out, const float* signs16, float* maxima4, int zero_first,
                                             void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rc = check(gate, up, dh, dgate, dup, rows, cols, ld_in, ld_out, signs16, maxima4);
  if (rc != NVFP4_OK) return rc;
  if (ld_dout < cols) return NVFP4_E_SHAPE;
  if ((ld_dout & 1) != 0) return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(maxima4, 0, 4 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
  if (wide_ok(gate, up, dh, dgate, dup, cols, ld_in, ld_out) && (ld_dout & 7) == 0)
    swiglu_bwd_wide_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(gate),
                                                      static_cast<const uint16_t*>(up),
                                                      static_cast<const uint16_t*>(dh), rows, cols, ld_in, ld_dout,
                                                      static_cast<uint16_t*>(dgate), static_cast<uint16_t*>(dup),
                                                      ld_out, signs16, maxima4);
  else
    swiglu_bwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(gate), static_cast<const uint16_t*>(up),
                                                 static_cast<const uint16_t*>(dh), rows, cols, ld_in, ld_dout,
                                                 static_cast<uint16_t*>(dgate), static_cast<uint16_t*>(dup), ld_out,
                                                 signs16, maxima4);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_swiglu_bwd_bf16(const void* gate, const void* up, const void* dh, int64_t rows, int64_t cols,
                                     int64_t ld_in, void* dgate, void* dup, int64_t ld_out, const float* signs16,
                                     float* maxima4, int zero_first, void* stream_) {
  return nvfp4_swiglu_bwd_strided_bf16(gate, up, dh, rows, cols, ld_in, ld_in, dgate, dup, ld_out, signs16, maxima4,
                                       zero_first, stream_);
}

// Squared ReLU and its backward with the maxima of the result (see relu2_wide_kernel).  Rows of 16
// bytes only (cols and both leading dimensions multiples of 8, 16-byte aligned pointers): other
// layouts get NVFP4_E_ALIGN and the caller keeps its own element-wise path.
extern "C" int nvfp4_relu2_fwd_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld_in, void* out,
                                    int64_t ld_out, const float* signs16, float* maxima2, int zero_first,
                                    void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rc = check(x, x, x, out, out, rows, cols, ld_in, ld_out, signs16, maxima2);
  if (rc != NVFP4_OK) return rc;
  if (!wide_ok(x, x, x, out, out, cols, ld_in, ld_out)) return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(maxima2, 0, 2 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
  relu2_wide_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), nullptr, rows, cols, ld_in,
                                                      static_cast<uint16_t*>(out), ld_out, signs16, maxima2);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_relu2_bwd_bf16(const void* x, const void* dout, int64_t rows, int64_t cols, int64_t ld_in,
                                    void* dx, int64_t ld_out, const float* signs16, float* maxima2, int zero_first,
                                    void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rc = check(x, dout, x, dx, dx, rows, cols, ld_in, ld_out, signs16, maxima2);
  if (rc != NVFP4_OK) return rc;
  if (!wide_ok(x, dout, x, dx, dx, cols, ld_in, ld_out)) return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(maxima2, 0, 2 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const dim3 grid((unsigned)((cols / 2 + 255) / 256), (unsigned)((rows + 63) / 64));
  relu2_wide_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(dout),
                                                     rows, cols, ld_in, static_cast<uint16_t*>(dx), ld_out, signs16,
                                                     maxima2);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}
