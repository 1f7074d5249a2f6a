// RMSNorm in front of the quantizer: h = x * rsqrt(mean(x^2) + eps) * w written once as bf16 together
// with the two per-tensor maxima the NVFP4 quantizations of h need -- max|h| for the forward operand
// and max|RHT_rows(h)| for the weight-gradient operand (16-point random-sign Hadamard over groups of
// 16 token rows) -- so that every quantization of h is one pass with the maximum given instead of a
// maximum pass plus a quantize pass.  The maxima are taken over the ROUNDED bf16 values with the
// operations of the quantizer's own maximum kernels, so the bytes that follow are the same.
//
// Call site in the reference: n1(x) / n2(x) feeding the q, k, v and up projections
// (nvfp4_train.py:105,114-122, scaling/train_text.py:41); there the norm is torch's rms_norm and each
// FP4Linear finds the maximum of the same tensor again.
//
// Forward: one CTA per 16 rows.  Phase A, one warp per two rows: sum of squares (16-byte loads,
// warp reduction) -> rstd.  Phase B, the tiling of the activation kernels (csrc/swiglu.cu): thread t
// and step k own eight columns of row 4k + t/64 of a 16 x 512 tile, the rounded results also go to a
// shared tile from which thread t reads its two columns of all 16 rows for the Hadamard maximum.
// x is read twice, the second time from L2 (a 16-row slab is at most 512 KiB).
// Backward: dx = rstd * (g*w - xhat * mean(g*w*xhat)), dw = sum over rows of g * xhat, one CTA per
// 32 rows, dw leaves the CTA as one atomic per column.
#include "common.cuh"
#include "nvfp4_b200.h"

namespace nvfp4 {
namespace rmsnorm {

constexpr int kTileCols = 512;
constexpr int kPitchWords = kTileCols / 2 + 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// eight consecutive elements of a row as fp32
template <bool F32>
__device__ __forceinline__ void load8(const void* base, int64_t idx, float (&v)[8]) {
  if (F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + idx));
    v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
    v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
  }
}
template <bool F32>
__device__ __forceinline__ void store8(void* base, int64_t idx, const float (&v)[8]) {
  if (F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + idx);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + idx) =
        make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
}

template <bool F32>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const void* __restrict__ x, const float* __restrict__ w,
                                                          int64_t rows, int64_t cols, float eps,
                                                          uint16_t* __restrict__ h, float* __restrict__ rstd_out,
                                                          const float* __restrict__ signs16,
                                                          float* __restrict__ maxima) {
  __shared__ __align__(16) uint32_t tile[16 * kPitchWords];
  __shared__ float rstd_s[16];
  __shared__ float part[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = (int64_t)blockIdx.x * 16;
  const bool rht = signs16 != nullptr;
  // ---- phase A: rstd of rows r0 + 2 * warp, + 1
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t r = r0 + 2 * warp + i;
    float ss = 0.0f;
    if (r < rows) {
      for (int64_t c = lane * 8; c < cols; c += 256) {
        float v[8];
        load8<F32>(x, r * cols + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) {
      const float rs = rsqrtf(ss / (float)cols + eps);
      rstd_s[2 * warp + i] = rs;
      if (r < rows) rstd_out[r] = rs;
    }
  }
  __syncthreads();
  // ---- phase B
  float sg[16];
  if (rht) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(signs16) + i);
      sg[4 * i] = s.x; sg[4 * i + 1] = s.y; sg[4 * i + 2] = s.z; sg[4 * i + 3] = s.w;
    }
  }
  const int cc = (threadIdx.x & 63) * 8;
  float m_plain = 0.0f, m_rht = 0.0f;
#pragma unroll 1
  for (int64_t c0 = 0; c0 < cols; c0 += kTileCols) {
    const bool col_in = c0 + cc < cols;
    float wv[8];
    if (col_in) load8<true>(w, c0 + cc, wv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rl = 4 * k + (threadIdx.x >> 6);
      const int64_t r = r0 + rl;
      uint4 h4 = make_uint4(0u, 0u, 0u, 0u);
      if (col_in && r < rows) {
        float v[8];
        load8<F32>(x, r * cols + c0 + cc, v);
        const float rs = rstd_s[rl];
        uint32_t hw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          hw[q] = pack_bf16x2((v[2 * q] * rs) * wv[2 * q], (v[2 * q + 1] * rs) * wv[2 * q + 1]);
          m_plain = fmaxf(m_plain, fmaxf(fabsf(bf16_lo(hw[q])), fabsf(bf16_hi(hw[q]))));
        }
        h4 = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4*>(h + r * cols + c0 + cc) = h4;
      }
      if (rht) *reinterpret_cast<uint4*>(&tile[rl * kPitchWords + (cc >> 1)]) = h4;
    }
    if (rht) {
      __syncthreads();
      if (c0 + 2 * (int64_t)threadIdx.x < cols) {
        float v0[16], v1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t t = tile[i * kPitchWords + threadIdx.x];
          v0[i] = bf16_lo(t) * sg[i];
          v1[i] = bf16_hi(t) * sg[i];
        }
        hadamard16_inplace(v0);
        hadamard16_inplace(v1);
#pragma unroll
        for (int i = 0; i < 16; ++i) m_rht = fmaxf(m_rht, fmaxf(fabsf(v0[i]), fabsf(v1[i])));
      }
      __syncthreads();
    }
  }
  // one atomic per CTA and word
  m_plain = warp_max(m_plain);
  m_rht = warp_max(m_rht);
  if (lane == 0) { part[0][warp] = m_plain; part[1][warp] = m_rht; }
  __syncthreads();
  if (warp == 0) {
    float a = lane < 8 ? part[0][lane] : 0.0f, b = lane < 8 ? part[1][lane] : 0.0f;
    a = warp_max(a);
    b = warp_max(b);
    if (lane == 0) {
      atomicMax(reinterpret_cast<unsigned int*>(maxima), __float_as_uint(a));
      if (rht) atomicMax(reinterpret_cast<unsigned int*>(maxima + 1), __float_as_uint(b));
    }
  }
}

// g: gradient of h (bf16 or fp32, G_F32), x and dx in the type of the input (F32).
constexpr int kBwdRows = 32;
template <bool F32, bool G_F32>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const void* __restrict__ x, const float* __restrict__ w,
                                                          const float* __restrict__ rstd, const void* __restrict__ g,
                                                          int64_t rows, int64_t cols, void* __restrict__ dx,
                                                          float* __restrict__ dw) {
  __shared__ float coef_s[kBwdRows];       // mean(g * w * xhat) of each row
  __shared__ float rstd_s[kBwdRows];
  __shared__ float red[4][64 * 8 + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = (int64_t)blockIdx.x * kBwdRows;
  // ---- phase A: per-row coefficient, four rows per warp
#pragma unroll 1
  for (int i = 0; i < kBwdRows / 8; ++i) {
    const int rl = (kBwdRows / 8) * warp + i;
    const int64_t r = r0 + rl;
    float acc = 0.0f, rs = 0.0f;
    if (r < rows) {
      rs = __ldg(rstd + r);
      for (int64_t c = lane * 8; c < cols; c += 256) {
        float xv[8], gv[8], wv[8];
        load8<F32>(x, r * cols + c, xv);
        load8<G_F32>(g, r * cols + c, gv);
        load8<true>(w, c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(gv[j] * wv[j], xv[j] * rs, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) { coef_s[rl] = acc / (float)cols; rstd_s[rl] = rs; }
  }
  __syncthreads();
  // ---- phase B: dx, and this CTA's part of dw
  const int cc = (threadIdx.x & 63) * 8, grp = threadIdx.x >> 6;
#pragma unroll 1
  for (int64_t c0 = 0; c0 < cols; c0 += kTileCols) {
    const bool col_in = c0 + cc < cols;
    float wv[8], dwv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col_in) load8<true>(w, c0 + cc, wv);
#pragma unroll 2
    for (int k = 0; k < kBwdRows / 4; ++k) {
      const int rl = 4 * k + grp;
      const int64_t r = r0 + rl;
      if (col_in && r < rows) {
        float xv[8], gv[8], o[8];
        load8<F32>(x, r * cols + c0 + cc, xv);
        load8<G_F32>(g, r * cols + c0 + cc, gv);
        const float rs = rstd_s[rl], cf = coef_s[rl];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = xv[j] * rs;
          o[j] = rs * (gv[j] * wv[j] - xh * cf);
          dwv[j] = fmaf(gv[j], xh, dwv[j]);
        }
        store8<F32>(dx, r * cols + c0 + cc, o);
      }
    }
    // the four row groups of the CTA -> one sum per column -> one atomic per column
#pragma unroll
    for (int j = 0; j < 8; ++j) red[grp][(threadIdx.x & 63) * 8 + j] = dwv[j];
    __syncthreads();
    for (int c = threadIdx.x; c < kTileCols; c += 256) {
      if (c0 + c < cols) atomicAdd(dw + c0 + c, (red[0][c] + red[1][c]) + (red[2][c] + red[3][c]));
    }
    __syncthreads();
  }
}

}  // namespace rmsnorm
}  // namespace nvfp4

using namespace nvfp4::rmsnorm;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int nvfp4_rmsnorm_fwd(const void* x, int x_is_f32, const float* weight, int64_t rows, int64_t cols,
                                 float eps, void* h_bf16, float* rstd, const float* signs16, float* maxima2,
                                 int zero_first, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !weight || !h_bf16 || !rstd || !maxima2) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || (cols & 7) != 0) return NVFP4_E_SHAPE;
  if (signs16 != nullptr && (rows & 15) != 0) return NVFP4_E_SHAPE;      // the row transform needs whole blocks
  if ((rows + 15) / 16 > 0x7fffffffLL) return NVFP4_E_LIMIT;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(h_bf16) || (signs16 != nullptr && !aligned16(signs16)) ||
      (reinterpret_cast<uintptr_t>(rstd) & 3u) != 0 || (reinterpret_cast<uintptr_t>(maxima2) & 3u) != 0)
    return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(maxima2, 0, 2 * sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const unsigned grid = (unsigned)((rows + 15) / 16);
  if (x_is_f32)
    rmsnorm_fwd_kernel<true><<<grid, 256, 0, stream>>>(x, weight, rows, cols, eps, static_cast<uint16_t*>(h_bf16), rstd,
                                                       signs16, maxima2);
  else
    rmsnorm_fwd_kernel<false><<<grid, 256, 0, stream>>>(x, weight, rows, cols, eps, static_cast<uint16_t*>(h_bf16), rstd,
                                                        signs16, maxima2);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}

extern "C" int nvfp4_rmsnorm_bwd(const void* x, int x_is_f32, const float* weight, const float* rstd, const void* g,
                                 int g_is_f32, int64_t rows, int64_t cols, void* dx, float* dweight, int zero_first,
                                 void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !weight || !rstd || !g || !dx || !dweight) return NVFP4_E_NULL;
  if (rows <= 0 || cols <= 0 || (cols & 7) != 0) return NVFP4_E_SHAPE;
  if ((rows + kBwdRows - 1) / kBwdRows > 0x7fffffffLL) return NVFP4_E_LIMIT;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(g) || !aligned16(dx) ||
      (reinterpret_cast<uintptr_t>(rstd) & 3u) != 0 || (reinterpret_cast<uintptr_t>(dweight) & 3u) != 0)
    return NVFP4_E_ALIGN;
  if (zero_first && cudaMemsetAsync(dweight, 0, (size_t)cols * sizeof(float), stream) != cudaSuccess)
    return NVFP4_E_LAUNCH;
  const unsigned grid = (unsigned)((rows + kBwdRows - 1) / kBwdRows);
  if (x_is_f32) {
    if (g_is_f32) rmsnorm_bwd_kernel<true, true><<<grid, 256, 0, stream>>>(x, weight, rstd, g, rows, cols, dx, dweight);
    else rmsnorm_bwd_kernel<true, false><<<grid, 256, 0, stream>>>(x, weight, rstd, g, rows, cols, dx, dweight);
  } else {
    if (g_is_f32) rmsnorm_bwd_kernel<false, true><<<grid, 256, 0, stream>>>(x, weight, rstd, g, rows, cols, dx, dweight);
    else rmsnorm_bwd_kernel<false, false><<<grid, 256, 0, stream>>>(x, weight, rstd, g, rows, cols, dx, dweight);
  }
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}
