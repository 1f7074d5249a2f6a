// Pieces shared by the single-launch quantizer kernels (quantize_fused.cu, quantize_tiled.cu): the
// 64-byte workspace, the exact block-scale shortcut, packed fp32 helpers, the E2M1 conversions,
// Philox with host-made round keys and the in-register Hadamard butterfly.
#pragma once
#include "common.cuh"
#include "nvfp4_b200.h"

namespace nvfp4 {
namespace fused {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // default of the bounded waits: 2 s

struct Workspace {          // 64 bytes of caller scratch, all zero before the first call.  Launch number e
  float amax[2];            // (counted in `epoch`) uses slot e & 1 of the maximum and of the arrival
  unsigned int arrived[2];  // counter and, once its grid barrier has opened, zeroes the other slot for
  int error;                // launch e + 1 and bumps `epoch`: nothing is left to do at the end of the
  unsigned int epoch;       // kernel.  error is sticky: 1 = the grid barrier gave up, 2 = a bulk copy
                            // never landed.
  unsigned long long start;      // diagnostics: globaltimer of CTA 0 at its start, then nanoseconds from
  unsigned int after[4];         // there to: streamed amax done, stashed amax done, barrier open, CTA 0 end
  unsigned long long last_end;   // latest end over all CTAs of the last launch
  unsigned int pad[2];
};
static_assert(sizeof(Workspace) == 64, "the ABI promises a 64-byte workspace");

struct FastDiv {            // n / d for 0 <= n < 2^31 and a fixed d, as one mulhi and a shift
  uint32_t mul, shift, d;
};

__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
  return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shift);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

struct Scale {
  float pts, inv_pts, c;     // c ~ 1 / (6 pts), only used for the checked shortcut
};

// E4M3 byte of clamp((amax_b / 6) / pts, 2^-6, 448), exactly as the two divisions give it.
__device__ __forceinline__ uint32_t block_scale_byte(float amax_b, const Scale& s) {
  const float t = amax_b * s.c;
  const float lo = fmaxf(t * 0.99999905f, kE4M3Eps);      // t (1 - 2^-20)
  const float hi = fmaxf(t * 1.00000095f, kE4M3Eps);      // t (1 + 2^-20)
  uint16_t both;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(both) : "f"(hi), "f"(lo));
  const uint32_t b_lo = both & 0xffu, b_hi = both >> 8;
  if (b_lo == b_hi) return b_lo;       // the exact quotient lies between lo and hi: same byte
  const float sbs = fminf(fmaxf(__fdiv_rn(__fdiv_rn(amax_b, kF4Max), s.pts), kE4M3Eps), kE4M3Max);
  return f32_to_e4m3(sbs);
}

__device__ __forceinline__ float amax_packed8(const uint32_t (&w)[8]) {
  // max |x| over 16 bf16 values held as 8 packed pairs; bf16 magnitudes order like their bits,
  // so the maximum is taken per 16-bit half with the three-input SIMD max
  const uint32_t k = 0x7fff7fffu;
  const uint32_t a = __vimax3_u16x2(w[0] & k, w[1] & k, w[2] & k);
  const uint32_t b = __vimax3_u16x2(w[3] & k, w[4] & k, w[5] & k);
  const uint32_t c = __vimax3_u16x2(w[6] & k, w[7] & k, a);
  const uint32_t m = __vimax3_u16x2(b, c, 0u);
  return __uint_as_float(max(m << 16, m & 0xffff0000u));
}

// ---- packed fp32 helpers (sm_100 has two-wide fp32 add / mul) ----------------------------------
__device__ __forceinline__ void mul2(float a, float b, float s, float& d0, float& d1) {
  asm("{.reg .b64 p, q, r; mov.b64 p, {%2, %3}; mov.b64 q, {%4, %4}; mul.rn.f32x2 r, p, q; mov.b64 {%0, %1}, r;}"
      : "=f"(d0), "=f"(d1) : "f"(a), "f"(b), "f"(s));
}
// (a, b) * s + 0: the product with an exact zero made +0 (-0 * s = -0, and -0 + +0 = +0), everything
// else unchanged -- what the reference's matmul with H leaves, whose accumulator starts at +0
__device__ __forceinline__ void mul2_poszero(float a, float b, float s, float& d0, float& d1) {
  asm("{.reg .b64 p, q, r, z; mov.b64 p, {%2, %3}; mov.b64 q, {%4, %4}; mov.b64 z, {%5, %5};"
      " fma.rn.f32x2 r, p, q, z; mov.b64 {%0, %1}, r;}"
      : "=f"(d0), "=f"(d1) : "f"(a), "f"(b), "f"(s), "f"(0.0f));
}
// (a0, a1) and (b0, b1) -> sums into a, differences into b
__device__ __forceinline__ void addsub2(float& a0, float& a1, float& b0, float& b1) {
  float s0, s1, d0, d1;
  asm("{.reg .b64 p, q, r, t; mov.b64 p, {%4, %5}; mov.b64 q, {%6, %7}; add.rn.f32x2 r, p, q; sub.rn.f32x2 t, p, q;"
      " mov.b64 {%0, %1}, r; mov.b64 {%2, %3}, t;}"
      : "=f"(s0), "=f"(s1), "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
  a0 = s0; a1 = s1; b0 = d0; b1 = d1;
}
// eight fp32 -> eight E2M1 codes in one word, round to nearest even; d[0] in the lowest nibble
__device__ __forceinline__ uint32_t e2m1x8_rn(const float* d) {
  uint32_t w;
  asm("{.reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};}"
      : "=r"(w) : "f"(d[0]), "f"(d[1]), "f"(d[2]), "f"(d[3]), "f"(d[4]), "f"(d[5]), "f"(d[6]), "f"(d[7]));
  return w;
}

struct PhiloxKeys { uint32_t k[10][2]; };     // round keys key + r * (0x9E3779B9, 0xBB67AE85), host-made

__device__ __forceinline__ Philox4 philox_rounds(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                 const PhiloxKeys& ks) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ ks.k[r][0];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ ks.k[r][1];
    c1 = (uint32_t)p1; c3 = (uint32_t)p0; c0 = n0; c2 = n2;
  }
  return Philox4{c0, c1, c2, c3};
}

// 16 bf16 (8 words) -> fp32 v[16].  RHT: signs are applied by flipping sign bits of the packed
// words, then the 16-point butterfly runs (strides 1, 2, 4, 8; the last three two lanes at a time);
// the result is 4x the Hadamard transform (the 1/4 is folded into the scale by the caller).
// An exact zero can leave the butterfly as -0 (a - b with a = -0, b = +0: a zero input under a
// negative sign beside a subtree that cancels); the caller's scaling turns every exact zero into +0.
template <bool RHT>
__device__ __forceinline__ void expand(const uint32_t (&w)[8], const uint32_t (&sm)[8], float (&v)[16]) {
  if constexpr (!RHT) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[2 * j] = bf16_lo(w[j]); v[2 * j + 1] = bf16_hi(w[j]); }
    return;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t x = w[j] ^ sm[j];
    const float lo = bf16_lo(x), hi = bf16_hi(x);
    v[2 * j] = lo + hi;
    v[2 * j + 1] = lo - hi;
  }
#pragma unroll
  for (int s = 2; s < 16; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      if ((i & s) == 0) addsub2(v[i], v[i + 1], v[i | s], v[(i | s) + 1]);
    }
  }
}

}  // namespace fused
}  // namespace nvfp4
