// Stand-alone driver of the C ABI (no Python, no torch): quantizes two random bf16 operands with the
// single-launch quantizer, runs the FP4 GEMM, reports TFLOP/s and optionally verifies the result on
// the host.  It plays the part of the reference's CUTLASS bench executables
// (cutlass_gemm/nvfp4_gemm_bf16out.cu: --m --n --k --iterations --verify, 20 warm-up runs, CUDA-event
// timing, relative-L2 < 1e-2 and no element more than 5 % off).
//
//   nvfp4_gemm_cli --m 4096 --n 4096 --k 4096 --iterations 50 --verify
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "nvfp4_b200.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return 2; } } while (0)
#define NV(x) do { int c_ = (x); if (c_ != NVFP4_OK) { \
  std::fprintf(stderr, "nvfp4 error %d (%s) at %s:%d\n", c_, nvfp4_status_string(c_), __FILE__, __LINE__); return 3; } } while (0)

static uint16_t f32_to_bf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);                      // round to nearest even
  return (uint16_t)(u >> 16);
}
static float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
static float e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  const float v = e == 0 ? std::ldexp((float)m, -9) : std::ldexp(1.0f + m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}
static const float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

struct Rng {                                            // xorshift + Box-Muller, deterministic
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 1) {}
  double uni() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return ((s >> 11) + 0.5) / 9007199254740992.0; }
  float normal() { return (float)(std::sqrt(-2.0 * std::log(uni())) * std::cos(6.283185307179586 * uni())); }
};

struct Quantized {
  uint8_t *q = nullptr, *sf = nullptr;
  float* pts = nullptr;
  int64_t rows, k, sf_rows, sf_cols;
};

static size_t sf_offset(int64_t r, int64_t c, int64_t col_tiles) {
  const int64_t tile = (r / 128) * col_tiles + c / 4, rr = r % 128;
  return (size_t)(tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + c % 4);
}

int main(int argc, char** argv) {
  int64_t M = 4096, N = 4096, K = 4096;
  int iterations = 50, verify = 0;
  uint64_t seed = 2;
  for (int i = 1; i < argc; ++i) {
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : "0"; };
    if (!std::strcmp(argv[i], "--m")) M = std::atoll(next());
    else if (!std::strcmp(argv[i], "--n")) N = std::atoll(next());
    else if (!std::strcmp(argv[i], "--k")) K = std::atoll(next());
    else if (!std::strcmp(argv[i], "--iterations")) iterations = std::atoi(next());
    else if (!std::strcmp(argv[i], "--seed")) seed = std::strtoull(next(), nullptr, 10);
    else if (!std::strcmp(argv[i], "--verify")) verify = 1;
    else { std::fprintf(stderr, "usage: %s [--m M] [--n N] [--k K] [--iterations I] [--seed S] [--verify]\n", argv[0]); return 1; }
  }
  if (K % 32 != 0) { std::fprintf(stderr, "K must be a multiple of 32\n"); return 1; }
  std::printf("nvfp4_gemm_cli: ABI version %d, M=%lld N=%lld K=%lld\n", nvfp4_version(), (long long)M, (long long)N, (long long)K);

  Rng rng(seed);
  std::vector<uint16_t> ha((size_t)M * K), hb((size_t)N * K);
  for (auto& v : ha) v = f32_to_bf16(rng.normal());
  for (auto& v : hb) v = f32_to_bf16(rng.normal());
  uint16_t *da, *db;
  CK(cudaMalloc(&da, ha.size() * 2)); CK(cudaMalloc(&db, hb.size() * 2));
  CK(cudaMemcpy(da, ha.data(), ha.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(db, hb.data(), hb.size() * 2, cudaMemcpyHostToDevice));
  void* ws; CK(cudaMalloc(&ws, 64)); CK(cudaMemset(ws, 0, 64));

  Quantized qa{nullptr, nullptr, nullptr, M, K, (M + 127) / 128 * 128, (K / 16 + 3) / 4 * 4};
  Quantized qb{nullptr, nullptr, nullptr, N, K, (N + 127) / 128 * 128, (K / 16 + 3) / 4 * 4};
  for (Quantized* q : {&qa, &qb}) {
    CK(cudaMalloc(&q->q, (size_t)q->rows * K / 2)); CK(cudaMalloc(&q->sf, (size_t)q->sf_rows * q->sf_cols));
    CK(cudaMalloc(&q->pts, 4));
  }
  NV(nvfp4_quantize_fused_bf16(da, M, K, K, NVFP4_ROUND_NEAREST, 0, nullptr, 0, 0, qa.q, qa.sf, qa.pts, ws, 64, nullptr));
  NV(nvfp4_quantize_fused_bf16(db, N, K, K, NVFP4_ROUND_NEAREST, 0, nullptr, 0, 0, qb.q, qb.sf, qb.pts, ws, 64, nullptr));
  uint16_t* dd; CK(cudaMalloc(&dd, (size_t)M * N * 2));
  int32_t* status; CK(cudaMalloc(&status, 4)); CK(cudaMemset(status, 0, 4));

  auto run = [&]() { return nvfp4_gemm(qa.q, qa.sf, qa.pts, qb.q, qb.sf, qb.pts, dd, NVFP4_OUT_BF16, M, N, K, N, status, nullptr); };
  for (int i = 0; i < 20; ++i) NV(run());
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0));
  for (int i = 0; i < iterations; ++i) NV(run());
  CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1));
  float ms = 0; CK(cudaEventElapsedTime(&ms, e0, e1));
  int32_t hstatus = 0; CK(cudaMemcpy(&hstatus, status, 4, cudaMemcpyDeviceToHost));
  const double avg_ms = ms / iterations;
  std::printf("  avg runtime %.4f ms, %.1f TFLOP/s, device status word %d\n", avg_ms, 2.0 * M * N * K / avg_ms / 1e9, hstatus);

  int rc = hstatus == 0 ? 0 : 4;
  if (verify) {
    std::vector<uint8_t> aq((size_t)M * K / 2), bq((size_t)N * K / 2), asf((size_t)qa.sf_rows * qa.sf_cols), bsf((size_t)qb.sf_rows * qb.sf_cols);
    float apts, bpts;
    std::vector<uint16_t> hd((size_t)M * N);
    CK(cudaMemcpy(aq.data(), qa.q, aq.size(), cudaMemcpyDeviceToHost)); CK(cudaMemcpy(bq.data(), qb.q, bq.size(), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(asf.data(), qa.sf, asf.size(), cudaMemcpyDeviceToHost)); CK(cudaMemcpy(bsf.data(), qb.sf, bsf.size(), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&apts, qa.pts, 4, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(&bpts, qb.pts, 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(hd.data(), dd, hd.size() * 2, cudaMemcpyDeviceToHost));
    const int64_t ct = (K / 16 + 3) / 4;
    auto deq = [&](const std::vector<uint8_t>& q, const std::vector<uint8_t>& sf, int64_t r, int64_t kk) {
      const uint8_t byte = q[(size_t)r * (K / 2) + kk / 2];
      const uint8_t code = (kk & 1) ? (byte >> 4) : (byte & 15);
      const float v = (code & 8) ? -kE2M1[code & 7] : kE2M1[code & 7];
      return v * e4m3_to_f32(sf[sf_offset(r, kk / 16, ct)]);
    };
    // every element for small problems, otherwise a deterministic sample of 4096 outputs
    const bool all = (double)M * N * K <= 3.0e8;
    const int64_t samples = all ? M * N : 4096;
    Rng pick(seed + 17);
    double err2 = 0, ref2 = 0; int64_t bad = 0;
    for (int64_t s = 0; s < samples; ++s) {
      const int64_t i = all ? s / N : (int64_t)(pick.uni() * M), j = all ? s % N : (int64_t)(pick.uni() * N);
      double acc = 0;
      for (int64_t kk = 0; kk < K; ++kk) acc += (double)deq(aq, asf, i, kk) * deq(bq, bsf, j, kk);
      const double ref = acc * apts * bpts, got = bf16_to_f32(hd[(size_t)i * N + j]);
      err2 += (got - ref) * (got - ref); ref2 += ref * ref;
      if (std::fabs(got - ref) > 0.05 * std::fabs(ref) + 0.02 * std::sqrt(ref2 / (s + 1))) ++bad;
    }
    const double rel = std::sqrt(err2 / (ref2 > 0 ? ref2 : 1));
    const bool passed = rel < 1e-2 && bad == 0;
    std::printf("  verify (%lld outputs, bf16): relative L2 error %.3e, %lld elements more than 5 %% off\n",
                (long long)samples, rel, (long long)bad);
    std::printf("  Disposition: %s\n", passed ? "Passed" : "Failed");
    if (!passed) rc = 5;
  }
  return rc;
}
