// nvfp4_gemm: argument checks, tensor maps, kernel choice (C ABI; declared in include/nvfp4_b200.h).
#include "gemm_common.cuh"

namespace nvfp4 { namespace gemm3 {
int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const gemm::Params& p,
                cudaStream_t stream);
}}
namespace nvfp4 { namespace gemm {
int launch_1cta(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const Params& p,
                cudaStream_t stream);
}}

#include <atomic>

static std::atomic<int> g_gemm_mode{0};
// test hooks (nvfp4_test_hooks): the wait limit of the next launches and the dropped arrival
static std::atomic<unsigned long long> g_gemm_wait_ns{0};
static std::atomic<int> g_gemm_drop_arrival{0};
namespace nvfp4 { namespace gemm {
void set_test_hooks(unsigned long long wait_ns, int drop_arrival) {
  g_gemm_wait_ns.store(wait_ns, std::memory_order_relaxed);
  g_gemm_drop_arrival.store(drop_arrival, std::memory_order_relaxed);
}
}}
extern "C" int nvfp4_gemm_set_mode(int mode) {
  if (mode < 0 || mode > 2) return NVFP4_E_MODE;
  g_gemm_mode.store(mode, std::memory_order_relaxed);
  return NVFP4_OK;
}

// Automatic choice: the persistent pair kernel (mode 2), which measured fastest on every shape with
// more than one row tile; the one-CTA kernel (mode 1) when M <= 128 (a pair would compute 128 rows of
// padding) and for the split-K case below.  Modes 1 and 2 force a kernel, for tuning and tests.
namespace nvfp4 { namespace gemm {
__global__ void pts_from_amax_kernel(const float* __restrict__ amax, float* __restrict__ pts) {
  *pts = __fdiv_rn(fmaxf(*amax, kAmaxFloor), kGlobalDiv);
}
int launch_pts_from_amax(const float* amax, float* pts, cudaStream_t stream) {
  pts_from_amax_kernel<<<1, 1, 0, stream>>>(amax, pts);
  return cudaGetLastError() == cudaSuccess ? NVFP4_OK : NVFP4_E_LAUNCH;
}
}}

static int gemm_any(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts, const uint8_t* b_q,
                    const uint8_t* b_sf, const float* b_pts, void* d, int out_dtype, int64_t M, int64_t N,
                    int64_t K, int64_t ldd, uint8_t* d_sf, const float* d_amax, float* d_amax_out, int32_t* status,
                    void* stream_) {
  using namespace nvfp4::gemm;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool fp4_out = d_sf != nullptr;
  if (!a_q || !a_sf || !a_pts || !b_q || !b_sf || !b_pts || !d) return NVFP4_E_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (K & 31) != 0 || ldd < N) return NVFP4_E_SHAPE;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return NVFP4_E_SHAPE;
  if (out_dtype != NVFP4_OUT_BF16 && out_dtype != NVFP4_OUT_F32) return NVFP4_E_MODE;
  auto mis = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (mis(a_q, 16) || mis(b_q, 16) || mis(a_sf, 16) || mis(b_sf, 16) || mis(d, 16)) return NVFP4_E_ALIGN;
  // split K (one-CTA kernel only, see below) when a small fp32 output would leave most SMs idle
  const int64_t tiles_1cta = ((N + 255) / 256) * ((M + 127) / 128), slices = (K + 255) / 256;
  // (partial sums have no maximum of their own: no split when the caller wants max|D|)
  const bool want_split = out_dtype == NVFP4_OUT_F32 && tiles_1cta <= 74 && slices >= 16 && d_amax_out == nullptr;
  if (d_amax_out != nullptr) {
    if (fp4_out) return NVFP4_E_MODE;
    if (cudaMemsetAsync(d_amax_out, 0, sizeof(float), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  }
  const int forced = g_gemm_mode.load(std::memory_order_relaxed);
  const int mode = forced != 0 ? forced : ((M > 128 && !want_split) ? 2 : 1);
  const bool pair = mode == 2;
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, a_q, M, K, 128) || !make_operand_map(&map_b, b_q, N, K, pair ? 128 : 256))
    return NVFP4_E_DRIVER;
  Params p{a_sf, b_sf, a_pts, b_pts, d, M, N, K, ldd, out_dtype == NVFP4_OUT_F32 ? 1 : 0, status, 1, 0,
           g_gemm_wait_ns.load(std::memory_order_relaxed), g_gemm_drop_arrival.load(std::memory_order_relaxed),
           d_sf, d_amax, fp4_out ? 1 : 0, d_amax_out};
  // Split K when a small fp32 output (the weight gradient: few tiles, K = tokens) would leave most SMs
  // idle: the CTAs of a tile add their partial sums into the zeroed output.  Summation order then
  // varies from run to run in the last bits, so it is used only where it pays: fewer tiles than half
  // the SMs and at least 16 K slices (8 or more per CTA).
  if (!pair && want_split) {
    {
      int64_t s = 148 / tiles_1cta;
      if (s > slices / 8) s = slices / 8;              // at least 8 slices per CTA
      if (s > 1) {
        p.splits = (int)s;
        cudaError_t e = (ldd == N) ? cudaMemsetAsync(d, 0, (size_t)M * N * 4, stream)
                                   : cudaMemset2DAsync(d, (size_t)ldd * 4, 0, (size_t)N * 4, (size_t)M, stream);
        if (e != cudaSuccess) return NVFP4_E_LAUNCH;
      }
    }
  }
  // The epilogue stores through TMA when the row pitch allows a tensor map (a multiple of 16 bytes)
  // and the output is written, not accumulated into.
  CUtensorMap map_d = map_a;                                   // placeholder when unused
  if (p.splits == 1 && !fp4_out && (ldd * (p.out_f32 ? 4 : 2)) % 16 == 0) {
    if (!make_output_map(&map_d, d, M, N, ldd, p.out_f32 != 0)) return NVFP4_E_DRIVER;
    p.tma_store = 1;
  }
  return pair ? nvfp4::gemm3::launch_pair(map_a, map_b, map_d, p, stream) : launch_1cta(map_a, map_b, map_d, p, stream);
}

extern "C" int nvfp4_gemm(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts, const uint8_t* b_q,
                          const uint8_t* b_sf, const float* b_pts, void* d, int out_dtype, int64_t M, int64_t N,
                          int64_t K, int64_t ldd, int32_t* status, void* stream_) {
  return gemm_any(a_q, a_sf, a_pts, b_q, b_sf, b_pts, d, out_dtype, M, N, K, ldd, nullptr, nullptr, nullptr, status,
                  stream_);
}

extern "C" int nvfp4_gemm_amax(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts, const uint8_t* b_q,
                               const uint8_t* b_sf, const float* b_pts, void* d, int out_dtype, int64_t M, int64_t N,
                               int64_t K, int64_t ldd, float* d_amax_out, int32_t* status, void* stream_) {
  if (!d_amax_out) return NVFP4_E_NULL;
  return gemm_any(a_q, a_sf, a_pts, b_q, b_sf, b_pts, d, out_dtype, M, N, K, ldd, nullptr, nullptr, d_amax_out, status,
                  stream_);
}

extern "C" int nvfp4_gemm_fp4out(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts, const uint8_t* b_q,
                                 const uint8_t* b_sf, const float* b_pts, int64_t M, int64_t N, int64_t K,
                                 const float* d_amax, uint8_t* d_q, uint8_t* d_sf, float* d_pts, int32_t* status,
                                 void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!d_amax || !d_q || !d_sf || !d_pts) return NVFP4_E_NULL;
  if ((N & 15) != 0) return NVFP4_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(d_sf) & 15u) != 0) return NVFP4_E_ALIGN;
  // padding of the tiled scale buffer reads as zero; the per-tensor scale is the given maximum / 2688
  const int64_t sm = (M + 127) / 128 * 128, sk = (N / 16 + 3) / 4 * 4;
  if ((sm != M || sk != N / 16) && cudaMemsetAsync(d_sf, 0, (size_t)(sm * sk), stream) != cudaSuccess) return NVFP4_E_LAUNCH;
  const int rc = gemm_any(a_q, a_sf, a_pts, b_q, b_sf, b_pts, d_q, NVFP4_OUT_BF16, M, N, K, N, d_sf, d_amax, nullptr, status,
                          stream_);
  if (rc != NVFP4_OK) return rc;
  return nvfp4::gemm::launch_pts_from_amax(d_amax, d_pts, stream);
}
