/*
 * nvfp4_b200.h -- C ABI of libnvfp4_b200.so, the sm_100a (B200) implementation of the
 * NVFP4 training hot path: per-tensor amax, fused NVFP4 quantizer, block-scaled FP4 GEMM.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless a comment says "host".
 *   - Nothing here allocates or frees device memory; work is enqueued on `stream`
 *     (a cudaStream_t passed as void*; NULL = the legacy default stream) and the call returns
 *     without synchronising.
 *   - Return value: NVFP4_OK (0) or a negative NVFP4_E_* code for an argument or launch error.
 *     Nothing throws.  nvfp4_status_string() names a code.
 *   - Data formats are those of the reference's NVFP4Tensor (nvfp4_gemm.py:45-48):
 *       qdata   uint8 [rows, K/2], low nibble = even k, E2M1 codes (bit 3 = sign)
 *       scales  uint8 E4M3 bits, one per 16 elements along K, stored in 128x4 tiles of
 *               512 bytes: offset = ((r/128)*ceil(K/64) + c/4)*512 + (r%32)*16 + ((r%128)/32)*4 + c%4
 *               buffer size = ceil(rows/128)*128 * ceil(K/64)*4 bytes, padding bytes are zero
 *       pts     float, the per-tensor scale amax / (6 * 448)
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_ABI_VERSION 1

enum {
  NVFP4_OK = 0,
  NVFP4_E_NULL = -1,      /* a required pointer is NULL */
  NVFP4_E_SHAPE = -2,     /* a dimension is not positive, or not a multiple of what the op needs */
  NVFP4_E_ALIGN = -3,     /* a pointer or leading dimension breaks the alignment the op needs */
  NVFP4_E_MODE = -4,      /* unknown mode / flag value */
  NVFP4_E_LAUNCH = -5,    /* the CUDA runtime refused the launch (see cudaGetLastError) */
  NVFP4_E_DRIVER = -6,    /* a driver entry point needed for TMA descriptors is missing */
  NVFP4_E_WORKSPACE = -7, /* workspace too small */
  NVFP4_E_LIMIT = -8      /* size beyond a stated maximum of the entry point */
};

/* Rounding of the E2M1 elements. */
enum { NVFP4_ROUND_NEAREST = 0, NVFP4_ROUND_STOCHASTIC = 1 };
/* Output element type of the GEMM. */
enum { NVFP4_OUT_BF16 = 0, NVFP4_OUT_F32 = 1 };

int nvfp4_version(void);
const char* nvfp4_status_string(int code); /* host string, static storage */

/*
 * Per-tensor absolute maximum of a bf16 matrix x[rows, cols] (row stride `ld` elements),
 * max-merged into *amax (fp32).  With zero_first != 0 the word is cleared on the stream first.
 * rht != 0: the maximum is taken AFTER the 16-point random-sign Hadamard transform of every
 * 16-element block (signs16: 16 floats of +-1), blocks running along the columns
 * (transpose == 0) or along the rows (transpose != 0).
 * Replaces `tf.abs().amax()` of quant_nvfp4 (nvfp4_gemm.py:34-36) and the bf16 amax of
 * quant_nvfp4_cuda (nvfp4_cuda.py:170).  A tensor sharded over several GPUs calls this on the
 * local shard, max-reduces the word across ranks, then calls nvfp4_quantize_bf16.
 */
int nvfp4_amax_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld,
                    int rht, int transpose, const float* signs16,
                    float* amax, int zero_first, void* stream);

/*
 * NVFP4 quantization of a bf16 matrix x[rows, cols] given its per-tensor amax.
 *   transpose == 0: 16-element blocks run along the columns; the result describes the
 *                   [rows, cols] operand (contraction dim = cols).
 *   transpose != 0: blocks run along the rows; the result describes the TRANSPOSED operand
 *                   [cols, rows] (contraction dim = rows), i.e. what the reference gets from
 *                   quant(x.t().contiguous()) (nvfp4_gemm.py:55, nvfp4_train.py:53,77).
 *   mode: NVFP4_ROUND_NEAREST (ties to even) or NVFP4_ROUND_STOCHASTIC (hardware
 *         cvt.rs with a Philox4x32-10 stream: one call per block, counter = (block index,
 *         philox_offset), key = philox_seed; block index = out_row * (K/16) + k/16).
 *   rht != 0: 16-point random-sign Hadamard of every block before scaling (signs16 as above).
 *   amax: the word nvfp4_amax_bf16 produced (same rht/transpose); the global scale
 *         pts = max(amax, 1e-12) / 2688 is computed on the device and written to *pts_out.
 * Outputs: qdata, scales (layouts above; scales padding is zeroed by this call).
 * Requirements: contraction dim % 16 == 0, the other dim % 2 == 0, x 16-byte aligned,
 * ld % 8 == 0.
 * Replaces quant_nvfp4 (nvfp4_gemm.py:30-48), quant_kernel/quant_launch
 * (nvfp4_cuda.py:52-133) and the to_blocked swizzle that follows it (nvfp4_cuda.py:184-185).
 */
int nvfp4_quantize_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld,
                        int transpose, int mode, int rht, const float* signs16,
                        const float* amax, uint64_t philox_seed, uint64_t philox_offset,
                        uint8_t* qdata, uint8_t* scales, float* pts_out, void* stream);

/*
 * nvfp4_quantize_bf16 for a tensor that is one SHARD of a larger one (tensor parallelism): the
 * stochastic-rounding counter of an output block (out_row, k/16) is
 *     out_row * counter_pitch + counter_base + k/16
 * instead of the block's index in the shard, so that a shard draws the random bits the whole tensor
 * would draw for the same elements and the sharded result is bit-identical to the corresponding part
 * of the unsharded one (given the group-reduced amax).  Examples: a [T, N/p] column shard (rank r)
 * quantized along N: pitch = N/16, base = r * (N/p)/16; the same shard quantized transposed (output
 * rows = its N/p columns, blocks along T): pitch = T/16, base = r * (N/p) * (T/16).
 * nvfp4_quantize_bf16 is this call with pitch = K/16 and base = 0.  No counterpart in the reference
 * (it is single-GPU).
 */
int nvfp4_quantize_shard_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              int transpose, int mode, int rht, const float* signs16,
                              const float* amax, uint64_t philox_seed, uint64_t philox_offset,
                              uint64_t counter_pitch, uint64_t counter_base,
                              uint8_t* qdata, uint8_t* scales, float* pts_out, void* stream);

/*
 * The same quantization as nvfp4_amax_bf16 + nvfp4_quantize_bf16(transpose == 0) in ONE launch:
 * a persistent cooperative kernel finds the per-tensor maximum, crosses a grid-wide barrier and
 * quantizes, keeping as much of the tensor as fits in shared memory between the two phases so
 * that HBM is read once.  Bit-identical outputs.  `workspace` is caller scratch of at least
 * nvfp4_quantize_fused_workspace_bytes() bytes (16-byte aligned) that must be ALL ZERO before
 * its first use (one cudaMemset after allocating it); every call that ends normally leaves it
 * ready for the next call (it carries a launch counter and two alternating barrier slots, each
 * launch clearing the slot of the next), so it is reused without clearing.  int32 word 4 of the
 * workspace becomes non-zero when a bounded wait inside the kernel gave up (outputs are then
 * undefined; clear the whole workspace before using it again).  Calls that share a workspace must not
 * overlap on the GPU: use one workspace per stream.  Needs rows * cols / 16 < 2^31.
 * Replaces the whole body of quant_nvfp4_cuda (nvfp4_cuda.py:158-187): amax, pts, quant_launch,
 * to_blocked.
 */
size_t nvfp4_quantize_fused_workspace_bytes(void);
int nvfp4_quantize_fused_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld,
                              int mode, int rht, const float* signs16,
                              uint64_t philox_seed, uint64_t philox_offset,
                              uint8_t* qdata, uint8_t* scales, float* pts_out,
                              void* workspace, size_t workspace_bytes, void* stream);

/*
 * Both quantized layouts of a weight w[rows, cols] (bf16, row stride ld) from ONE read, round to
 * nearest, given the per-tensor amax word (nvfp4_amax_bf16, rht = 0):
 *   qdata_rows / scales_rows   the [rows, cols] operand, blocks along cols  (fprop: quant(w))
 *   qdata_cols / scales_cols   the [cols, rows] operand, blocks along rows  (dgrad: quant(w.t()))
 * two_d == 0: every block has its own 1 x 16 scale: the bytes nvfp4_quantize_bf16 gives with
 *             transpose = 0 and = 1.  Replaces the two weight quantizations of FP4Linear.forward
 *             (nvfp4_train.py:72-78: quant(w) and quant(w.t().contiguous())).
 * two_d != 0: one scale per 16 x 16 tile, used by the row-wise and the column-wise blocks that cross
 *             it, so that both layouts dequantize to the same matrix -- the weight scaling of the
 *             reference's simulator (quantize_nvfp4_2d, nvfp4_validate.py:68-82), here producing real
 *             NVFP4 operands (the reference never ran this mode on FP4 hardware).
 * Requirements: rows % 16 == 0, cols % 16 == 0, 16-byte aligned pointers, ld % 8 == 0.
 */
int nvfp4_quantize_weight_bf16(const void* w, int64_t rows, int64_t cols, int64_t ld, int two_d,
                               const float* amax, uint8_t* qdata_rows, uint8_t* scales_rows,
                               uint8_t* qdata_cols, uint8_t* scales_cols, float* pts_out, void* stream);

/*
 * Both quantized layouts of an ACTIVATION or GRADIENT x[rows, cols] (bf16, row stride ld) from ONE
 * read, each with its own rounding mode, per-tensor maximum, seed and Philox counters:
 *   qdata_rows / scales_rows / pts_rows   x itself, blocks along cols, no Hadamard: the bytes of
 *       nvfp4_quantize_shard_bf16(transpose 0, mode_rows, rht 0, amax_rows, seed_rows)
 *   qdata_cols / scales_cols / pts_cols   x^T [cols, rows], blocks along the rows of x, random-sign
 *       Hadamard along those rows: the bytes of nvfp4_quantize_shard_bf16(transpose 1, mode_cols,
 *       rht 1, amax_cols, seed_cols)
 * amax_cols is the maximum AFTER the Hadamard transform (nvfp4_amax_both_bf16 gives both maxima
 * from one read; a fused producer may know them already).  counters4 = {pitch_rows, base_rows,
 * pitch_cols, base_cols} as in nvfp4_quantize_shard_bf16, or NULL for a whole tensor.
 * Requirements: rows % 16 == 0, cols % 16 == 0, 16-byte aligned pointers, ld % 8 == 0.
 * Replaces the pairs quant(x) / quant(x.t(), rht) and quant(gy, SR) / quant(gy.t(), rht, SR) of
 * FP4LinearFn (nvfp4_train.py:36-38, 44-55), which read the tensor once per layout (and once more
 * per maximum).
 */
int nvfp4_quantize_dual_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, int mode_rows, int mode_cols,
                             const float* signs16, const float* amax_rows, const float* amax_cols,
                             uint64_t seed_rows, uint64_t seed_cols, uint64_t offset, const uint64_t* counters4,
                             uint8_t* qdata_rows, uint8_t* scales_rows, float* pts_rows,
                             uint8_t* qdata_cols, uint8_t* scales_cols, float* pts_cols, void* stream);

/*
 * maxima2[0] = max|x| and maxima2[1] = max|RHT_rows(x)| (16-point random-sign Hadamard over groups
 * of 16 rows) from one read of x[rows, cols]; rows % 16 == 0, cols even.  The two words are what
 * nvfp4_amax_bf16 gives with (rht 0) and with (rht 1, transpose 1).
 */
int nvfp4_amax_both_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld, const float* signs16,
                         float* maxima2, int zero_first, void* stream);

/*
 * nvfp4_quantize_fused_bf16 for callers that cannot allocate device memory where they call from
 * (a C / FFI binding inside a runtime that gave all of HBM to its own pool, a callback that must
 * not hit cudaMalloc's implicit synchronisation): the kernel's scratch is a 256-byte device array
 * inside the library instead of a caller workspace, so the caller passes inputs and outputs only.
 * The call allocates nothing.  Same outputs, bit for bit.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the array: calls that can overlap on the GPU (different
 *     streams) race on it.  Calls on one stream are safe; each call clears what it needs.
 *   - Limit: rows * cols / 16 <= 2^31 - 1, otherwise NVFP4_E_LIMIT.
 *   - A bounded wait inside the kernel that gives up (outputs then undefined) sets an error word in
 *     the library's array; the call itself has long returned NVFP4_OK by then.  The word stays set
 *     across later calls until nvfp4_quantize_static_status reads and clears it.
 * This entry point has no counterpart in the reference.
 */
int nvfp4_quantize_static_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld,
                               int mode, int rht, const float* signs16,
                               uint64_t philox_seed, uint64_t philox_offset,
                               uint8_t* qdata, uint8_t* scales, float* pts_out, void* stream);

/*
 * Error word of nvfp4_quantize_static_bf16 on the current device, copied to *host_out (HOST
 * pointer): 0 = every call since the last clear ran to its end, 1 = a grid barrier gave up,
 * 2 = a bulk copy never landed.  The copy is enqueued on `stream` behind the calls already there,
 * and this function waits for it (cudaStreamSynchronize), so *host_out is valid on return; with
 * clear != 0 the word is zeroed behind the copy.  Allocates nothing.  Do not call it during stream
 * capture.  No counterpart in the reference (the workspace entry point exposes the same word as
 * int32 word 4 of the caller's workspace).
 */
int nvfp4_quantize_static_status(int32_t* host_out, int clear, void* stream);

/*
 * Block-scaled FP4 GEMM  D[M, N] = (A . sfA) (B . sfB)^T * (*a_pts) * (*b_pts)
 * with fp32 accumulation on the tcgen05 tensor cores.
 *   a_q [M, K/2], b_q [N, K/2]: packed E2M1, both K-major; a_sf, b_sf: swizzled E4M3 scales;
 *   a_pts, b_pts: device floats; d: [M, ldd] bf16 or fp32.
 *   status: optional device int32; a bounded wait inside the kernel that gives up writes a
 *   non-zero code there (the call itself still returns NVFP4_OK).
 * Requirements: K % 32 == 0 (16-byte rows for TMA), a_q/b_q/d 16-byte aligned.
 * Replaces torchao's _addmm_nvfp4_dispatch -> torch._scaled_mm as called at
 * nvfp4_gemm.py:57 and nvfp4_cuda.py:193,200.
 */
int nvfp4_gemm(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts,
               const uint8_t* b_q, const uint8_t* b_sf, const float* b_pts,
               void* d, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldd,
               int32_t* status, void* stream);

/*
 * nvfp4_gemm that also leaves max|D| in *d_amax_out (fp32 device word; the call zeroes it on the
 * stream first): the maximum over the stored output after its rounding to the output type, i.e.
 * what nvfp4_amax_bf16 would find by reading D again.  A quantizer that takes D next
 * (nvfp4_quantize_fused_bf16 with this word as amax_in) then needs one pass, not two.  The K split
 * of small fp32 outputs is not used with this entry point.
 * Replaces the `tf.abs().amax()` pass of quant_nvfp4 (nvfp4_gemm.py:34-36) over a GEMM output, e.g.
 * between `up` and `down` at nvfp4_train.py:111-123; the quantization overhead it removes is the one
 * the reference names at README.md:80-83.
 */
int nvfp4_gemm_amax(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts,
                    const uint8_t* b_q, const uint8_t* b_sf, const float* b_pts,
                    void* d, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldd,
                    float* d_amax_out, int32_t* status, void* stream);

/*
 * The same GEMM with an NVFP4 OUTPUT for chained GEMMs: every output row is rounded to bf16 and
 * quantized in blocks of 16 along N (round to nearest) inside the epilogue, with the per-tensor
 * maximum *d_amax supplied by the caller (a value known from the previous step or a bound; elements
 * beyond it saturate).  Outputs: d_q [M, N/2] packed E2M1, d_sf the swizzled E4M3 scales of the
 * [M, N] operand, *d_pts = max(*d_amax, 1e-12) / 2688 -- exactly what nvfp4_quantize_bf16 would make
 * of the bf16 output of nvfp4_gemm with the same amax word, without that tensor ever reaching
 * memory.  Requirements of nvfp4_gemm, and N % 16 == 0.
 * Counterpart in the reference: the E2M1 output + scale-factor epilogue of its CUTLASS example
 * (cutlass_gemm/nvfp4_gemm.cu:106-108, :149-154: LinCombBlockScaleFactor), which takes the
 * normalisation constant from the caller in the same way.
 */
int nvfp4_gemm_fp4out(const uint8_t* a_q, const uint8_t* a_sf, const float* a_pts,
                      const uint8_t* b_q, const uint8_t* b_sf, const float* b_pts,
                      int64_t M, int64_t N, int64_t K, const float* d_amax,
                      uint8_t* d_q, uint8_t* d_sf, float* d_pts, int32_t* status, void* stream);

/*
 * Kernel choice of nvfp4_gemm for this process: 0 = automatic (the default), 1 = always the
 * one-CTA 128x256 kernel, 2 = always the persistent two-CTA 256x256 kernel.  For tuning and tests;
 * results are the same to rounding of the accumulation order.  No counterpart in the reference.
 */
int nvfp4_gemm_set_mode(int mode);

/*
 * Producer fusion in front of the quantizer: SwiGLU and its backward in one pass each that also
 * leaves the per-tensor maxima the following quantizations need, so that those run as one
 * nvfp4_quantize_bf16 call with the amax given (no separate amax pass).
 *   fwd: out = silu(gate) * up; maxima2[0] = max|out|, maxima2[1] = max|RHT(out)| where RHT is the
 *        16-point random-sign Hadamard along the ROW dimension in groups of 16 rows (the transform of
 *        the transposing quantizer, nvfp4_quantize_bf16 with transpose = 1, rht = 1).
 *   bwd: dgate = dout * up * silu'(gate), dup = dout * silu(gate); maxima4 = {max|dgate|,
 *        max|RHT(dgate)|, max|dup|, max|RHT(dup)|}.
 * All tensors [rows, cols] bf16 row-major (cols even; inputs with leading dimension ld_in, outputs
 * ld_out).  fp32 arithmetic, one rounding to bf16; the maxima are taken over the rounded values with
 * the operations of nvfp4_amax_bf16, so they equal what nvfp4_amax_bf16 would return for the stored
 * tensors.  signs16 == NULL skips the RHT maxima (then rows need not be a multiple of 16).
 * zero_first != 0 clears the maxima first; with 0 the call max-accumulates into them.
 * The reference computes these with torch element-wise kernels; it has no fused counterpart
 * (its models use a squared-ReLU MLP, nvfp4_train.py:120-123; SwiGLU is its FFN benchmark block).
 */
int nvfp4_swiglu_fwd_bf16(const void* gate, const void* up, int64_t rows, int64_t cols, int64_t ld_in,
                          void* out, int64_t ld_out, const float* signs16, float* maxima2,
                          int zero_first, void* stream);
int nvfp4_swiglu_bwd_bf16(const void* gate, const void* up, const void* dout, int64_t rows, int64_t cols,
                          int64_t ld_in, void* dgate, void* dup, int64_t ld_out, const float* signs16,
                          float* maxima4, int zero_first, void* stream);

/*
 * nvfp4_swiglu_bwd_bf16 with its own leading dimension for dout: gate and up may then be the two
 * halves of one [rows, 2 cols] tensor (a fused gate|up projection, ld_in = 2 cols) while dout is a
 * plain [rows, cols] tensor, and dgate / dup the two halves of one [rows, 2 cols] gradient
 * (ld_out = 2 cols) that the fused projection's backward consumes as it is.
 */
int nvfp4_swiglu_bwd_strided_bf16(const void* gate, const void* up, const void* dout, int64_t rows, int64_t cols,
                                  int64_t ld_in, int64_t ld_dout, void* dgate, void* dup, int64_t ld_out,
                                  const float* signs16, float* maxima4, int zero_first, void* stream);

/*
 * The same producer fusion for the squared-ReLU MLP of the reference's models
 * (nvfp4_train.py:120-123): out = relu(x)^2, and backward dx = 2 relu(x) * dout, each with
 * maxima2 = {max|result|, max|RHT_rows(result)|} as above.  Only for 16-byte rows (cols, ld_in,
 * ld_out multiples of 8, 16-byte aligned pointers); NVFP4_E_ALIGN otherwise.  No fused
 * counterpart in the reference (torch element-wise kernels there).
 */
int nvfp4_relu2_fwd_bf16(const void* x, int64_t rows, int64_t cols, int64_t ld_in, void* out, int64_t ld_out,
                         const float* signs16, float* maxima2, int zero_first, void* stream);
int nvfp4_relu2_bwd_bf16(const void* x, const void* dout, int64_t rows, int64_t cols, int64_t ld_in,
                         void* dx, int64_t ld_out, const float* signs16, float* maxima2, int zero_first,
                         void* stream);

/*
 * RMSNorm as a producer for the quantizer: h = x * rsqrt(mean(x^2, row) + eps) * weight, written once as
 * bf16 [rows, cols] (contiguous), with rstd[rows] for the backward and maxima2 = {max|h|,
 * max|RHT_rows(h)|} of the ROUNDED result (the second only if signs16 is given; rows % 16 == 0 then).
 * Every NVFP4 quantization of h that follows (the q, k, v / up projections in both layouts) is then one
 * pass with the maximum given.  x is fp32 (x_is_f32 != 0) or bf16, contiguous; cols % 8 == 0; pointers
 * 16-byte aligned.  Backward: dx (in x's type) and dweight (fp32 [cols], zeroed first if zero_first,
 * accumulated with atomics) from g = dL/dh (bf16, or fp32 when g_is_f32 != 0).
 * Call site in the reference: nn.RMSNorm n1 / n2 in front of the FP4 projections
 * (nvfp4_train.py:105,114-122); there each FP4Linear searches the maximum of the same tensor again.
 */
int nvfp4_rmsnorm_fwd(const void* x, int x_is_f32, const float* weight, int64_t rows, int64_t cols, float eps,
                      void* h_bf16, float* rstd, const float* signs16, float* maxima2, int zero_first,
                      void* stream);
int nvfp4_rmsnorm_bwd(const void* x, int x_is_f32, const float* weight, const float* rstd, const void* g,
                      int g_is_f32, int64_t rows, int64_t cols, void* dx, float* dweight, int zero_first,
                      void* stream);

/*
 * Test hooks of the bounded waits, process-wide, for the launches that follow.  Every spin inside
 * the kernels (grid barrier, mbarrier) gives up after a time limit, records a code (workspace word
 * 4 / the static error word for the quantizer, *status for the GEMM) and lets the kernel drain and
 * return; these hooks let a test make that happen in a millisecond instead of never:
 *   wait_limit_ns                    the limit (0 = the default, 2 s)
 *   quantizer_extra_arrivals         the quantizer's grid barrier expects this many arrivals more
 *                                    than the grid has CTAs, so it can only run out (code 1)
 *   gemm_drop_first_scale_arrival    != 0: the scale-factor warps never announce K slice 0, so the
 *                                    MMA issuer's first wait runs out (code 2) and every role leaves
 * nvfp4_test_hooks(0, 0, 0) restores normal operation.  No GPU fault, trap or endless loop is
 * involved: the kernels return through their documented give-up path.  No counterpart in the
 * reference.
 */
int nvfp4_test_hooks(uint64_t wait_limit_ns, int quantizer_extra_arrivals, int gemm_drop_first_scale_arrival);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
