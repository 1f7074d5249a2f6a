"""FP4 matmul wrappers with the reference's signatures (nvfp4_gemm.py:51-57,
nvfp4_cuda.py:190-200) on top of the tcgen05 block-scaled GEMM."""
from __future__ import annotations

import torch

from . import _lib
from .quant import quant_nvfp4, _stream
from .tensor import NVFP4Tensor

_STATUS = {}


def _status_word(device):
    if device not in _STATUS:
        _STATUS[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[device]


def gemm_status(device=None) -> int:
    """Device status word of the GEMM kernels on `device`: 0, or the code of the first bounded
    wait that gave up.  Reading it synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return int(_status_word(device).item())


def nvfp4_mm(a: NVFP4Tensor, b: NVFP4Tensor, out_dtype=None, out=None, amax_out=None) -> torch.Tensor:
    """a @ b for a = quant(A) [M, K] and b = quant(B.t()).t() (a transposed view whose storage is
    [N, K]): the call shape of torchao's _addmm_nvfp4_dispatch(a, b, aten.mm) at nvfp4_gemm.py:57.
    fp32 accumulation; result in out_dtype (default: a's original dtype, bf16 unless fp32).
    amax_out: optional 1-element fp32 CUDA tensor that the GEMM epilogue fills with max|result|, so
    that quant_nvfp4(result, amax=amax_out) needs no pass of its own to find it."""
    if a._transposed or not b._transposed:
        raise ValueError("nvfp4_mm expects a = quant(A) and b = quant(B.t()).t()")
    m, k2 = a.qdata.shape
    n, k2b = b.qdata.shape
    if k2 != k2b:
        raise ValueError(f"contraction mismatch: {k2 * 2} vs {k2b * 2}")
    if out is not None:
        if tuple(out.shape) != (m, n) or out.stride(1) != 1 or (out_dtype is not None and out.dtype != out_dtype):
            raise ValueError("out must be [M, N] with unit column stride and the requested dtype")
        out_dtype = out.dtype
    if out_dtype is None:
        out_dtype = torch.float32 if a.orig_dtype == torch.float32 else torch.bfloat16
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    if amax_out is not None and (amax_out.dtype != torch.float32 or amax_out.numel() != 1):
        raise ValueError("amax_out must be a 1-element float32 tensor")
    dev = _lib.cuda_device_of(a.qdata, a.scale, a.per_tensor_scale, b.qdata, b.scale, b.per_tensor_scale, out, amax_out)
    d = out if out is not None else torch.empty((m, n), dtype=out_dtype, device=dev)
    args = (a.qdata.data_ptr(), a.scale.data_ptr(), a.per_tensor_scale.data_ptr(),
            b.qdata.data_ptr(), b.scale.data_ptr(), b.per_tensor_scale.data_ptr(),
            d.data_ptr(), _lib.OUT_F32 if out_dtype == torch.float32 else _lib.OUT_BF16,
            m, n, k2 * 2, d.stride(0))
    with torch.cuda.device(dev):                   # the C side launches on the current device
        if amax_out is None:
            code = _lib.lib().nvfp4_gemm(*args, _status_word(dev).data_ptr(), _stream(dev))
        else:
            code = _lib.lib().nvfp4_gemm_amax(*args, amax_out.data_ptr(), _status_word(dev).data_ptr(), _stream(dev))
    _lib.check(code, "nvfp4_gemm")
    return d


def nvfp4_mm_fp4out(a: NVFP4Tensor, b: NVFP4Tensor, out_amax: torch.Tensor) -> NVFP4Tensor:
    """a @ b delivered as an NVFP4Tensor [M, N] quantized along N (round to nearest) inside the GEMM
    epilogue, for a GEMM that feeds another one: equal to quant_nvfp4(nvfp4_mm(a, b, bfloat16),
    amax=out_amax) without the bf16 tensor in memory.  out_amax: 1-element fp32 CUDA tensor, the
    per-tensor maximum to scale with (known from an earlier step, or a bound: larger values saturate)."""
    from .tensor import BLK, swizzled_scale_dims
    if a._transposed or not b._transposed:
        raise ValueError("nvfp4_mm_fp4out expects a = quant(A) and b = quant(B.t()).t()")
    m, k2 = a.qdata.shape
    n, k2b = b.qdata.shape
    if k2 != k2b:
        raise ValueError(f"contraction mismatch: {k2 * 2} vs {k2b * 2}")
    if n % BLK != 0:
        raise AssertionError(f"N={n} must be divisible by {BLK}")
    dev = _lib.cuda_device_of(a.qdata, a.scale, a.per_tensor_scale, b.qdata, b.scale, b.per_tensor_scale, out_amax)
    sm, sk = swizzled_scale_dims(m, n)
    qd = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
    sc = torch.empty((sm, sk), dtype=torch.uint8, device=dev)
    pts = torch.empty((), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        code = _lib.lib().nvfp4_gemm_fp4out(
            a.qdata.data_ptr(), a.scale.data_ptr(), a.per_tensor_scale.data_ptr(),
            b.qdata.data_ptr(), b.scale.data_ptr(), b.per_tensor_scale.data_ptr(),
            m, n, k2 * 2, out_amax.data_ptr(), qd.data_ptr(), sc.data_ptr(), pts.data_ptr(),
            _status_word(dev).data_ptr(), _stream(dev))
    _lib.check(code, "nvfp4_gemm_fp4out")
    return NVFP4Tensor(qd, sc.view(torch.float8_e4m3fn), BLK, torch.bfloat16, pts, True)


def _quant_rhs(B, stochastic, rht, H, signs, seed):
    """quant(B.t()) for B [K, N] without materialising the transpose."""
    if B.stride(0) == 1 and B.dim() == 2:           # B is itself a transposed view: B.t() is row-major
        return quant_nvfp4(B.t(), stochastic, rht, H, signs, seed)
    return quant_nvfp4(B, stochastic, rht, H, signs, seed, transpose=True)


def fp4_matmul(A, B, sr_a=False, sr_b=False, rht=False, H=None, signs=None, seed=None, out_dtype=None):
    """A @ B with both operands quantized along K (A: [M, K], B: [K, N]); nvfp4_gemm.py:51-57."""
    a = quant_nvfp4(A, sr_a, rht, H, signs, seed)
    bt = _quant_rhs(B, sr_b, rht, H, signs, seed)
    return nvfp4_mm(a, bt.t(), out_dtype)


fp4_matmul_cuda = fp4_matmul         # nvfp4_cuda.py:190-193


def fp4_mm_preqB(A, Bq_t, sr_a=False, rht=False, H=None, signs=None, seed=None, out_dtype=None):
    """A @ B where Bq_t = quant(B.t()) was made earlier (a constant weight quantized once and
    reused); nvfp4_cuda.py:196-200."""
    a = quant_nvfp4(A, sr_a, rht, H, signs, seed)
    return nvfp4_mm(a, Bq_t.t(), out_dtype)
