"""NVFP4 quantizer: the reference's `quant_nvfp4` / `quant_nvfp4_cuda` surface
(nvfp4_gemm.py:30-48, nvfp4_cuda.py:158-187) on top of the sm_100a kernels."""
from __future__ import annotations

import math

import torch

from . import _lib
from .tensor import BLK, NVFP4Tensor, swizzled_scale_dims

F4_MAX, F8E4M3_MAX, E4M3_EPS = 6.0, 448.0, 0.015625

_SEED = [0]          # auto-advancing seed of stochastic calls, like nvfp4_cuda.py:154,160-162
_H_OK = {}           # H tensors already checked to be the Sylvester matrix / 4
_ONES = {}


def hadamard16(device="cuda"):
    """Sylvester Hadamard matrix of order 16, divided by 4 (nvfp4_gemm.py:23-27).  The kernels
    apply exactly this transform as an in-register butterfly; the matrix exists for callers
    that pass it around."""
    h = torch.ones(1, 1, device=device, dtype=torch.float32)
    while h.shape[0] < BLK:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(BLK)


def _check_h(H):
    if H is None:
        return
    key = (H.data_ptr(), H._version, H.device)
    if key not in _H_OK:
        if H.shape != (BLK, BLK) or not torch.equal(H.float().cpu(), hadamard16("cpu")):
            raise ValueError("H must be hadamard16(): the kernels implement the 16-point Sylvester "
                             "Hadamard transform only")
        _H_OK[key] = True


def _signs(signs, device):
    if signs is None:
        if device not in _ONES:
            _ONES[device] = torch.ones(BLK, device=device, dtype=torch.float32)
        return _ONES[device]
    s = signs.to(device=device, dtype=torch.float32).contiguous()
    if s.numel() != BLK:
        raise ValueError("signs must have 16 entries")
    return s


_WS = {}


def _workspace(device):
    """64-byte scratch of the single-launch quantizer, zeroed once, one per (device, stream): every
    launch leaves it ready for the next, and launches on one stream never overlap."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    if key not in _WS:
        _WS[key] = torch.zeros(16, dtype=torch.int32, device=device)
    return _WS[key]


def fused_error(device=None) -> int:
    """Sticky error word of the single-launch quantizer's workspace on the current stream
    (0 = none).  Reading it synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    return int(_WS[key][4].item()) if key in _WS else 0


def _stream(device=None):
    """Handle of torch's current stream on `device` (default: the current device)."""
    return torch.cuda.current_stream(device).cuda_stream


def _as_bf16_rows(t):
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if not t.is_cuda:
        raise _lib.NVFP4Error("the NVFP4 quantizer runs on a CUDA device only (no CPU path)")
    x = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.stride(0) < x.shape[1] or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    return x


def tensor_amax(t, rht=False, signs=None, transpose=False, out=None):
    """Per-tensor |x| maximum of a 2-D tensor as a 1-element fp32 CUDA tensor (after the Hadamard
    transform of its 16-blocks when rht).  No host synchronisation."""
    x = _as_bf16_rows(t)
    amax = out if out is not None else torch.empty(1, device=x.device, dtype=torch.float32)
    sg = _signs(signs, x.device) if rht else None
    dev = _lib.cuda_device_of(x, amax, sg)
    with torch.cuda.device(dev):                   # the C side launches on the current device
        code = _lib.lib().nvfp4_amax_bf16(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), int(rht),
                                          int(transpose), sg.data_ptr() if rht else None,
                                          amax.data_ptr(), 1, _stream(dev))
    _lib.check(code, "nvfp4_amax_bf16")
    return amax


def quant_nvfp4(t, stochastic=False, rht=False, H=None, signs=None, seed=None, *,
                transpose=False, amax=None, philox_offset=0, fused=True, counter=None):
    """t: [M, K] -> NVFP4Tensor blocked along K (K % 16 == 0), as nvfp4_gemm.py:30-48.

    transpose=True quantizes t.t() (blocks along the rows of t) without materialising the
    transpose: the result equals quant_nvfp4(t.t().contiguous(), ...).
    amax: optional 1-element fp32 CUDA tensor to use instead of computing the per-tensor
    maximum here (a tensor sharded across GPUs passes the all-reduced maximum).
    seed=None takes the module counter and advances it on stochastic calls.
    fused=False forces the two-launch path (amax kernel, then quantize kernel) where the
    single-launch cooperative kernel would be used; both give the same bytes.
    counter: (pitch, base) of the stochastic-rounding counter when t is a shard of a larger tensor
    (see nvfp4_quantize_shard_bf16 in the C header); needs amax (the group-reduced one)."""
    if counter is not None and amax is None:
        raise ValueError("a sharded tensor is quantized with the group-reduced amax: pass amax=")
    if seed is None:
        seed = _SEED[0]
        if stochastic:
            _SEED[0] += 1
    _check_h(H)
    x = _as_bf16_rows(t)
    rows, cols = x.shape
    m, k = (cols, rows) if transpose else (rows, cols)
    if k % BLK != 0:
        raise AssertionError(f"K={k} must be divisible by {BLK}")
    dev = x.device
    sg = _signs(signs, dev) if rht else None
    sm, sk = swizzled_scale_dims(m, k)
    qdata = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((sm, sk), dtype=torch.uint8, device=dev)
    pts = torch.empty((), dtype=torch.float32, device=dev)
    _lib.cuda_device_of(x, sg, amax)
    if fused and amax is None and not transpose and rows * (cols // BLK) < 2 ** 31:
        with torch.cuda.device(dev):               # the C side launches on the current device
            ws = _workspace(dev)
            code = _lib.lib().nvfp4_quantize_fused_bf16(
                x.data_ptr(), rows, cols, x.stride(0),
                _lib.ROUND_STOCHASTIC if stochastic else _lib.ROUND_NEAREST, int(rht),
                sg.data_ptr() if rht else None, int(seed) & (2 ** 64 - 1), int(philox_offset),
                qdata.data_ptr(), scale.data_ptr(), pts.data_ptr(), ws.data_ptr(), 64, _stream(dev))
        _lib.check(code, "nvfp4_quantize_fused_bf16")
        return NVFP4Tensor(qdata, scale.view(torch.float8_e4m3fn), BLK, t.dtype, pts, True)
    if amax is None:
        amax = tensor_amax(x, rht, sg, transpose)
    pitch, base = (k // BLK, 0) if counter is None else (int(counter[0]), int(counter[1]))
    with torch.cuda.device(dev):
        code = _lib.lib().nvfp4_quantize_shard_bf16(
            x.data_ptr(), rows, cols, x.stride(0), int(transpose),
            _lib.ROUND_STOCHASTIC if stochastic else _lib.ROUND_NEAREST, int(rht),
            sg.data_ptr() if rht else None, amax.data_ptr(), int(seed) & (2 ** 64 - 1), int(philox_offset),
            pitch, base, qdata.data_ptr(), scale.data_ptr(), pts.data_ptr(), _stream(dev))
    _lib.check(code, "nvfp4_quantize_shard_bf16")
    return NVFP4Tensor(qdata, scale.view(torch.float8_e4m3fn), BLK, t.dtype, pts, True)


def quant_weight_nvfp4(w, amax=None, two_d=False):
    """(quant(w), quant(w.t())) of a weight [N, K] from one read of w, round to nearest: the two
    operands FP4Linear needs (nvfp4_train.py:72-78).  two_d=True scales 16 x 16 tiles (the simulator's
    weight scaling, nvfp4_validate.py:68-82), so that both layouts dequantize to the same matrix.
    amax: optional 1-element fp32 CUDA tensor (a sharded weight passes the group-reduced maximum)."""
    x = _as_bf16_rows(w)
    rows, cols = x.shape
    if rows % BLK != 0 or cols % BLK != 0:
        raise AssertionError(f"weight dims {rows}x{cols} must be divisible by {BLK}")
    dev = x.device
    if amax is None:
        amax = tensor_amax(x)
    _lib.cuda_device_of(x, amax)
    sm_r, sk_r = swizzled_scale_dims(rows, cols)
    sm_c, sk_c = swizzled_scale_dims(cols, rows)
    q_r = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    s_r = torch.empty((sm_r, sk_r), dtype=torch.uint8, device=dev)
    q_c = torch.empty((cols, rows // 2), dtype=torch.uint8, device=dev)
    s_c = torch.empty((sm_c, sk_c), dtype=torch.uint8, device=dev)
    pts = torch.empty((), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        code = _lib.lib().nvfp4_quantize_weight_bf16(x.data_ptr(), rows, cols, x.stride(0), int(two_d), amax.data_ptr(),
                                                     q_r.data_ptr(), s_r.data_ptr(), q_c.data_ptr(), s_c.data_ptr(),
                                                     pts.data_ptr(), _stream(dev))
    _lib.check(code, "nvfp4_quantize_weight_bf16")
    return (NVFP4Tensor(q_r, s_r.view(torch.float8_e4m3fn), BLK, w.dtype, pts, True),
            NVFP4Tensor(q_c, s_c.view(torch.float8_e4m3fn), BLK, w.dtype, pts, True))


def tensor_amax_both(t, signs):
    """fp32 [2] = (max|t|, max|RHT_rows(t)|) from one read of t [rows, cols] (rows % 16 == 0): what
    tensor_amax(t) and tensor_amax(t, True, signs, transpose=True) find in two."""
    x = _as_bf16_rows(t)
    sg = _signs(signs, x.device)
    dev = _lib.cuda_device_of(x, sg)
    maxima = torch.empty(2, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        code = _lib.lib().nvfp4_amax_both_bf16(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), sg.data_ptr(),
                                               maxima.data_ptr(), 1, _stream(dev))
    _lib.check(code, "nvfp4_amax_both_bf16")
    return maxima


def quant_dual_nvfp4(t, signs, amax_rows=None, amax_cols=None, stochastic_rows=False, stochastic_cols=False,
                     seed_rows=None, seed_cols=None, philox_offset=0, counters=None):
    """(quant_nvfp4(t, stochastic_rows), quant_nvfp4(t, stochastic_cols, rht=True, signs=signs,
    transpose=True)) from ONE read of t [rows, cols]: the operand and its Hadamard-transformed
    transpose, which FP4Linear needs of every activation and gradient (nvfp4_train.py:36-55).
    amax_rows / amax_cols: 1-element fp32 CUDA tensors (the plain maximum and the maximum after the
    Hadamard transform along the rows); both are found in one extra read when either is missing.
    Seeds left None come from the module counter in the order rows, cols, as two separate stochastic
    calls would draw them.  counters: (pitch_rows, base_rows, pitch_cols, base_cols) for a shard."""
    if seed_rows is None:
        seed_rows = _SEED[0]
        if stochastic_rows:
            _SEED[0] += 1
    if seed_cols is None:
        seed_cols = _SEED[0]
        if stochastic_cols:
            _SEED[0] += 1
    x = _as_bf16_rows(t)
    rows, cols = x.shape
    if rows % BLK != 0 or cols % BLK != 0:
        raise AssertionError(f"dims {rows}x{cols} must be divisible by {BLK}")
    dev = x.device
    sg = _signs(signs, dev)
    if amax_rows is None and amax_cols is None:
        both = tensor_amax_both(x, sg)
        amax_rows, amax_cols = both[0:1], both[1:2]
    elif amax_cols is None:
        amax_cols = tensor_amax(x, True, sg, transpose=True)
    elif amax_rows is None:
        amax_rows = tensor_amax(x)
    _lib.cuda_device_of(x, sg, amax_rows, amax_cols)
    sm_r, sk_r = swizzled_scale_dims(rows, cols)
    sm_c, sk_c = swizzled_scale_dims(cols, rows)
    q_r = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    s_r = torch.empty((sm_r, sk_r), dtype=torch.uint8, device=dev)
    q_c = torch.empty((cols, rows // 2), dtype=torch.uint8, device=dev)
    s_c = torch.empty((sm_c, sk_c), dtype=torch.uint8, device=dev)
    pts_r = torch.empty((), dtype=torch.float32, device=dev)
    pts_c = torch.empty((), dtype=torch.float32, device=dev)
    ctr = None
    if counters is not None:
        import ctypes
        ctr = (ctypes.c_uint64 * 4)(*[int(v) for v in counters])
    mode = lambda sr: _lib.ROUND_STOCHASTIC if sr else _lib.ROUND_NEAREST
    with torch.cuda.device(dev):
        code = _lib.lib().nvfp4_quantize_dual_bf16(
            x.data_ptr(), rows, cols, x.stride(0), mode(stochastic_rows), mode(stochastic_cols), sg.data_ptr(),
            amax_rows.data_ptr(), amax_cols.data_ptr(), int(seed_rows) & (2 ** 64 - 1), int(seed_cols) & (2 ** 64 - 1),
            int(philox_offset), ctr, q_r.data_ptr(), s_r.data_ptr(), pts_r.data_ptr(), q_c.data_ptr(), s_c.data_ptr(),
            pts_c.data_ptr(), _stream(dev))
    _lib.check(code, "nvfp4_quantize_dual_bf16")
    return (NVFP4Tensor(q_r, s_r.view(torch.float8_e4m3fn), BLK, t.dtype, pts_r, True),
            NVFP4Tensor(q_c, s_c.view(torch.float8_e4m3fn), BLK, t.dtype, pts_c, True))


# the reference's second name for the same entry (nvfp4_cuda.py:158)
quant_nvfp4_cuda = quant_nvfp4
