"""RMSNorm fused with the search for the maxima the next NVFP4 quantizations need.

`rmsnorm_amax(x, weight, eps, signs)` returns (h, maxima): h = rms_norm(x) * weight as bf16, and
maxima = fp32 [2] = max|h| and max|RHT_tokens(h)|, which `FP4Linear.forward(h, amax=maxima,
amax_signs=signs)` takes in place of its own two passes over h.  The reference runs nn.RMSNorm
(nvfp4_train.py:105,114-122) and lets every FP4Linear that reads the result find its maximum again
(quant_nvfp4, nvfp4_gemm.py:34-36)."""
from __future__ import annotations

import torch

from . import _lib
from .quant import _signs, _stream


class RMSNormAmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, signs):
        if x.dtype not in (torch.float32, torch.bfloat16) or weight.dtype != torch.float32:
            raise ValueError("fused RMSNorm takes fp32 or bf16 activations and an fp32 weight")
        cols = x.shape[-1]
        if cols % 8 != 0 or weight.numel() != cols:
            raise ValueError("fused RMSNorm needs a last dimension that is a multiple of 8 and a weight of that size")
        dev = _lib.cuda_device_of(x, weight)
        x2 = x.reshape(-1, cols).contiguous()
        w = weight.contiguous()
        rows = x2.shape[0]
        use_rht = signs is not None and rows % 16 == 0
        sg = _signs(signs, dev) if use_rht else None
        h = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev)
        maxima = torch.empty(2, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):                  # the C side launches on the current device
            code = _lib.lib().nvfp4_rmsnorm_fwd(x2.data_ptr(), int(x2.dtype == torch.float32), w.data_ptr(), rows, cols,
                                                float(eps), h.data_ptr(), rstd.data_ptr(),
                                                sg.data_ptr() if use_rht else None, maxima.data_ptr(), 1, _stream(dev))
        _lib.check(code, "nvfp4_rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.xshape = x.shape
        ctx.mark_non_differentiable(maxima)
        return h.reshape(*x.shape[:-1], cols), maxima

    @staticmethod
    def backward(ctx, g, _gmax):
        x2, w, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        g2 = g.reshape(rows, cols)
        if g2.dtype not in (torch.float32, torch.bfloat16):
            g2 = g2.float()
        g2 = g2.contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty(cols, dtype=torch.float32, device=x2.device)
        with torch.cuda.device(x2.device):
            code = _lib.lib().nvfp4_rmsnorm_bwd(x2.data_ptr(), int(x2.dtype == torch.float32), w.data_ptr(),
                                                rstd.data_ptr(), g2.data_ptr(), int(g2.dtype == torch.float32), rows, cols,
                                                dx.data_ptr(), dw.data_ptr(), 1, _stream(x2.device))
        _lib.check(code, "nvfp4_rmsnorm_bwd")
        return dx.reshape(ctx.xshape), dw, None, None


def rmsnorm_amax(x, weight, eps=None, signs=None):
    """eps None = torch's default for nn.RMSNorm: the machine epsilon of x's dtype."""
    if eps is None:
        eps = torch.finfo(x.dtype).eps
    return RMSNormAmaxFn.apply(x, weight, eps, signs)
