"""Fused SwiGLU in front of the quantizer: h = silu(g) * u (and its backward) in one pass each that also
leaves the per-tensor maxima the next NVFP4 quantizations need (plain, and after the 16-point Hadamard
along the token dimension), so FP4Linear can skip its amax passes: the down projection gets the maxima
of h explicitly, the gate / up projections find the maxima of their output gradients through
`linear.hint_grad_amax`.  The reference does this with torch element-wise kernels and separate amax
reductions inside its quantizer (nvfp4_cuda.py:158-165)."""
from __future__ import annotations

import torch

from . import _lib
from . import linear as _linear
from .quant import _signs, _stream


def _rows(t):
    return t.reshape(-1, t.shape[-1])


class SwiGLUFn(torch.autograd.Function):
    """(g, u) -> (h, maxima) with maxima = fp32 [2]: max|h| and max|RHT_tokens(h)| (the second only
    when `signs` is given and the token count is a multiple of 16, else 0)."""

    @staticmethod
    def forward(ctx, g, u, signs):
        if g.dtype != torch.bfloat16 or u.dtype != torch.bfloat16 or g.shape != u.shape:
            raise ValueError("fused SwiGLU takes two bf16 tensors of one shape")
        g2, u2 = _rows(g).contiguous(), _rows(u).contiguous()
        rows, cols = g2.shape
        use_rht = signs is not None and rows % 16 == 0
        sg = _signs(signs, g.device) if use_rht else None
        h = torch.empty_like(g2)
        maxima = torch.empty(2, dtype=torch.float32, device=g.device)
        with torch.cuda.device(g2.device):           # the C side launches on the current device
            code = _lib.lib().nvfp4_swiglu_fwd_bf16(g2.data_ptr(), u2.data_ptr(), rows, cols, g2.stride(0), h.data_ptr(),
                                                    h.stride(0), sg.data_ptr() if use_rht else None, maxima.data_ptr(),
                                                    1, _stream(g2.device))
        _lib.check(code, "nvfp4_swiglu_fwd_bf16")
        ctx.save_for_backward(g2, u2)
        ctx.sg, ctx.use_rht, ctx.shape, ctx.signs_in = sg, use_rht, g.shape, signs
        ctx.mark_non_differentiable(maxima)
        return h.reshape(g.shape), maxima

    @staticmethod
    def backward(ctx, dh, _dmax):
        g2, u2 = ctx.saved_tensors
        d2 = _rows(dh)
        if d2.dtype != torch.bfloat16:
            d2 = d2.to(torch.bfloat16)
        d2 = d2.contiguous()
        rows, cols = g2.shape
        dg, du = torch.empty_like(g2), torch.empty_like(g2)
        maxima = torch.empty(4, dtype=torch.float32, device=g2.device)
        with torch.cuda.device(g2.device):           # the C side launches on the current device
            code = _lib.lib().nvfp4_swiglu_bwd_bf16(g2.data_ptr(), u2.data_ptr(), d2.data_ptr(), rows, cols, g2.stride(0),
                                                    dg.data_ptr(), du.data_ptr(), dg.stride(0),
                                                    ctx.sg.data_ptr() if ctx.use_rht else None, maxima.data_ptr(), 1,
                                                    _stream(g2.device))
        _lib.check(code, "nvfp4_swiglu_bwd_bf16")
        dg, du = dg.reshape(ctx.shape), du.reshape(ctx.shape)
        # the linears that produced g and u will quantize exactly these tensors in their backward
        _linear.hint_grad_amax(dg, maxima[0:2], ctx.use_rht, ctx.signs_in)
        _linear.hint_grad_amax(du, maxima[2:4], ctx.use_rht, ctx.signs_in)
        return dg, du, None


class SwiGLUPackedFn(torch.autograd.Function):
    """gu [*, 2H] = gate | up side by side (the output of one fused projection) -> (h [*, H], maxima):
    SwiGLUFn without the split: the kernels read the two halves in place (row stride 2H), and the
    backward writes dgate | dup into ONE [*, 2H] tensor, the gradient of the fused projection, and
    hints its maxima (the larger of the two halves') to that projection."""

    @staticmethod
    def forward(ctx, gu, signs):
        if gu.dtype != torch.bfloat16 or gu.shape[-1] % 16 != 0:
            raise ValueError("fused SwiGLU takes a bf16 tensor whose last dimension is 2H, H a multiple of 8")
        gu2 = _rows(gu).contiguous()
        rows, two_h = gu2.shape
        hid = two_h // 2
        use_rht = signs is not None and rows % 16 == 0
        sg = _signs(signs, gu.device) if use_rht else None
        h = torch.empty((rows, hid), dtype=torch.bfloat16, device=gu.device)
        maxima = torch.empty(2, dtype=torch.float32, device=gu.device)
        g_ptr, u_ptr = gu2.data_ptr(), gu2.data_ptr() + 2 * hid
        with torch.cuda.device(gu2.device):           # the C side launches on the current device
            code = _lib.lib().nvfp4_swiglu_fwd_bf16(g_ptr, u_ptr, rows, hid, two_h, h.data_ptr(), hid,
                                                    sg.data_ptr() if use_rht else None, maxima.data_ptr(), 1,
                                                    _stream(gu2.device))
        _lib.check(code, "nvfp4_swiglu_fwd_bf16")
        ctx.save_for_backward(gu2)
        ctx.sg, ctx.use_rht, ctx.shape, ctx.signs_in = sg, use_rht, gu.shape, signs
        ctx.mark_non_differentiable(maxima)
        return h.reshape(*gu.shape[:-1], hid), maxima

    @staticmethod
    def backward(ctx, dh, _dmax):
        (gu2,) = ctx.saved_tensors
        rows, two_h = gu2.shape
        hid = two_h // 2
        d2 = _rows(dh)
        if d2.dtype != torch.bfloat16:
            d2 = d2.to(torch.bfloat16)
        d2 = d2.contiguous()
        dgu = torch.empty_like(gu2)
        maxima = torch.empty(4, dtype=torch.float32, device=gu2.device)
        with torch.cuda.device(gu2.device):
            code = _lib.lib().nvfp4_swiglu_bwd_strided_bf16(
                gu2.data_ptr(), gu2.data_ptr() + 2 * hid, d2.data_ptr(), rows, hid, two_h, hid,
                dgu.data_ptr(), dgu.data_ptr() + 2 * hid, two_h, ctx.sg.data_ptr() if ctx.use_rht else None,
                maxima.data_ptr(), 1, _stream(gu2.device))
        _lib.check(code, "nvfp4_swiglu_bwd_strided_bf16")
        both = torch.maximum(maxima[0:2], maxima[2:4])            # maxima of dgate | dup as one tensor
        dgu = dgu.reshape(ctx.shape)
        _linear.hint_grad_amax(dgu, both, ctx.use_rht, ctx.signs_in)
        return dgu, None


def swiglu_packed(gu, signs=None):
    """h = silu(gu[..., :H]) * gu[..., H:] and the maxima of h (see SwiGLUPackedFn)."""
    return SwiGLUPackedFn.apply(gu, signs)


def swiglu(g, u, signs=None):
    """h = silu(g) * u and the maxima of h (see SwiGLUFn)."""
    return SwiGLUFn.apply(g, u, signs)


class ReLU2Fn(torch.autograd.Function):
    """x -> (relu(x)^2, maxima): the MLP activation of the reference's models (nvfp4_train.py:120-123)
    fused with the maxima of its result, like SwiGLUFn; the backward hints the maxima of dx to the
    linear that produced x."""

    @staticmethod
    def forward(ctx, x, signs):
        if x.dtype != torch.bfloat16 or x.shape[-1] % 8 != 0:
            raise ValueError("fused squared ReLU takes a bf16 tensor whose last dimension is a multiple of 8")
        x2 = _rows(x).contiguous()
        rows, cols = x2.shape
        use_rht = signs is not None and rows % 16 == 0
        sg = _signs(signs, x.device) if use_rht else None
        out = torch.empty_like(x2)
        maxima = torch.empty(2, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x2.device):           # the C side launches on the current device
            code = _lib.lib().nvfp4_relu2_fwd_bf16(x2.data_ptr(), rows, cols, x2.stride(0), out.data_ptr(), out.stride(0),
                                                   sg.data_ptr() if use_rht else None, maxima.data_ptr(), 1, _stream(x2.device))
        _lib.check(code, "nvfp4_relu2_fwd_bf16")
        ctx.save_for_backward(x2)
        ctx.sg, ctx.use_rht, ctx.shape, ctx.signs_in = sg, use_rht, x.shape, signs
        ctx.mark_non_differentiable(maxima)
        return out.reshape(x.shape), maxima

    @staticmethod
    def backward(ctx, dout, _dmax):
        (x2,) = ctx.saved_tensors
        d2 = _rows(dout)
        if d2.dtype != torch.bfloat16:
            d2 = d2.to(torch.bfloat16)
        d2 = d2.contiguous()
        rows, cols = x2.shape
        dx = torch.empty_like(x2)
        maxima = torch.empty(2, dtype=torch.float32, device=x2.device)
        with torch.cuda.device(x2.device):           # the C side launches on the current device
            code = _lib.lib().nvfp4_relu2_bwd_bf16(x2.data_ptr(), d2.data_ptr(), rows, cols, x2.stride(0), dx.data_ptr(),
                                                   dx.stride(0), ctx.sg.data_ptr() if ctx.use_rht else None,
                                                   maxima.data_ptr(), 1, _stream(x2.device))
        _lib.check(code, "nvfp4_relu2_bwd_bf16")
        dx = dx.reshape(ctx.shape)
        _linear.hint_grad_amax(dx, maxima, ctx.use_rht, ctx.signs_in)
        return dx, None


def relu2(x, signs=None):
    """relu(x)^2 and the maxima of the result (see ReLU2Fn)."""
    return ReLU2Fn.apply(x, signs)
