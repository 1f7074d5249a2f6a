"""FP4Linear: a linear layer whose three GEMMs run in NVFP4 (nvfp4_train.py:19-88).

  fprop  Y  = X  W^T     X: round-to-nearest, W: round-to-nearest            (contraction K)
  dgrad  dX = dY W       dY: stochastic rounding, W^T: round-to-nearest      (contraction N)
  wgrad  dW = dY^T X     both through the 16-point random-sign Hadamard along the token
                         dimension; dY^T: stochastic rounding, X^T: nearest  (contraction M)

Every transposed operand (W^T, dY^T, X^T) is produced by the transposing quantizer straight from
the row-major tensor, so no transposed copy is ever written (the reference materialises three:
nvfp4_gemm.py:55, nvfp4_train.py:53,77).

NVFP4_AMORTIZE=1 (read at import, like nvfp4_train.py:20-21) caches the two weight quantizations
per optimizer step; mark_step() must be called after every optimizer step or the cache goes stale
(tests/parity_check.py in the reference shows exactly that behaviour)."""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .gemm import nvfp4_mm
from .quant import hadamard16, quant_dual_nvfp4, quant_nvfp4, quant_weight_nvfp4, tensor_amax, tensor_amax_both
from .tensor import BLK, NVFP4Tensor

_STEP = [0]          # bumped once per optimizer step; the weight-quant cache keys on it
# The reference also wants NVFP4_CUDA=1 before it amortizes, because only its CUDA backend can;
# here there is one backend, so NVFP4_AMORTIZE alone decides and NVFP4_CUDA is accepted and ignored.
_AMORTIZE = os.environ.get("NVFP4_AMORTIZE", "0") == "1"


def mark_step():
    """Invalidate every FP4Linear's cached weight quantization (call after optimizer.step())."""
    _STEP[0] += 1
    _GRAD_AMAX.clear()


# Maxima of gradient tensors that a fused producer already knows (swiglu.SwiGLUFn.backward): keyed by
# the address of the gradient, which the entry keeps alive so that the address cannot be reused while
# the hint exists.  FP4LinearFn.backward takes the hint of the gradient it is handed and then skips
# its amax passes.  Entries that are never taken are dropped by mark_step(), and the table never
# holds more than _GRAD_AMAX_MAX of them (oldest dropped first), so a caller that never calls
# mark_step() does not keep gradients alive without bound.
_GRAD_AMAX = {}
_GRAD_AMAX_MAX = 64


_SIGNS_EQ = {}


def _signs_key(signs):
    """Identity of a sign vector as the kernels saw it: its storage address and version counter."""
    return None if signs is None else (signs.data_ptr(), signs._version)


def _same_signs(a, b):
    """Do two sign vectors hold the same 16 values?  Compared once per pair of (address, version) --
    the comparison reads the device -- and remembered, so the hot path never synchronises."""
    if a is None or b is None:
        return a is b
    ka, kb = _signs_key(a), _signs_key(b)
    if ka == kb:
        return True
    key = (ka, kb)
    if key not in _SIGNS_EQ:
        if len(_SIGNS_EQ) > 256:
            _SIGNS_EQ.clear()
        _SIGNS_EQ[key] = bool(a.device == b.device and a.shape == b.shape and torch.equal(a, b))
    return _SIGNS_EQ[key]


def hint_grad_amax(grad, maxima2, has_rht, signs=None):
    """maxima2: fp32 [2] on the device = max|grad| and max|RHT_tokens(grad)|.  The second is valid if
    has_rht and was computed with the sign vector `signs`; a consumer with another sign vector
    recomputes it."""
    while len(_GRAD_AMAX) >= _GRAD_AMAX_MAX:
        _GRAD_AMAX.pop(next(iter(_GRAD_AMAX)))
    _GRAD_AMAX[grad.data_ptr()] = (grad, maxima2, bool(has_rht), signs, None if signs is None else signs._version)


def _take_grad_amax(gy2, signs=None):
    e = _GRAD_AMAX.pop(gy2.data_ptr(), None)
    if e is None or e[0].numel() != gy2.numel() or e[0].dtype != gy2.dtype or e[0].shape[-1] != gy2.shape[-1]:
        return None, None
    rht_ok = e[2] and (e[3] is None or (e[3]._version == e[4] and _same_signs(e[3], signs)))
    return e[1][0:1], (e[1][1:2] if rht_ok else None)


_DUAL = [True]
# The one-read kernel wins where launches and re-reads dominate (measured on a B200: 43 us against 64 us
# for the two layouts of a 4096 x 4096 tensor) and loses to the two streaming kernels on large tensors
# (150 us against 127 us at 4096 x 28672), so it takes tensors up to this many elements.
_DUAL_MAX_ELEMS = 1 << 24


def set_dual_quant(flag: bool):
    """Quantize every activation and gradient in both layouts from one read (the default), or with one
    kernel per layout (False: the two-step path, kept for comparison and for tensors whose token count
    is not a multiple of 16)."""
    _DUAL[0] = bool(flag)


def set_amortize(flag: bool):
    """Switch the per-step weight-quant cache on or off after import (tests, benchmarks)."""
    global _AMORTIZE
    _AMORTIZE = bool(flag)


def _grad_dtype(w):
    return torch.float32 if w.dtype == torch.float32 else torch.bfloat16


class FP4LinearFn(torch.autograd.Function):
    """x: [*, K], w: [N, K] -> [*, N].  wq_K = quant(w) and wq_N = quant(w.t()) may be passed in
    pre-computed (the amortized path); amax_reduce, if given, is called on every per-tensor amax
    word of a tensor that is sharded across ranks before it is used (tensor parallelism)."""

    @staticmethod
    def forward(ctx, x, w, H, signs, wq_K, wq_N, amax_reduce=None, sharded=(False, False), x_amax=None,
                x_amax_rht=True, dx_reduce=None, y_amax_out=None, x_quant=None):
        # dx_reduce: optional callable(dx) -> handle with .wait(): starts the sum of the input gradient
        # over a tensor-parallel group right after the dgrad GEMM, so that it runs beside the wgrad
        # quantizations and GEMM; the handle is waited for before the backward returns
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        x_sharded, y_sharded = sharded[0], sharded[1]  # is the K dim / the N dim split across ranks?
        # x_amax: fp32 [2] from a fused producer = max|x| and max|RHT_tokens(x)| (what the two amax
        # passes over x would find); the token count must then be a multiple of 16
        if x_amax is not None and (x2.shape[0] % BLK != 0 or x2.dtype != torch.bfloat16):
            x_amax = None
        if x_amax is not None and x_amax.numel() == 1:           # the plain maximum only
            x_amax_rht = False
        x_red = amax_reduce if x_sharded else None
        if x_amax is not None and x_red is not None:
            # both maxima of a sharded x in ONE collective; the backward reuses the second
            x_amax = x_amax.clone()
            x_red(x_amax)
            x_red = None
        ctx.x_reduced = x_amax is not None and x_sharded and amax_reduce is not None
        # Both layouts of x from ONE read when the weight gradient will want x^T: the row-wise operand
        # for the GEMM below and the Hadamard-transformed transpose for wgrad, which then needs neither
        # x nor another pass in backward.  (A sharded x without producer maxima keeps the two-step path:
        # its maxima are reduced over the group one by one.)
        have_both = x_amax is not None and x_amax_rht and x_amax.numel() >= 2
        # (inside torch.no_grad() needs_input_grad still reflects requires_grad: ask the grad mode too)
        dual = (_DUAL[0] and ctx.needs_input_grad[1] and torch.is_grad_enabled() and x2.is_cuda and x2.shape[0] % BLK == 0
                and x2.numel() <= _DUAL_MAX_ELEMS and (x_red is None) and (have_both or not x_sharded))
        xtq = None
        if x_quant is not None:
            # x_quant = quant_input(x, ...) made once by a caller that feeds x to several layers holding
            # the same sign vector (q, k, v of a block): (row-wise operand, transformed transpose or None;
            # without the transpose the backward quantizes x^T itself, as on the plain path)
            xq, xtq = x_quant
        elif dual:
            xq, xtq = quant_dual_nvfp4(x2, signs, None if x_amax is None else x_amax[0:1],
                                       x_amax[1:2] if have_both else None)
        else:
            xq = _quant(x2, x_red, amax=None if x_amax is None else x_amax[0:1])
        if wq_K is None:
            wq_K = _quant(w, amax_reduce)
        # y_amax_out: optional fp32 [1] that the fprop GEMM's epilogue fills with max|y| (for a consumer
        # that quantizes y next; only meaningful when y stays bf16, i.e. x is bf16)
        y = nvfp4_mm(xq, wq_K.t(), torch.bfloat16, amax_out=y_amax_out)
        if xtq is None:
            ctx.save_for_backward(x2, w)
        else:
            ctx.save_for_backward(w, xtq.qdata, xtq.scale, xtq.per_tensor_scale)
        ctx.have_xtq = xtq is not None
        ctx.H, ctx.signs, ctx.xshape, ctx.wq_N = H, signs, x.shape, wq_N
        ctx.amax_reduce, ctx.sharded, ctx.x_amax = amax_reduce, sharded, x_amax
        ctx.x_amax_rht = bool(x_amax_rht)        # False: the Hadamard maximum came from another sign vector
        ctx.dx_reduce = dx_reduce
        return y.reshape(*x.shape[:-1], w.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        if ctx.have_xtq:
            w, xt_q, xt_s, xt_p = ctx.saved_tensors
            x2 = None
            xtq = NVFP4Tensor(xt_q, xt_s, BLK, torch.bfloat16, xt_p, True)
        else:
            x2, w = ctx.saved_tensors
            xtq = None
        H, signs, wq_N, red = ctx.H, ctx.signs, ctx.wq_N, ctx.amax_reduce
        x_sharded, y_sharded = ctx.sharded[0], ctx.sharded[1]
        gy2 = gy.reshape(-1, w.shape[0])
        # a gradient split along N draws the stochastic-rounding bits of its place in the whole tensor:
        # sharded = (x_sharded, y_sharded, (rank, world)) gives the place (see nvfp4_quantize_shard_bf16)
        ctr_rows = ctr_cols = None
        if y_sharded and len(ctx.sharded) > 2 and ctx.sharded[2] is not None:
            rank, world = ctx.sharded[2]
            n_local, tokens = w.shape[0], gy2.shape[0]
            ctr_rows = (n_local * world // BLK, rank * n_local // BLK)
            ctr_cols = (tokens // BLK, rank * n_local * (tokens // BLK))
        g_amax, g_amax_rht = _take_grad_amax(gy2, signs)      # known to a fused producer of gy, else None
        g_red = red if y_sharded else None
        # dY in both layouts from one read when both gradients are wanted (a sharded dY needs its
        # counters, which come with the rank)
        dual_g = (_DUAL[0] and ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and gy2.is_cuda
                  and gy2.shape[0] % BLK == 0 and gy2.numel() <= _DUAL_MAX_ELEMS
                  and (g_red is None or ctr_rows is not None))
        if dual_g and (g_amax is None or g_amax_rht is None):
            both = tensor_amax_both(gy2, signs)               # one read for the two maxima
            if g_red is not None:
                g_red(both)
            g_amax, g_amax_rht = both[0:1], both[1:2]
        elif g_amax is not None and g_red is not None:
            # a sharded gradient: reduce the producer's maxima over the group, both in ONE collective
            both = torch.cat([g_amax, g_amax_rht]) if g_amax_rht is not None else g_amax.clone()
            g_red(both)
            g_amax, g_amax_rht = both[0:1], (both[1:2] if g_amax_rht is not None else None)
        x_amax_rht = None if (ctx.x_amax is None or not ctx.x_amax_rht) else ctx.x_amax[1:2]
        # the Hadamard maximum of a sharded x was reduced in forward together with the plain one;
        # when it has to be recomputed here (none given, or another sign vector) it is reduced here
        xt_red = None if (x_amax_rht is not None and ctx.x_reduced) else (red if x_sharded else None)
        dx = dw = None
        gq = gtq = None
        if dual_g:
            counters = None if ctr_rows is None else (ctr_rows[0], ctr_rows[1], ctr_cols[0], ctr_cols[1])
            gq, gtq = quant_dual_nvfp4(gy2, signs, g_amax, g_amax_rht, True, True, counters=counters)
        if ctx.needs_input_grad[0]:
            # dgrad: dX = dY @ W, contraction over N; dY gets stochastic rounding
            if gq is None:
                gq = _quant(gy2, None if g_amax is not None else g_red, stochastic=True, amax=g_amax, counter=ctr_rows)
            if wq_N is None:
                wq_N = _quant(w, red, transpose=True)
            dx = nvfp4_mm(gq, wq_N.t(), torch.bfloat16).reshape(ctx.xshape).to(gy.dtype)
        pending = ctx.dx_reduce(dx) if (dx is not None and ctx.dx_reduce is not None) else None
        if ctx.needs_input_grad[1]:
            # wgrad: dW = dY^T @ X, contraction over tokens; Hadamard on both, SR on the gradient
            if gtq is None:
                gtq = _quant(gy2, None if g_amax_rht is not None else g_red, stochastic=True, rht=True, H=H, signs=signs,
                             transpose=True, amax=g_amax_rht, counter=ctr_cols)
            if xtq is None:
                xtq = _quant(x2, xt_red, rht=True, H=H, signs=signs, transpose=True, amax=x_amax_rht)
            dw = nvfp4_mm(gtq, xtq.t(), _grad_dtype(w)).to(w.dtype)
        if pending is not None:
            pending.wait()
        return dx, dw, None, None, None, None, None, None, None, None, None, None, None


def _quant(t, amax_reduce, stochastic=False, rht=False, H=None, signs=None, transpose=False, amax=None, counter=None):
    """amax: the per-tensor maximum if a producer already knows it (this rank's part when sharded);
    counter: (pitch, base) of the stochastic-rounding counter of a shard."""
    if amax_reduce is None:
        if counter is not None and amax is None:
            amax = tensor_amax(t, rht, signs, transpose)
        return quant_nvfp4(t, stochastic, rht, H, signs, transpose=transpose, amax=amax, counter=counter)
    amax = tensor_amax(t, rht, signs, transpose) if amax is None else amax.clone()
    amax_reduce(amax)
    return quant_nvfp4(t, stochastic, rht, H, signs, transpose=transpose, amax=amax, counter=counter)


class WeightQuantCache:
    """quant(w) and quant(w.t()) of one weight, recomputed when the global step moves
    (nvfp4_train.py:72-78): one amax pass, then both layouts from one read of the weight.
    two_d: 16 x 16 scaling tiles instead of 1 x 16 blocks (both layouts then hold the same values)."""

    def __init__(self, two_d=False):
        self.step, self.wq_K, self.wq_N, self.two_d = -1, None, None, bool(two_d)

    def get(self, weight, amax_reduce=None):
        if not _AMORTIZE:
            return None, None
        if self.step != _STEP[0]:
            w = weight.detach()
            if w.dtype != torch.bfloat16:
                w = w.to(torch.bfloat16)          # one cast of the fp32 master weight serves all three kernels
            amax = tensor_amax(w)
            if amax_reduce is not None:
                amax_reduce(amax)
            # [N, K] with contraction K (fprop) and [K, N] with contraction N (dgrad)
            self.wq_K, self.wq_N = quant_weight_nvfp4(w, amax=amax, two_d=self.two_d)
            self.step = _STEP[0]
        return self.wq_K, self.wq_N


class FP4Linear(nn.Module):
    """Drop-in for nn.Linear(cin, cout, bias=False) with fp32 master weights (nvfp4_train.py:58-80)."""

    def __init__(self, cin, cout, device="cuda", weight_scaling="1d"):
        """weight_scaling: "1d" (1 x 16 blocks, the reference's real-FP4 path) or "2d" (16 x 16 tiles, its
        simulator's weight scaling; takes effect on the cached path, NVFP4_AMORTIZE=1)."""
        super().__init__()
        assert cin % BLK == 0 and cout % BLK == 0
        assert weight_scaling in ("1d", "2d")
        self.weight = nn.Parameter(torch.empty(cout, cin, device=device))
        nn.init.normal_(self.weight, std=0.02)
        self.register_buffer("H", hadamard16(device))
        g = torch.Generator().manual_seed(1)
        self.register_buffer("signs", (torch.randint(0, 2, (BLK,), generator=g).float() * 2 - 1).to(device))
        self._cache = WeightQuantCache(two_d=weight_scaling == "2d")

    # the reference's field names (nvfp4_train.py:67-68)
    @property
    def _cache_step(self):
        return self._cache.step

    @property
    def _wq_K(self):
        return self._cache.wq_K

    @property
    def _wq_N(self):
        return self._cache.wq_N

    def quant_input(self, x, amax=None, amax_signs=None):
        """Quantize x once for several FP4Linear layers that share this layer's sign vector (the q, k, v
        projections of one normalized activation): returns what their `forward(x, x_quant=...)` takes.
        With gradients on, that is the row-wise operand and the Hadamard-transformed transpose from one
        read; without, the row-wise operand alone."""
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        x2 = x.reshape(-1, x.shape[-1])
        both = (amax is not None and amax.numel() >= 2 and x2.shape[0] % BLK == 0 and x2.dtype == torch.bfloat16
                and (amax_signs is None or _same_signs(amax_signs, self.signs)))
        plain = amax[0:1] if (amax is not None and x2.dtype == torch.bfloat16) else None
        if torch.is_grad_enabled() and self.weight.requires_grad and x2.shape[0] % BLK == 0:
            return quant_dual_nvfp4(x2, self.signs, plain, amax[1:2] if both else None)
        return (quant_nvfp4(x2, amax=plain), None)

    def forward(self, x, amax=None, amax_signs=None, amax_out=None, x_quant=None):
        """amax: optional fp32 [2] from a fused producer of x (see FP4LinearFn.forward), or fp32 [1] = the
        plain maximum alone; amax_signs: the sign vector its Hadamard maximum was computed with (None =
        this layer's own).  When it is not this layer's vector, only the plain maximum is used and the
        other is recomputed.  amax_out: optional fp32 [1] CUDA tensor the forward GEMM fills with max|y|
        (bf16 activations), to be handed to the next layer as its `amax`.  x_quant: x already quantized by
        `quant_input` of a layer with the same sign vector (amax is then not needed)."""
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))       # what autocast does for nn.Linear
        wq_K, wq_N = self._cache.get(self.weight)
        rht_ok = amax_signs is None or _same_signs(amax_signs, self.signs)
        return FP4LinearFn.apply(x, self.weight, self.H, self.signs, wq_K, wq_N, None, (False, False), amax, rht_ok,
                                 None, amax_out, x_quant)

    def extra_repr(self):
        return f"in_features={self.weight.shape[1]}, out_features={self.weight.shape[0]}, bias=False, nvfp4"


def make_linear(cin, cout, use_fp4, device="cuda"):
    """nvfp4_train.py:83-88."""
    if use_fp4:
        return FP4Linear(cin, cout, device)
    lin = nn.Linear(cin, cout, bias=False, device=device)
    nn.init.normal_(lin.weight, std=0.02)
    return lin
