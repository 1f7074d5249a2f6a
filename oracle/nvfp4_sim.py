"""The reference's NVFP4 training RECIPE as a fake-quant simulator.  TEST INFRASTRUCTURE ONLY.

Restates, with plain torch ops that run on the CPU or on a CUDA device alike, the simulator the
reference validated its recipe with before it had real FP4 GEMMs (paths inside the reference
project):

  quantize_1d / quantize_2d   nvfp4_validate.py:51-65, :68-82   quantize -> dequantize in one step;
                              two-level scaling (fp32 per tensor, E4M3 per block); blocks of 1x16
                              along the last dim, or 16x16 for weights so that W and W^T quantize
                              to the same values
  rht_lastdim                 nvfp4_validate.py:92-99           random-sign Hadamard in tiles of 16
  SimLinearFn                 nvfp4_validate.py:104-140         fprop: x 1-D RNE, w 2-D RNE;
                              dgrad: gy 1-D with stochastic rounding, the same 2-D w;
                              wgrad: both operands transposed, token dim padded to a multiple of 16,
                              Hadamard on both, x^T RNE, gy^T stochastic
  SimLinear / sim_make_linear nvfp4_validate.py:143-164

It differs from the real-FP4 path (oracle/nvfp4_oracle.py, the kernels) in three documented ways:
no 2^-6 clamp of the block scale, round-to-nearest ties go to the LOWER level, and weights use
16x16 blocks.  The product never imports this module; tests use it as the "reference recipe" whose
loss curve the real-FP4 run has to track, and `tests/golden/make_golden.py` pins it to the
reference's own functions."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

BLK = 16
F4_MAX = 6.0
E4M3_MAX = 448.0
_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def snap_e2m1(v: torch.Tensor, stochastic: bool, u: torch.Tensor | None = None) -> torch.Tensor:
    """Values -> the E2M1 grid (nvfp4_validate.py:35-48).  Stochastic: up with probability
    (|v| - lo) / (hi - lo), decided by `u < p` (u drawn with torch.rand_like when not given).
    Otherwise nearest, a tie going to the lower level."""
    grid = torch.tensor(_GRID, device=v.device, dtype=v.dtype)
    mag = v.abs().clamp(max=F4_MAX)
    k = torch.bucketize(mag, grid, right=True).clamp(1, 7)
    above, below = grid[k], grid[k - 1]
    step = (above - below).clamp_min(1e-9)
    if stochastic:
        p = (mag - below) / step
        draw = torch.rand_like(mag) if u is None else u
        snapped = torch.where(draw < p, above, below)
    else:
        snapped = torch.where((mag - below) <= (above - mag), below, above)
    return torch.sign(v) * snapped


def _fake_quant(blocks: torch.Tensor, reduce_dims, amax_all: torch.Tensor, stochastic: bool, u=None) -> torch.Tensor:
    """Shared body of the 1-D and 2-D forms: `blocks` is the tensor viewed so that `reduce_dims` span
    one scaling block.  Encode scale 2688 / amax_all, block scale (amax_b / 6) * encode scale cast to
    E4M3 (no lower clamp), effective step = that E4M3 value / encode scale (floored at 1e-12)."""
    enc = (F4_MAX * E4M3_MAX) / amax_all
    dec = 1.0 / enc
    amax_b = blocks.abs().amax(dim=reduce_dims, keepdim=True).clamp_min(1e-12)
    sf = ((amax_b / F4_MAX) * enc).to(torch.float8_e4m3fn).float()
    step = (sf * dec).clamp_min(1e-12)
    return snap_e2m1(blocks / step, stochastic, u) * step


def quantize_1d(x: torch.Tensor, stochastic: bool = False, u: torch.Tensor | None = None) -> torch.Tensor:
    """Fake-quant with 1x16 blocks along the last dim (nvfp4_validate.py:51-65)."""
    assert x.shape[-1] % BLK == 0, f"last dim {x.shape[-1]} not divisible by {BLK}"
    xf = x.float()
    amax_all = xf.abs().amax().clamp_min(1e-12)
    blocks = xf.reshape(*x.shape[:-1], x.shape[-1] // BLK, BLK)
    if u is not None:
        u = u.reshape(blocks.shape)
    return _fake_quant(blocks, -1, amax_all, stochastic, u).reshape(x.shape).to(x.dtype)


def quantize_2d(w: torch.Tensor, stochastic: bool = False) -> torch.Tensor:
    """Fake-quant of a weight [out, in] with one scale per 16x16 tile (nvfp4_validate.py:68-82): the
    quantized weight is then the same whether it is read along `in` (fprop) or along `out` (dgrad)."""
    out, cin = w.shape
    wf = w.float()
    amax_all = wf.abs().amax().clamp_min(1e-12)
    tiles = wf.reshape(out // BLK, BLK, cin // BLK, BLK)
    return _fake_quant(tiles, (1, 3), amax_all, stochastic).reshape(out, cin).to(w.dtype)


def hadamard16(device, dtype=torch.float32) -> torch.Tensor:
    h = torch.ones(1, 1, device=device, dtype=dtype)
    while h.shape[0] < BLK:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(BLK)


def rht_lastdim(x: torch.Tensor, H: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """(x_tile * signs) @ H over tiles of 16 along the last dim (nvfp4_validate.py:92-99)."""
    tiles = x.reshape(*x.shape[:-1], x.shape[-1] // BLK, BLK)
    return ((tiles * signs) @ H).reshape(x.shape)


class SimLinearFn(torch.autograd.Function):
    """x [N, Cin], w [Cout, Cin] -> [N, Cout] with the recipe of nvfp4_validate.py:104-140.
    sr / rht switch the stochastic rounding of gradients and the Hadamard of the wgrad operands."""

    @staticmethod
    def forward(ctx, x, w, sr, rht, H, signs):
        y = (quantize_1d(x).float() @ quantize_2d(w).float().t()).to(x.dtype)
        ctx.save_for_backward(x, w)
        ctx.sr, ctx.rht, ctx.H, ctx.signs = sr, rht, H, signs
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        # dgrad: dY along Cout (stochastic), the same 2-D quantized weight as forward
        dx = (quantize_1d(gy, stochastic=ctx.sr).float() @ quantize_2d(w).float()).to(x.dtype)
        # wgrad: contraction over tokens -> transpose both, pad the token dim to a multiple of 16
        xt, gt = x.t().contiguous(), gy.t().contiguous()
        pad = (-xt.shape[-1]) % BLK
        if pad:
            xt, gt = F.pad(xt, (0, pad)), F.pad(gt, (0, pad))
        if ctx.rht:
            xt, gt = rht_lastdim(xt, ctx.H, ctx.signs), rht_lastdim(gt, ctx.H, ctx.signs)
        dw = (quantize_1d(gt, stochastic=ctx.sr).float() @ quantize_1d(xt).float().t()).to(w.dtype)
        return dx, dw, None, None, None, None


class SimLinear(nn.Module):
    """nn.Linear(cin, cout, bias=False) whose three matmuls go through the simulator
    (nvfp4_validate.py:143-157).  Same initialisation and sign vector as the reference."""

    def __init__(self, cin, cout, sr=True, rht=True, device="cpu"):
        super().__init__()
        assert cin % BLK == 0 and cout % BLK == 0
        self.weight = nn.Parameter(torch.empty(cout, cin, device=device))
        nn.init.normal_(self.weight, std=0.02)
        self.sr, self.rht = sr, rht
        self.register_buffer("H", hadamard16(device), persistent=False)
        g = torch.Generator().manual_seed(1)
        self.register_buffer("signs", (torch.randint(0, 2, (BLK,), generator=g).float() * 2 - 1).to(device),
                             persistent=False)

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        y = SimLinearFn.apply(x2, self.weight, self.sr, self.rht, self.H, self.signs)
        return y.reshape(*x.shape[:-1], -1)
