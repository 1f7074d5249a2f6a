"""SwiGLU feed-forward block built from FP4Linear (or bf16 nn.Linear as the comparator): the FFN of
benchmark config 4 (d_model 4096, hidden 14336, three linears, Kaiming-uniform weights)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import FP4Linear, make_linear
from .swiglu import swiglu


class SwiGLUFFN(nn.Module):
    """y = down(silu(gate(x)) * up(x)); every linear is an FP4Linear when use_fp4.  With FP4 linears
    and bf16 activations the SwiGLU product and its backward run as fused kernels that also hand
    the following quantizations their per-tensor maxima (fused=False keeps the torch ops)."""

    def __init__(self, d_model, hidden, use_fp4=True, device="cuda", seed=None, fused=True):
        super().__init__()
        self.fused = bool(fused and use_fp4)
        self.gate = make_linear(d_model, hidden, use_fp4, device)
        self.up = make_linear(d_model, hidden, use_fp4, device)
        self.down = make_linear(hidden, d_model, use_fp4, device)
        g = None
        if seed is not None:
            g = torch.Generator(device=device).manual_seed(seed)
        with torch.no_grad():
            for lin in (self.gate, self.up, self.down):
                bound = 1.0 / math.sqrt(lin.weight.shape[1])          # kaiming_uniform_(a=sqrt(5))
                lin.weight.uniform_(-bound, bound, generator=g)

        # One sign vector serves the Hadamard maxima the fused kernels compute; a consumer whose own
        # vector differs (a checkpoint may change the buffers) recomputes that maximum, see
        # FP4Linear.forward(amax_signs=) and linear.hint_grad_amax(signs=).

    def forward(self, x):
        g, u = self.gate(x), self.up(x)
        if self.fused and isinstance(self.down, FP4Linear) and g.dtype == torch.bfloat16 and g.is_cuda:
            h, h_max = swiglu(g, u, self.gate.signs if g.numel() // g.shape[-1] % 16 == 0 else None)
            return self.down(h, amax=h_max, amax_signs=self.gate.signs)
        return self.down(F.silu(g) * u)


def ffn_flops(tokens, d_model, hidden):
    """Forward + backward matmul flops of one microbatch: 3 linears x 3 GEMMs x 2 T d h."""
    return 3 * 3 * 2.0 * tokens * d_model * hidden
