"""SwiGLU feed-forward block built from FP4Linear (or bf16 nn.Linear as the comparator): the FFN of
BASELINE config 4 (d_model 4096, hidden 14336, three linears, Kaiming-uniform weights)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import make_linear


class SwiGLUFFN(nn.Module):
    """y = down(silu(gate(x)) * up(x)); every linear is an FP4Linear when use_fp4."""

    def __init__(self, d_model, hidden, use_fp4=True, device="cuda", seed=None):
        super().__init__()
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

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


def ffn_flops(tokens, d_model, hidden):
    """Forward + backward matmul flops of one microbatch: 3 linears x 3 GEMMs x 2 T d h."""
    return 3 * 3 * 2.0 * tokens * d_model * hidden
