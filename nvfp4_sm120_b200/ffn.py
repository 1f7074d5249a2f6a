"""SwiGLU feed-forward block built from FP4Linear (or bf16 nn.Linear as the comparator): the FFN of
benchmark config 4 (d_model 4096, hidden 14336, three linears, Kaiming-uniform weights)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import FP4Linear, make_linear
from .swiglu import swiglu, swiglu_packed


class SwiGLUFFN(nn.Module):
    """y = down(silu(gate(x)) * up(x)); every linear is an FP4Linear when use_fp4.  With FP4 linears
    and bf16 activations the SwiGLU product and its backward run as fused kernels that also hand
    the following quantizations their per-tensor maxima (fused=False keeps the torch ops)."""

    def __init__(self, d_model, hidden, use_fp4=True, device="cuda", seed=None, fused=True, fuse_gate_up=False):
        """fuse_gate_up: keep the gate and up weights as ONE [2 hidden, d_model] projection (rows 0..hidden-1
        gate, the rest up; same initial values as the two separate linears).  x is then quantized once
        per layout instead of twice, the two input-gradient GEMMs and their sum become one GEMM over
        K = 2 hidden, and the SwiGLU kernels read / write the packed [tokens, 2 hidden] tensors in place.
        The per-tensor scale of the fused weight and of its output gradient spans both halves."""
        super().__init__()
        self.fused = bool(fused and use_fp4)
        self.fuse_gate_up = bool(fuse_gate_up and self.fused)
        self.hidden = hidden
        g = None
        if seed is not None:
            g = torch.Generator(device=device).manual_seed(seed)
        if self.fuse_gate_up:
            self.gate_up = make_linear(d_model, 2 * hidden, use_fp4, device)
            self.down = make_linear(hidden, d_model, use_fp4, device)
            with torch.no_grad():
                bound = 1.0 / math.sqrt(d_model)
                self.gate_up.weight[:hidden].uniform_(-bound, bound, generator=g)      # gate rows ...
                self.gate_up.weight[hidden:].uniform_(-bound, bound, generator=g)      # ... then up rows
                self.down.weight.uniform_(-1.0 / math.sqrt(hidden), 1.0 / math.sqrt(hidden), generator=g)
            return
        self.gate = make_linear(d_model, hidden, use_fp4, device)
        self.up = make_linear(d_model, hidden, use_fp4, device)
        self.down = make_linear(hidden, d_model, use_fp4, device)
        with torch.no_grad():
            for lin in (self.gate, self.up, self.down):
                bound = 1.0 / math.sqrt(lin.weight.shape[1])          # kaiming_uniform_(a=sqrt(5))
                lin.weight.uniform_(-bound, bound, generator=g)

        # One sign vector serves the Hadamard maxima the fused kernels compute; a consumer whose own
        # vector differs (a checkpoint may change the buffers) recomputes that maximum, see
        # FP4Linear.forward(amax_signs=) and linear.hint_grad_amax(signs=).

    def forward(self, x):
        if self.fuse_gate_up:
            gu = self.gate_up(x)
            if gu.dtype == torch.bfloat16 and gu.is_cuda:
                h, h_max = swiglu_packed(gu, self.gate_up.signs if gu.numel() // gu.shape[-1] % 16 == 0 else None)
                return self.down(h, amax=h_max, amax_signs=self.gate_up.signs)
            return self.down(F.silu(gu[..., :self.hidden]) * gu[..., self.hidden:])
        g, u = self.gate(x), self.up(x)
        if self.fused and isinstance(self.down, FP4Linear) and g.dtype == torch.bfloat16 and g.is_cuda:
            h, h_max = swiglu(g, u, self.gate.signs if g.numel() // g.shape[-1] % 16 == 0 else None)
            return self.down(h, amax=h_max, amax_signs=self.gate.signs)
        return self.down(F.silu(g) * u)


def ffn_flops(tokens, d_model, hidden):
    """Forward + backward matmul flops of one microbatch: 3 linears x 3 GEMMs x 2 T d h."""
    return 3 * 3 * 2.0 * tokens * d_model * hidden
