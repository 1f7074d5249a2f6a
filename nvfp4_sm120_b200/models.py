"""Decoder-only language models whose linears are FP4Linear: the callers of the hot path.

`GPT` is the nanoGPT-style model of the reference's scaling study (scaling/train_text.py:37-92:
RMSNorm, rotary positions, grouped-query attention, squared-ReLU MLP, tied head, first block and the
last `hp_tail` blocks kept in high precision); `LM` is the small model of its addition-task trainer
(nvfp4_train.py:101-140: same block, untied head, hp rule `i == 0 or i >= n_layers - hp_tail`).
Attention, norms, embedding and head stay bf16/fp32 torch ops, as in the reference."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import FP4Linear, make_linear
from .norm import rmsnorm_amax
from .swiglu import relu2


@dataclass
class GPTConfig:
    vocab: int = 50257
    dim: int = 768
    n_layers: int = 12
    n_heads: int = 12
    n_kv_heads: int = 12
    mlp_ratio: int = 4
    use_fp4: bool = True
    hp_tail: int = 1           # last blocks kept dense (scaling/train_text.py:66-67)
    dense_first: bool = True   # block 0 kept dense, the reference's rule; False + hp_tail 0 = every
                               # linear of every block in FP4 (benchmark config 5 as written)
    tie_head: bool = True


def rotary_tables(seq_len, head_dim, device):
    """cos / sin tables [1, 1, T, head_dim / 2] with base 10000 (nvfp4_train.py:91-98)."""
    half = head_dim // 2
    freq = 10000.0 ** (-torch.arange(half, device=device, dtype=torch.float32) / half)
    angle = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * freq[None, :]
    return angle.cos()[None, None], angle.sin()[None, None]


def apply_rotary(x, cos, sin):
    """Rotate the two halves of the head dimension against each other."""
    a, b = x.chunk(2, dim=-1)
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


class DecoderBlock(nn.Module):
    """linear_factory: optional callable (cin, cout) -> module that builds the block's low-precision
    linears in place of FP4Linear (used to run the same model with another implementation of the
    recipe, e.g. a fake-quant simulator, for loss-curve comparisons)."""

    def __init__(self, dim, n_heads, n_kv_heads, hidden, use_fp4, device, linear_factory=None):
        super().__init__()
        assert dim % n_heads == 0 and n_heads % n_kv_heads == 0
        self.n_heads, self.n_kv, self.head_dim = n_heads, n_kv_heads, dim // n_heads
        self.norm_attn, self.norm_mlp = nn.RMSNorm(dim, device=device), nn.RMSNorm(dim, device=device)
        kv_dim = n_kv_heads * self.head_dim
        if use_fp4 and linear_factory is not None:
            mk = lambda cin, cout: linear_factory(cin, cout)
        else:
            mk = lambda cin, cout: make_linear(cin, cout, use_fp4, device)
        self.q = mk(dim, dim)
        self.k = mk(dim, kv_dim)
        self.v = mk(dim, kv_dim)
        self.o = mk(dim, dim)
        self.up = mk(dim, hidden)
        self.down = mk(hidden, dim)
        # the fused activation computes the Hadamard maxima for `down` and for `up`'s gradient with
        # `down`'s sign vector; a consumer holding another vector recomputes its maximum (checked at
        # call time: a checkpoint may change the buffers)
        self.fused_act = bool(use_fp4) and isinstance(self.up, FP4Linear) and isinstance(self.down, FP4Linear)
        # the norms in front of FP4 projections run as the fused kernel that also finds the maxima of
        # its output (one sign vector serves q, k, v; each consumer checks it against its own)
        self.fused_norm = bool(use_fp4) and all(isinstance(m, FP4Linear) for m in (self.q, self.k, self.v, self.up))

    def _norm(self, norm, x, consumer):
        """norm(x) -> (h, maxima or None): the fused kernel when the consumers are FP4Linear on the GPU."""
        if (self.fused_norm and x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.shape[-1] % 8 == 0
                and norm.weight is not None and norm.weight.dtype == torch.float32):
            tokens = x.numel() // x.shape[-1]
            return rmsnorm_amax(x, norm.weight, norm.eps, consumer.signs if tokens % 16 == 0 else None)
        return norm(x), None

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        h, h_max = self._norm(self.norm_attn, x, self.q)
        split = lambda t, n: t.view(B, T, n, self.head_dim).transpose(1, 2)
        if h_max is not None:
            from .linear import _same_signs
            if _same_signs(self.q.signs, self.k.signs) and _same_signs(self.q.signs, self.v.signs):
                # one quantization of h (both layouts) serves the three projections
                hq = self.q.quant_input(h, h_max, self.q.signs)
                q, k, v = self.q(h, x_quant=hq), self.k(h, x_quant=hq), self.v(h, x_quant=hq)
            else:
                kw = dict(amax=h_max, amax_signs=self.q.signs)
                q, k, v = self.q(h, **kw), self.k(h, **kw), self.v(h, **kw)
        else:
            q, k, v = self.q(h), self.k(h), self.v(h)
        q, k, v = split(q, self.n_heads), split(k, self.n_kv), split(v, self.n_kv)
        q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
        if self.n_kv != self.n_heads:
            rep = self.n_heads // self.n_kv
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o(att.transpose(1, 2).reshape(B, T, -1))
        h2, h2_max = self._norm(self.norm_mlp, x, self.up)
        u = self.up(h2, amax=h2_max, amax_signs=self.up.signs) if h2_max is not None else self.up(h2)
        if (self.fused_act and isinstance(self.down, FP4Linear) and u.is_cuda and u.dtype == torch.bfloat16
                and u.shape[-1] % 8 == 0):
            # fused relu^2 that also hands `down` the maxima of its input (and `up` those of its gradient)
            a, a_max = relu2(u, self.down.signs if (B * T) % 16 == 0 else None)
            return x + self.down(a, amax=a_max, amax_signs=self.down.signs)
        return x + self.down(F.relu(u).square())


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, device="cuda", linear_factory=None):
        super().__init__()
        self.cfg = cfg
        self.emb = nn.Embedding(cfg.vocab, cfg.dim, device=device)
        fp4_at = lambda i: cfg.use_fp4 and not ((i == 0 and cfg.dense_first) or i >= cfg.n_layers - cfg.hp_tail)
        self.blocks = nn.ModuleList(
            DecoderBlock(cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.mlp_ratio * cfg.dim, fp4_at(i), device, linear_factory)
            for i in range(cfg.n_layers))
        self.norm = nn.RMSNorm(cfg.dim, device=device)
        self.head = nn.Linear(cfg.dim, cfg.vocab, bias=False, device=device)
        if cfg.tie_head:
            self.head.weight = self.emb.weight
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
        self._rope = None

    def forward(self, idx, targets=None):
        T = idx.shape[1]
        if self._rope is None or self._rope[0].shape[2] != T or self._rope[0].device != idx.device:
            self._rope = rotary_tables(T, self.cfg.dim // self.cfg.n_heads, idx.device)
        cos, sin = self._rope
        x = self.emb(idx)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits, None
        return logits, F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1))

    def num_params(self):
        """Non-embedding parameter count (the tied head counts once, as the embedding)."""
        return sum(p.numel() for p in self.parameters()) - self.emb.weight.numel()

    def fp4_linears(self):
        from .linear import FP4Linear
        return [m for m in self.modules() if isinstance(m, FP4Linear)]


class LM(GPT):
    """The addition-task model of nvfp4_train.py:126-140: untied head, hp_tail counted from the end,
    block 0 dense when FP4 is on."""

    def __init__(self, vocab, dim, nl, nh, nkv, hd, ffn, use_fp4, hp_tail=0, device="cuda", linear_factory=None):
        assert hd * nh == dim and ffn % dim == 0
        super().__init__(GPTConfig(vocab=vocab, dim=dim, n_layers=nl, n_heads=nh, n_kv_heads=nkv,
                                   mlp_ratio=ffn // dim, use_fp4=use_fp4, hp_tail=hp_tail, tie_head=False), device,
                         linear_factory)

    def forward(self, idx):
        return super().forward(idx)[0]
