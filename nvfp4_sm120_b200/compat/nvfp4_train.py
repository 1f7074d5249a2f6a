"""Drop-in for the FP4 part of the reference's nvfp4_train module (nvfp4_train.py:19-88)."""
from nvfp4_sm120_b200 import linear as _linear
from nvfp4_sm120_b200.linear import FP4Linear, FP4LinearFn, mark_step, make_linear, _STEP      # noqa: F401
from nvfp4_sm120_b200.gemm import fp4_matmul                                                   # noqa: F401
from nvfp4_sm120_b200.quant import hadamard16                                                  # noqa: F401
from nvfp4_sm120_b200.tensor import BLK                                                        # noqa: F401

DEV = "cuda"


def __getattr__(name):
    if name == "_AMORTIZE":            # live value: the cache switch can be flipped after import
        return _linear._AMORTIZE
    raise AttributeError(name)


# ---- model / trainer names of nvfp4_train.py:91-200, backed by models.py and addition.py ----------
import torch as _torch
import torch.nn as _nn

from nvfp4_sm120_b200 import addition as _addition
from nvfp4_sm120_b200.models import DecoderBlock as _DecoderBlock, LM as _LM, apply_rotary as _apply_rotary, \
    rotary_tables as _rotary_tables


def rope(x, T):
    """x: [B, H, T, Dh] -> rotary-embedded x (nvfp4_train.py:91-98)."""
    cos, sin = _rotary_tables(T, x.shape[-1], x.device)
    return _apply_rotary(x, cos, sin)


class Block(_nn.Module):
    """Block(dim, nh, nkv, hd, ffn, use_fp4) with forward(x), as nvfp4_train.py:101-123."""

    def __init__(self, dim, nh, nkv, hd, ffn, use_fp4):
        super().__init__()
        assert nh * hd == dim
        self.inner = _DecoderBlock(dim, nh, nkv, ffn, use_fp4, DEV)

    def forward(self, x):
        cos, sin = _rotary_tables(x.shape[1], self.inner.head_dim, x.device)
        return self.inner(x, cos, sin)


def LM(vocab, dim, nl, nh, nkv, hd, ffn, use_fp4, hp_tail=0):
    return _LM(vocab, dim, nl, nh, nkv, hd, ffn, use_fp4, hp_tail, device=DEV)


def evaluate(model, val, g, n=8, bs=512):
    """(held-out loss, exact-answer accuracy), nvfp4_train.py:143-156; `val` = the held-out pairs as
    nvfp4_validate.build_dataset returns them (a list of (a, b) tuples) or as a tensor of pair indices."""
    return _addition.evaluate(model, _addition.as_pair_indices(val), g, DEV, batches=n, batch=bs)


def run(tag, steps, use_fp4, hp_tail=0, seed=0):
    """One addition-task training run with the reference's settings (nvfp4_train.py:159-185)."""
    return _addition.run(tag, steps, use_fp4, hp_tail, seed, device=DEV)
