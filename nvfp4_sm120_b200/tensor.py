"""Container for an NVFP4-quantized operand, with the attribute names the reference's code
reads from torchao's NVFP4Tensor (constructed at nvfp4_gemm.py:48, read at tests/cuda_val.py:5-8)."""
from __future__ import annotations

import torch

BLK = 16


def swizzled_scale_dims(m: int, k: int) -> tuple[int, int]:
    """Padded [rows, cols] of the 128x4-tiled scale buffer of an [m, k] operand."""
    return ((m + 127) // 128) * 128, ((k // BLK + 3) // 4) * 4


class NVFP4Tensor:
    """qdata uint8 [M, K/2] (low nibble = even k), scale float8_e4m3fn swizzled [sM, sK],
    per_tensor_scale fp32 scalar tensor.  `.t()` returns a transposed VIEW object that shares the
    buffers (the reference passes `quant(B.t()).t()` as the right operand: nvfp4_gemm.py:56)."""

    __slots__ = ("qdata", "scale", "block_size", "orig_dtype", "per_tensor_scale",
                 "is_swizzled_scales", "_transposed")

    def __init__(self, qdata, scale, block_size=BLK, orig_dtype=torch.bfloat16, per_tensor_scale=None,
                 is_swizzled_scales=True, _transposed=False):
        self.qdata = qdata
        self.scale = scale
        self.block_size = block_size
        self.orig_dtype = orig_dtype
        self.per_tensor_scale = per_tensor_scale
        self.is_swizzled_scales = is_swizzled_scales
        self._transposed = _transposed

    @property
    def shape(self):
        m, k2 = self.qdata.shape
        return torch.Size((k2 * 2, m) if self._transposed else (m, k2 * 2))

    @property
    def device(self):
        return self.qdata.device

    @property
    def dtype(self):
        return self.orig_dtype

    def t(self):
        return NVFP4Tensor(self.qdata, self.scale, self.block_size, self.orig_dtype,
                           self.per_tensor_scale, self.is_swizzled_scales, not self._transposed)

    def __repr__(self):
        return (f"NVFP4Tensor(shape={tuple(self.shape)}, transposed_view={self._transposed}, "
                f"orig_dtype={self.orig_dtype})")
