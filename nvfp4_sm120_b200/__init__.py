"""B200-native (sm_100a) NVFP4 training hot path behind the reference's Python API.

quant_nvfp4 / fp4_matmul / fp4_mm_preqB, FP4Linear (fprop RNE, dgrad SR, wgrad RHT+SR) and the
NVFP4_AMORTIZE weight-quant cache with mark_step(), all on hand-written CUDA reached through the
C ABI of libnvfp4_b200.so."""
from .tensor import NVFP4Tensor, BLK, swizzled_scale_dims            # noqa: F401
from .quant import (quant_nvfp4, quant_nvfp4_cuda, quant_weight_nvfp4, quant_dual_nvfp4, tensor_amax, tensor_amax_both, hadamard16,      # noqa: F401
                    F4_MAX, F8E4M3_MAX, E4M3_EPS)
from .gemm import nvfp4_mm, nvfp4_mm_fp4out, fp4_matmul, fp4_matmul_cuda, fp4_mm_preqB, gemm_status      # noqa: F401
from .linear import FP4Linear, FP4LinearFn, mark_step, make_linear, set_amortize, set_dual_quant      # noqa: F401
from . import linear      # noqa: F401
