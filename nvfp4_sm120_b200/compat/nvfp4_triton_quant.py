"""Drop-in for the reference's nvfp4_triton_quant module (nvfp4_triton_quant.py:132-175).  There
is no Triton in this build: the names resolve to the same sm_100a CUDA kernels as nvfp4_cuda, which
do in one launch what the reference's Triton kernel does (in-kernel Hadamard, counter-based
stochastic rounding, packed nibbles and swizzled scales)."""
from nvfp4_sm120_b200.quant import quant_nvfp4 as quant_nvfp4_fused, hadamard16      # noqa: F401
from nvfp4_sm120_b200.gemm import fp4_matmul as fp4_matmul_fused                    # noqa: F401
from nvfp4_sm120_b200.tensor import BLK                                             # noqa: F401
