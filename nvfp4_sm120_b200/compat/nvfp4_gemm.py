"""Drop-in for the reference's nvfp4_gemm module (nvfp4_gemm.py:20-57)."""
from nvfp4_sm120_b200.quant import quant_nvfp4, hadamard16, F4_MAX, F8E4M3_MAX, E4M3_EPS      # noqa: F401
from nvfp4_sm120_b200.gemm import fp4_matmul                                                 # noqa: F401
from nvfp4_sm120_b200.tensor import BLK, NVFP4Tensor                                         # noqa: F401
