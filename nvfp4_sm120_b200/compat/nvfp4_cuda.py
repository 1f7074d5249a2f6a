"""Drop-in for the reference's nvfp4_cuda module (nvfp4_cuda.py:154-207)."""
from nvfp4_sm120_b200.quant import (quant_nvfp4_cuda, hadamard16, _SEED,                     # noqa: F401
                                    F4_MAX, F8E4M3_MAX, E4M3_EPS)
from nvfp4_sm120_b200.gemm import fp4_matmul_cuda, fp4_mm_preqB                              # noqa: F401
from nvfp4_sm120_b200.tensor import BLK                                                      # noqa: F401
from nvfp4_sm120_b200 import _lib


def _ext():
    """The loaded native library (the reference returns its JIT-built extension module here,
    nvfp4_cuda.py:143-151).  Raises if libnvfp4_b200.so has not been built."""
    return _lib.lib()
