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
