"""ctypes binding of libnvfp4_b200.so (the C ABI declared in include/nvfp4_b200.h).

There is no fallback: if the library is missing or a call fails, an exception says so."""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# NVFP4_B200_LIB: another build of the same library (e.g. one compiled with different options)
LIB_PATH = os.environ.get("NVFP4_B200_LIB") or os.path.join(_PKG, "libnvfp4_b200.so")

OK = 0
ROUND_NEAREST, ROUND_STOCHASTIC = 0, 1
OUT_BF16, OUT_F32 = 0, 1

_c = ctypes
_SIGS = {
    "nvfp4_version": (_c.c_int, []),
    "nvfp4_status_string": (_c.c_char_p, [_c.c_int]),
    "nvfp4_amax_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                   _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_quantize_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                       _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_uint64, _c.c_uint64,
                                       _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nvfp4_quantize_shard_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                             _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_uint64, _c.c_uint64,
                                             _c.c_uint64, _c.c_uint64, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                             _c.c_void_p]),
    "nvfp4_quantize_fused_workspace_bytes": (_c.c_size_t, []),
    "nvfp4_quantize_fused_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                             _c.c_void_p, _c.c_uint64, _c.c_uint64, _c.c_void_p, _c.c_void_p,
                                             _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "nvfp4_quantize_static_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                              _c.c_void_p, _c.c_uint64, _c.c_uint64, _c.c_void_p, _c.c_void_p,
                                              _c.c_void_p, _c.c_void_p]),
    "nvfp4_quantize_weight_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p,
                                              _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_void_p]),
    "nvfp4_quantize_static_status": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_swiglu_fwd_bf16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p,
                                         _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_swiglu_bwd_bf16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64,
                                         _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int,
                                         _c.c_void_p]),
    "nvfp4_swiglu_bwd_strided_bf16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64,
                                                 _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int64,
                                                 _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_relu2_fwd_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int64,
                                        _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_relu2_bwd_bf16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p,
                                        _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_rmsnorm_fwd": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_float,
                                     _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_rmsnorm_bwd": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                     _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nvfp4_quantize_dual_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
                                            _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_uint64, _c.c_uint64,
                                            _c.c_uint64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                            _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nvfp4_amax_both_bf16": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p,
                                        _c.c_int, _c.c_void_p]),
    "nvfp4_gemm_set_mode": (_c.c_int, [_c.c_int]),
    "nvfp4_gemm_fp4out": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                     _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                     _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nvfp4_test_hooks": (_c.c_int, [_c.c_uint64, _c.c_int, _c.c_int]),
    "nvfp4_gemm_amax": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                   _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                   _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nvfp4_gemm": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                              _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                              _c.c_void_p, _c.c_void_p]),
}

_lib = None


class NVFP4Error(RuntimeError):
    pass


def lib():
    """The loaded library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NVFP4Error(
                f"{LIB_PATH} is missing: build it with `python -m nvfp4_sm120_b200.build` "
                "(needs nvcc; targets sm_100a).  There is no CPU or library fallback.")
        handle = _c.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)       # AttributeError here = a symbol the header declares is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def exported_symbols():
    return list(_SIGS)


def check(code, what):
    if code != OK:
        msg = lib().nvfp4_status_string(code).decode()
        raise NVFP4Error(f"{what} failed: {msg} (code {code})")


def cuda_device_of(*tensors):
    """The one CUDA device all `tensors` live on.  Raises NVFP4Error for a CPU tensor or for
    operands on different devices: the C side launches on the CURRENT device with the pointers it
    is given, so the wrappers make the operands' device current around every call."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise NVFP4Error(f"expected CUDA tensors, got one on {t.device} (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise NVFP4Error(f"operands on different devices: {dev} and {t.device}")
    if dev is None:
        raise NVFP4Error("no tensor operand")
    return dev
