"""The C-ABI library builds, loads without a GPU, and exports every symbol include/nvfp4_b200.h
declares.  No compute calls here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from nvfp4_sm120_b200 import build, _lib
    build.build()
    return _lib


def test_header_declares_the_path():
    names = _declared()
    for want in ("nvfp4_amax_bf16", "nvfp4_quantize_bf16", "nvfp4_quantize_fused_bf16", "nvfp4_gemm",
                 "nvfp4_version", "nvfp4_status_string"):
        assert want in names


def test_every_declared_symbol_is_exported_and_bound(lib):
    handle = ctypes.CDLL(lib.LIB_PATH)
    for name in _declared():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert sorted(lib.exported_symbols()) == _declared()     # the ctypes table binds exactly the header


def test_version_and_status_strings(lib):
    L = lib.lib()
    assert L.nvfp4_version() == 1
    assert L.nvfp4_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert len(L.nvfp4_status_string(code)) > 3
    assert L.nvfp4_quantize_fused_workspace_bytes() == 64


def test_argument_validation_needs_no_gpu(lib):
    L = lib.lib()
    assert L.nvfp4_amax_bf16(None, 1, 16, 16, 0, 0, None, None, 1, None) == -1            # NULL
    assert L.nvfp4_quantize_bf16(None, 16, 32, 32, 0, 0, 0, None, None, 0, 0, None, None, None, None) == -1
    assert L.nvfp4_gemm(None, None, None, None, None, None, None, 0, 1, 1, 32, 1, None, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 255) & ~255                     # host memory: only argument checks run
    assert L.nvfp4_quantize_bf16(p, 16, 24, 24, 0, 0, 0, None, p, 0, 0, p, p, None, None) == -2   # K % 16
    assert L.nvfp4_quantize_bf16(p, 16, 32, 32, 0, 7, 0, None, p, 0, 0, p, p, None, None) == -4   # bad mode
    assert L.nvfp4_quantize_bf16(p + 2, 16, 32, 32, 0, 0, 0, None, p, 0, 0, p, p, None, None) == -3   # alignment
    assert L.nvfp4_gemm(p, p, p, p, p, p, p, 0, 128, 128, 48, 128, None, None) == -2               # K % 32
    assert L.nvfp4_quantize_fused_bf16(p, 16, 32, 32, 0, 0, None, 0, 0, p, p, None, p, 8, None) == -7  # workspace


def test_no_cpu_path_and_loud_failure(lib, monkeypatch):
    import torch
    import nvfp4_sm120_b200 as Q
    with pytest.raises(lib.NVFP4Error):
        Q.quant_nvfp4(torch.zeros(16, 32, dtype=torch.bfloat16))
    monkeypatch.setattr(lib, "LIB_PATH", "/nonexistent/libnvfp4_b200.so")
    monkeypatch.setattr(lib, "_lib", None)
    with pytest.raises(lib.NVFP4Error):
        lib.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "nvfp4_sm120_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle", src, flags=re.M), f
