"""The drop-in claim: with `nvfp4_sm120_b200/compat` on sys.path the reference's module names
(`nvfp4_gemm`, `nvfp4_cuda`, `nvfp4_train`, `nvfp4_validate`, `nvfp4_triton_quant`) resolve to this
build, and the bodies of the reference's own check scripts run against them unchanged.  The bodies
are restated here (the GPU box has no reference checkout): tests/parity_check.py:5-26,
tests/cuda_val.py:9-26 and tests/verify_amort.py:11-23, with their printed relations turned into
assertions and the loop counts cut to seconds."""
import os
import sys

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMPAT = os.path.join(ROOT, "nvfp4_sm120_b200", "compat")
NAMES = ("nvfp4_gemm", "nvfp4_cuda", "nvfp4_train", "nvfp4_validate", "nvfp4_triton_quant")


@pytest.fixture()
def ref_names():
    """The reference's module names, imported from the compat directory."""
    import importlib
    saved_path = list(sys.path)
    saved_mods = {n: sys.modules.pop(n, None) for n in NAMES}
    sys.path.insert(0, COMPAT)
    try:
        mods = {n: importlib.import_module(n) for n in NAMES}
        for n, m in mods.items():
            assert os.path.dirname(os.path.abspath(m.__file__)) == COMPAT, n
        yield mods
    finally:
        sys.path[:] = saved_path
        for n in NAMES:
            sys.modules.pop(n, None)
            if saved_mods[n] is not None:
                sys.modules[n] = saved_mods[n]
        from nvfp4_sm120_b200 import linear
        linear.set_amortize(False)


def test_module_surface(ref_names):
    """Every name the reference's scripts import or call exists under the reference's module names."""
    G, C, TR, D, T = (ref_names[n] for n in NAMES)
    for name in ("quant_nvfp4", "fp4_matmul", "hadamard16", "BLK", "F4_MAX", "F8E4M3_MAX", "E4M3_EPS"):
        assert hasattr(G, name), name
    for name in ("quant_nvfp4_cuda", "fp4_matmul_cuda", "fp4_mm_preqB", "hadamard16", "_ext"):
        assert hasattr(C, name), name
    for name in ("FP4Linear", "FP4LinearFn", "mark_step", "make_linear", "_AMORTIZE", "_STEP", "LM", "Block",
                 "rope", "evaluate", "run"):
        assert hasattr(TR, name), name
    for name in ("VOCAB", "STOI", "SEQ", "ANS_SLICE", "encode_pair", "build_dataset", "make_batch"):
        assert hasattr(D, name), name
    assert hasattr(T, "quant_nvfp4_fused") and hasattr(T, "fp4_matmul_fused")
    assert C._ext() is not None
    assert "".join(D.VOCAB[i] for i in D.encode_pair(7, 456)) == "007+456=0463\n"


def test_parity_check_body(ref_names):
    """tests/parity_check.py:5-26 of the reference, its three printed relations asserted."""
    TR = ref_names["nvfp4_train"]
    from nvfp4_sm120_b200 import linear
    linear.set_amortize(True)                       # the script is run with NVFP4_AMORTIZE=1
    assert TR._AMORTIZE is True
    FP4Linear, mark_step = TR.FP4Linear, TR.mark_step
    dev = "cuda"
    torch.manual_seed(0)
    m = FP4Linear(512, 512).cuda()
    x = torch.randn(256, 512, device=dev, dtype=torch.bfloat16, requires_grad=True)
    mark_step()
    y1 = m(x)
    y2 = m(x)
    assert torch.equal(y1, y2)                                        # same-step fprop identical
    with torch.no_grad():
        m.weight.add_(1.0)
    mark_step()
    y3 = m(x)
    assert not torch.allclose(y1, y3)                                 # cache refreshed
    with torch.no_grad():
        m.weight.add_(1.0)
    y4 = m(x)
    assert torch.allclose(y3, y4)                                     # stale without mark_step


def _pk(t):
    """tests/cuda_val.py:5-8: the packed bytes of a quantized tensor, whatever the attribute is called."""
    for a in ("qdata", "_data", "data"):
        v = getattr(t, a, None)
        if isinstance(v, torch.Tensor) and v.dtype == torch.uint8:
            return v


def test_cuda_val_body(ref_names):
    """tests/cuda_val.py:9-26: RNE byte match between the two quantizer names over its shape sweep,
    GEMM error against fp32 and stochastic-rounding unbiasedness over 32 draws (on its first GEMM
    shape; the second differs only in size)."""
    G, C = ref_names["nvfp4_gemm"], ref_names["nvfp4_cuda"]
    torch.manual_seed(0)
    dev = "cuda"
    worst = 1.0
    for (M, K) in [(256, 512), (1024, 1024), (8192, 4096), (5328, 768), (2048, 2048)]:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16) * 3
        worst = min(worst, (_pk(G.quant_nvfp4(x)) == _pk(C.quant_nvfp4_cuda(x))).float().mean().item())
    assert worst == 1.0
    M, K, N = 2048, 2048, 2048
    A = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    B = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
    ref = A.float() @ B.float()
    rn = ref.norm()
    rne = ((C.fp4_matmul_cuda(A, B).float() - ref).norm() / rn).item()
    acc = torch.zeros_like(ref)
    for i in range(32):
        acc += C.fp4_matmul_cuda(A, B, sr_a=True, sr_b=True, seed=100 + i).float()
    sr = ((acc / 32 - ref).norm() / rn).item()
    assert sr < rne                                                   # "SR unbiased"
    assert 0.05 < rne < 0.2
    # the Triton module name gives the same bytes and the same product
    T = ref_names["nvfp4_triton_quant"]
    assert torch.equal(_pk(T.quant_nvfp4_fused(A)), _pk(C.quant_nvfp4_cuda(A)))
    assert torch.equal(T.fp4_matmul_fused(A, B), C.fp4_matmul_cuda(A, B))


def test_verify_amort_body(ref_names):
    """tests/verify_amort.py:11-23: the FFN it times (RMSNorm, two FP4Linear, squared ReLU, residual),
    G microbatches per step with one mark_step(), runs and gives finite gradients; amortized and
    non-amortized steps agree exactly when fed the same stochastic-rounding seeds."""
    TR = ref_names["nvfp4_train"]
    from nvfp4_sm120_b200 import linear, quant
    FP4Linear, mark_step = TR.FP4Linear, TR.mark_step
    dev = "cuda"

    class FFN(nn.Module):
        def __init__(s, d, h):
            super().__init__()
            s.up = FP4Linear(d, h)
            s.dn = FP4Linear(h, d)
            s.n = nn.RMSNorm(d).cuda()

        def forward(s, x):
            return x + s.dn(F.relu(s.up(s.n(x))) ** 2)

    T_, d, h, Gm = 512, 1024, 3584, 4
    torch.manual_seed(0)
    m = FFN(d, h).to(dev)
    xs = [torch.randn(T_, d, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(Gm)]

    def step():
        mark_step()
        out = []
        for g in range(Gm):
            y = m(xs[g])
            out.append(torch.autograd.grad(y.sum(), [xs[g]] + list(m.parameters())))
        return out

    res = {}
    for amort in (False, True):
        linear.set_amortize(amort)
        quant._SEED[0] = 4242
        res[amort] = step()
    for ga, gb in zip(res[False], res[True]):
        for a, b in zip(ga, gb):
            assert torch.isfinite(a).all()
            assert torch.equal(a, b)
