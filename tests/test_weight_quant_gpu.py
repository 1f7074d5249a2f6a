"""The dual-output weight quantizer (both operand layouts from one read of the weight): 1 x 16 scaling
bit-exact against the two separate quantizations and the oracle, and the 16 x 16 scaling mode of the
reference's simulator (nvfp4_validate.py:68-82) as real NVFP4 operands against its oracle restatement."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _same(q, o, what):
    assert torch.equal(q.qdata.cpu(), o.qdata), f"{what}: packed nibbles differ"
    assert torch.equal(q.scale.view(torch.uint8).cpu(), o.scale), f"{what}: block scales differ"
    assert torch.equal(q.per_tensor_scale.cpu().reshape(()), o.per_tensor_scale), f"{what}: pts differs"


@pytest.mark.parametrize("shape", [(64, 64), (48, 80), (256, 512), (1040, 272), (768, 3072)])
def test_one_d_matches_the_two_separate_quantizations(Q, shape):
    w = O.synthetic_tensor(shape[0], shape[1], 51)
    wr, wc = Q.quant_weight_nvfp4(w.cuda())
    _same(wr, O.quant_nvfp4(w), "rows")
    _same(wc, O.quant_nvfp4(w.t().contiguous()), "cols")
    a, b = Q.quant_nvfp4(w.cuda()), Q.quant_nvfp4(w.cuda(), transpose=True)
    assert torch.equal(wr.qdata, a.qdata) and torch.equal(wc.qdata, b.qdata)
    assert torch.equal(wr.scale.view(torch.uint8), a.scale.view(torch.uint8))
    assert torch.equal(wc.scale.view(torch.uint8), b.scale.view(torch.uint8))


@pytest.mark.parametrize("shape", [(64, 64), (48, 80), (256, 512), (1040, 272)])
def test_two_d_matches_oracle_and_layouts_agree(Q, shape):
    w = O.synthetic_tensor(shape[0], shape[1], 52)
    wr, wc = Q.quant_weight_nvfp4(w.cuda(), two_d=True)
    orow, ocol = O.quant_nvfp4_weight_2d(w)
    _same(wr, orow, "rows 2-D")
    _same(wc, ocol, "cols 2-D")
    n, k = shape
    dr = O.dequant_parts(wr.qdata, wr.scale.view(torch.uint8), wr.per_tensor_scale, n, k)
    dc = O.dequant_parts(wc.qdata, wc.scale.view(torch.uint8), wc.per_tensor_scale, k, n)
    assert torch.equal(dr, dc.t())                      # fprop and dgrad see the same quantized weight


def test_linear_with_two_d_weight_scaling(Q):
    """FP4Linear(weight_scaling="2d") on the cached path: forward and backward run, gradients stay at
    the quantisation level of the exact linear, and the cached operands are the 2-D ones."""
    from nvfp4_sm120_b200 import quant
    Q.set_amortize(True)
    try:
        Q.mark_step()
        torch.manual_seed(2)
        lin = Q.FP4Linear(256, 384, weight_scaling="2d")
        x = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        gy = torch.randn(128, 384, device="cuda", dtype=torch.bfloat16)
        quant._SEED[0] = 9
        y = lin(x)
        y.backward(gy)
        w = lin.weight.detach()
        orow, _ = O.quant_nvfp4_weight_2d(w.cpu().to(torch.bfloat16))
        assert torch.equal(lin._wq_K.qdata.cpu(), orow.qdata)
        rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
        assert rel(y, x.detach().float() @ w.t()) < 0.2
        assert rel(x.grad, gy.float() @ w) < 0.25
        assert rel(lin.weight.grad, gy.float().t() @ x.detach().float()) < 0.25
    finally:
        Q.set_amortize(False)
