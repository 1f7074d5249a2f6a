"""FP4Linear autograd and the per-step weight-quant cache (nvfp4_train.py:19-88,
tests/parity_check.py of the reference)."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


@pytest.fixture(autouse=True)
def _reset(Q):
    Q.set_amortize(False)
    yield
    Q.set_amortize(False)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_forward_backward_match_oracle_recipe(Q):
    """fprop RNE, dgrad SR, wgrad RHT+SR reproduced on the CPU oracle with the same Philox seeds:
    outputs agree to the GEMM tolerance (bf16 rounding of y and dx on top)."""
    from nvfp4_sm120_b200 import quant
    M, K, N = 256, 512, 384
    lin = Q.FP4Linear(K, N)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(N, K, generator=g) * 0.02)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    xc = x.cuda().requires_grad_(True)
    quant._SEED[0] = 1000
    y = lin(xc)
    y.backward(gy.cuda())
    assert quant._SEED[0] == 1002                 # two stochastic quantizations: dgrad dY, wgrad dY^T

    w = lin.weight.detach().cpu().to(torch.bfloat16)
    signs = O.signs_from_seed(1)
    y_ref = O.dequant(O.quant_nvfp4(x)) @ O.dequant(O.quant_nvfp4(w)).t()
    assert _rel(y.cpu(), y_ref.to(torch.bfloat16)) < 2e-3
    # dgrad: seed 1000
    rb = O.philox_block_bits(M * N // 16, 1000, 0)
    gq = O.dequant(O.quant_nvfp4(gy, stochastic=True, rbits=rb))
    dx_ref = gq @ O.dequant(O.quant_nvfp4(w.t().contiguous())).t()
    assert _rel(xc.grad.cpu(), dx_ref.to(torch.bfloat16)) < 2e-3
    # wgrad: seed 1001, Hadamard along the token dim on both operands
    gyt, xt = gy.t().contiguous(), x.t().contiguous()
    rb = O.philox_block_bits(M * N // 16, 1001, 0)
    gtq = O.dequant(O.quant_nvfp4(gyt, stochastic=True, rht=True, signs=signs, rbits=rb, rht_impl="butterfly"))
    xtq = O.dequant(O.quant_nvfp4(xt, rht=True, signs=signs, rht_impl="butterfly"))
    dw_ref = gtq @ xtq.t()
    assert lin.weight.grad.dtype == torch.float32
    assert _rel(lin.weight.grad.cpu(), dw_ref) < 1e-3


def test_gradients_close_to_exact(Q):
    """Quantisation-level agreement with the exact bf16 linear, like the simulator's
    (nvfp4_validate.py:104-140) error levels."""
    M, K, N = 512, 1024, 768
    lin = Q.FP4Linear(K, N)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y = lin(x)
    y.backward(gy)
    w = lin.weight.detach().float()
    assert _rel(y, x.detach().float() @ w.t()) < 0.2
    assert _rel(x.grad, gy.float() @ w) < 0.25
    assert _rel(lin.weight.grad, gy.float().t() @ x.detach().float()) < 0.25
    assert y.dtype == torch.bfloat16 and x.grad.dtype == torch.bfloat16


def test_3d_input_and_fp32_activation(Q):
    lin = Q.FP4Linear(256, 128)
    x = torch.randn(4, 32, 256, device="cuda", requires_grad=True)          # fp32 in -> fp32 out
    y = lin(x)
    assert y.shape == (4, 32, 128) and y.dtype == torch.float32
    y.sum().backward()
    assert x.grad.shape == x.shape and lin.weight.grad.shape == (128, 256)


def test_amortized_cache_semantics(Q):
    """tests/parity_check.py: same step -> identical (cached); weight change + mark_step -> output
    changes; weight change WITHOUT mark_step -> stale output."""
    Q.set_amortize(True)
    torch.manual_seed(0)
    m = Q.FP4Linear(512, 512)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    Q.mark_step()
    y1 = m(x)
    y2 = m(x)
    assert torch.equal(y1, y2)
    with torch.no_grad():
        m.weight.add_(1.0)
    Q.mark_step()
    y3 = m(x)
    assert not torch.allclose(y1, y3)
    with torch.no_grad():
        m.weight.add_(1.0)
    y4 = m(x)
    assert torch.allclose(y3, y4)            # stale: training must call mark_step() every step


def test_amortized_equals_non_amortized(Q):
    """The cached weight quantizations are the ones the non-amortized path computes per call."""
    from nvfp4_sm120_b200 import quant
    torch.manual_seed(1)
    m = Q.FP4Linear(256, 384)
    x = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    gy = torch.randn(128, 384, device="cuda", dtype=torch.bfloat16)
    outs = []
    for amort in (False, True):
        Q.set_amortize(amort)
        Q.mark_step()
        quant._SEED[0] = 50
        xi = x.clone().requires_grad_(True)
        m.weight.grad = None
        y = m(xi)
        y.backward(gy)
        outs.append((y.detach().clone(), xi.grad.clone(), m.weight.grad.clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_make_linear(Q):
    assert isinstance(Q.make_linear(64, 32, True), Q.FP4Linear)
    lin = Q.make_linear(64, 32, False)
    assert isinstance(lin, torch.nn.Linear) and lin.bias is None
    with pytest.raises(AssertionError):
        Q.FP4Linear(40, 32)


def test_chained_linears_pass_the_maximum_through_the_gemm_epilogue(Q):
    """y = l1(x, amax_out=word); z = l2(y, amax=word): the first layer's GEMM leaves max|y| for the second
    layer's quantizer.  Outputs and all gradients equal those of the plain chain, bit for bit."""
    from nvfp4_sm120_b200 import quant
    torch.manual_seed(11)
    l1, l2 = Q.FP4Linear(256, 512), Q.FP4Linear(512, 128)
    x0 = torch.randn(192, 256, device="cuda", dtype=torch.bfloat16)
    gz = torch.randn(192, 128, device="cuda", dtype=torch.bfloat16)

    def run(chained):
        for l in (l1, l2):
            l.weight.grad = None
        quant._SEED[0] = 500
        x = x0.clone().requires_grad_(True)
        if chained:
            word = torch.zeros(1, dtype=torch.float32, device="cuda")
            y = l1(x, amax_out=word)
            assert float(word) == float(y.detach().abs().max().float())
            z = l2(y, amax=word)
        else:
            z = l2(l1(x))
        z.backward(gz)
        return z.detach(), x.grad, l1.weight.grad.clone(), l2.weight.grad.clone()

    for a, b in zip(run(True), run(False)):
        assert torch.equal(a, b)


def test_shared_input_quantization_equals_per_layer_quantization(Q):
    """quant_input: one quantization of an activation (both layouts) handed to several layers through
    x_quant= gives the outputs and gradients of the layers quantizing it themselves, bit for bit; without
    gradients (evaluation) only the row-wise operand is made."""
    from nvfp4_sm120_b200 import quant
    torch.manual_seed(12)
    a, b = Q.FP4Linear(256, 128), Q.FP4Linear(256, 384)
    for tokens in (192, 224):
        x0 = torch.randn(tokens, 256, device="cuda", dtype=torch.bfloat16)
        ga = torch.randn(tokens, 128, device="cuda", dtype=torch.bfloat16)
        gb = torch.randn(tokens, 384, device="cuda", dtype=torch.bfloat16)

        def run(shared):
            for l in (a, b):
                l.weight.grad = None
            quant._SEED[0] = 700
            x = x0.clone().requires_grad_(True)
            if shared:
                xq = a.quant_input(x)
                assert xq[1] is not None
                ya, yb = a(x, x_quant=xq), b(x, x_quant=xq)
            else:
                ya, yb = a(x), b(x)
            torch.autograd.backward([ya, yb], [ga, gb])
            return ya.detach(), yb.detach(), x.grad, a.weight.grad.clone(), b.weight.grad.clone()

        for u, v in zip(run(True), run(False)):
            assert torch.equal(u, v)
    with torch.no_grad():
        xq = a.quant_input(x0)
        assert xq[1] is None and torch.equal(a(x0, x_quant=xq), a(x0))
