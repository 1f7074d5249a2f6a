"""RMSNorm fused with the maxima of its output (csrc/rmsnorm.cu) against torch's rms_norm, and the
quantizations that take those maxima against the two-pass quantizations of the same tensor."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _signs(seed=1):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (16,), generator=g).float() * 2 - 1).cuda()


@pytest.mark.parametrize("rows,cols", [(256, 768), (48, 520), (37, 64), (1024, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forward_matches_torch_and_maxima_are_those_of_the_output(Q, rows, cols, dtype):
    from nvfp4_sm120_b200.norm import rmsnorm_amax
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = (torch.randn(rows, cols, device="cuda", generator=g) * 3).to(dtype)
    w = torch.rand(cols, device="cuda", generator=g) + 0.5
    signs = _signs()
    h, maxima = rmsnorm_amax(x, w, None, signs)
    ref = F.rms_norm(x.float(), (cols,), w, torch.finfo(dtype).eps)
    assert h.dtype == torch.bfloat16 and h.shape == x.shape
    # one rounding to bf16 of an fp32 result that may differ from torch's in the last bits
    assert (h.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    assert (h != ref.to(torch.bfloat16)).float().mean().item() < 2e-3
    assert float(maxima[0]) == float(h.abs().max().float())
    if rows % 16 == 0:
        assert float(maxima[1]) == float(Q.tensor_amax(h, rht=True, signs=signs, transpose=True))
    else:
        assert float(maxima[1]) == 0.0


def test_quantizations_with_the_given_maxima_equal_the_two_pass_ones(Q):
    from nvfp4_sm120_b200.norm import rmsnorm_amax
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(512, 768, device="cuda", generator=g)
    w = torch.rand(768, device="cuda", generator=g) + 0.5
    signs = _signs(3)
    h, maxima = rmsnorm_amax(x, w, None, signs)
    a, b = Q.quant_nvfp4(h, amax=maxima[0:1]), Q.quant_nvfp4(h)
    assert torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))
    assert torch.equal(a.per_tensor_scale, b.per_tensor_scale)
    H = Q.hadamard16("cuda")
    a = Q.quant_nvfp4(h, False, True, H, signs, transpose=True, amax=maxima[1:2])
    b = Q.quant_nvfp4(h, False, True, H, signs, transpose=True)
    assert torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))
    assert torch.equal(a.per_tensor_scale, b.per_tensor_scale)


@pytest.mark.parametrize("rows,cols", [(256, 768), (40, 520), (1000, 1024)])
@pytest.mark.parametrize("dtype,gdtype", [(torch.float32, torch.bfloat16), (torch.float32, torch.float32),
                                          (torch.bfloat16, torch.bfloat16)])
def test_backward_matches_torch_autograd(Q, rows, cols, dtype, gdtype):
    from nvfp4_sm120_b200.norm import rmsnorm_amax
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype).requires_grad_(True)
    w = (torch.rand(cols, device="cuda", generator=g) + 0.5).requires_grad_(True)
    gh = torch.randn(rows, cols, device="cuda", generator=g).to(gdtype)
    h, _ = rmsnorm_amax(x, w, None, None)
    (h.float() * gh.float()).sum().backward()
    dx, dw = x.grad.clone(), w.grad.clone()
    assert dx.dtype == dtype and dw.dtype == torch.float32
    x64 = x.detach().double().requires_grad_(True)
    w64 = w.detach().double().requires_grad_(True)
    ref = F.rms_norm(x64, (cols,), w64, torch.finfo(dtype).eps)
    # the fused function's gradient reaches it as bf16 (h is bf16): the same rounding here
    gh_seen = gh.float().to(torch.bfloat16).double() if True else gh.double()
    (ref * gh_seen).sum().backward()
    rel = lambda a, b: ((a.double() - b).norm() / b.norm()).item()
    assert rel(dx, x64.grad) < (3e-3 if dtype == torch.bfloat16 else 1e-5)
    assert rel(dw, w64.grad) < 1e-5


def test_block_with_fused_norms_tracks_the_block_with_torch_norms(Q):
    """The decoder block's fused norms change nothing but the last bits of h: outputs and gradients stay
    within the quantization tolerance of the block run with torch's RMSNorm."""
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.models import DecoderBlock, rotary_tables
    Q.set_amortize(False)
    torch.manual_seed(2)
    blk = DecoderBlock(128, 4, 4, 512, True, "cuda")
    assert blk.fused_norm
    gen = torch.Generator(device="cuda").manual_seed(3)
    x0 = torch.randn(2, 64, 128, device="cuda", generator=gen)
    gy = torch.randn(2, 64, 128, device="cuda", generator=gen)
    cos, sin = rotary_tables(64, 32, "cuda")

    def run(fused):
        blk.fused_norm = fused
        for p in blk.parameters():
            p.grad = None
        quant._SEED[0] = 900
        x = x0.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = blk(x, cos, sin)
        y.backward(gy)
        return [y.detach(), x.grad] + [p.grad.clone() for p in blk.parameters()]

    a, b = run(True), run(False)
    for u, v in zip(a, b):
        assert ((u.float() - v.float()).norm() / v.float().norm()).item() < 0.05
