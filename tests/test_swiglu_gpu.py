"""Fused SwiGLU (+ backward) with the maxima for the following quantizers: values against an fp32
torch reference, maxima bit-equal to the stand-alone amax kernels, and the FFN built on it against
the FFN built from torch element-wise ops."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _bits(t):
    return t.view(torch.int32)


@pytest.mark.parametrize("shape", [(16, 32), (256, 384), (1024, 14336), (48, 144)])
def test_forward_values_and_maxima(Q, shape):
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.swiglu import swiglu
    from oracle import nvfp4_oracle as O
    gen = torch.Generator(device="cuda").manual_seed(5)
    g = (torch.randn(*shape, device="cuda", generator=gen) * 2).to(torch.bfloat16)
    u = torch.randn(*shape, device="cuda", generator=gen).to(torch.bfloat16)
    signs = O.signs_from_seed(3).cuda()
    h, mx = swiglu(g, u, signs)
    ref = F.silu(g.float()) * u.float()
    assert h.dtype == torch.bfloat16 and h.shape == g.shape
    # one rounding to bf16 of an fp32 result computed with fast exp / divide
    assert torch.allclose(h.float(), ref, rtol=2.0 ** -7, atol=1e-6)
    # the maxima are those of the stored tensor, bit for bit
    assert torch.equal(_bits(mx[0:1]), _bits(quant.tensor_amax(h)))
    assert torch.equal(_bits(mx[1:2]), _bits(quant.tensor_amax(h, rht=True, signs=signs, transpose=True)))
    # so a quantizer that is handed them produces the bytes of the stand-alone path
    a = Q.quant_nvfp4(h, amax=mx[0:1])
    b = Q.quant_nvfp4(h)
    assert torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))
    at = Q.quant_nvfp4(h, rht=True, signs=signs, transpose=True, amax=mx[1:2])
    bt = Q.quant_nvfp4(h, rht=True, signs=signs, transpose=True)
    assert torch.equal(at.qdata, bt.qdata) and torch.equal(at.scale.view(torch.uint8), bt.scale.view(torch.uint8))


def test_rows_not_multiple_of_16_skip_the_row_transform(Q):
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.swiglu import swiglu
    g = torch.randn(37, 64, device="cuda").to(torch.bfloat16)
    u = torch.randn(37, 64, device="cuda").to(torch.bfloat16)
    h, mx = swiglu(g, u, torch.ones(16, device="cuda"))
    assert torch.allclose(h.float(), F.silu(g.float()) * u.float(), rtol=2.0 ** -7, atol=1e-6)
    assert torch.equal(_bits(mx[0:1]), _bits(quant.tensor_amax(h))) and float(mx[1]) == 0.0


def test_backward_values_maxima_and_hints(Q):
    from nvfp4_sm120_b200 import linear, quant
    from nvfp4_sm120_b200.swiglu import swiglu
    from oracle import nvfp4_oracle as O
    gen = torch.Generator(device="cuda").manual_seed(6)
    g = (torch.randn(512, 768, device="cuda", generator=gen) * 2).to(torch.bfloat16).requires_grad_(True)
    u = torch.randn(512, 768, device="cuda", generator=gen).to(torch.bfloat16).requires_grad_(True)
    dh = torch.randn(512, 768, device="cuda", generator=gen).to(torch.bfloat16)
    signs = O.signs_from_seed(3).cuda()
    linear._GRAD_AMAX.clear()
    h, _ = swiglu(g, u, signs)
    dg, du = torch.autograd.grad(h, [g, u], grad_outputs=dh)
    gf, uf = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
    rg, ru = torch.autograd.grad(F.silu(gf) * uf, [gf, uf], grad_outputs=dh.float())
    assert torch.allclose(dg.float(), rg, rtol=2.0 ** -6, atol=1e-5)
    assert torch.allclose(du.float(), ru, rtol=2.0 ** -6, atol=1e-5)
    # the hints registered for the two gradients are the maxima of the stored gradients
    for t in (dg, du):
        plain, rht = linear._take_grad_amax(t.reshape(-1, t.shape[-1]), signs)
        assert torch.equal(_bits(plain), _bits(quant.tensor_amax(t)))
        assert torch.equal(_bits(rht), _bits(quant.tensor_amax(t, rht=True, signs=signs, transpose=True)))
    assert linear._take_grad_amax(dg)[0] is None            # taken once


def test_fused_ffn_matches_unfused_ffn(Q):
    """Same weights, same input, same stochastic-rounding seeds: the fused block differs from the torch
    element-wise block only through the single rounding of h and of the two gradients."""
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.ffn import SwiGLUFFN
    Q.set_amortize(False)
    a = SwiGLUFFN(256, 512, use_fp4=True, device="cuda", seed=4, fused=True)
    b = SwiGLUFFN(256, 512, use_fp4=True, device="cuda", seed=4, fused=False)
    assert a.fused and not b.fused
    x = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    gy = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    outs = []
    for m in (a, b):
        quant._SEED[0] = 1000
        xi = x.clone().requires_grad_(True)
        y = m(xi)
        grads = torch.autograd.grad(y, [xi] + list(m.parameters()), grad_outputs=gy)
        outs.append((y, grads))
    (ya, ga), (yb, gb) = outs
    rel = lambda p, q: ((p.float() - q.float()).norm() / q.float().norm()).item()
    assert rel(ya, yb) < 5e-2                    # bf16-ulp changes of h flip some FP4 codes
    for p, q in zip(ga, gb):
        assert rel(p, q) < 0.15                  # FP4 noise of a changed operand, not an error in the recipe
    # against exact arithmetic both are equally far
    wg, wu, wd = [p.detach().float() for p in a.parameters()]
    exact = (F.silu(x.float() @ wg.t()) * (x.float() @ wu.t())) @ wd.t()
    assert abs(rel(ya, exact) - rel(yb, exact)) < 2e-2 and rel(ya, exact) < 0.3


def test_narrow_kernels_match_wide_kernels(Q):
    """Rows that are not a multiple of 16 bytes take the 4-byte kernels: same values and maxima as the
    16-byte kernels on a zero-padded copy (silu(0) * 0 = 0 adds nothing to a maximum)."""
    from nvfp4_sm120_b200 import linear
    from nvfp4_sm120_b200.swiglu import swiglu
    gen = torch.Generator(device="cuda").manual_seed(8)
    rows, cols, pad = 64, 44, 48
    signs = (torch.randint(0, 2, (16,), device="cuda", generator=gen).float() * 2 - 1)
    g = torch.zeros(rows, pad, device="cuda", dtype=torch.bfloat16)
    u = torch.zeros(rows, pad, device="cuda", dtype=torch.bfloat16)
    d = torch.zeros(rows, pad, device="cuda", dtype=torch.bfloat16)
    for t in (g, u, d):
        t[:, :cols] = torch.randn(rows, cols, device="cuda", generator=gen).to(torch.bfloat16)
    res = []
    for w in (cols, pad):
        gi = g[:, :w].contiguous().requires_grad_(True)
        ui = u[:, :w].contiguous().requires_grad_(True)
        linear._GRAD_AMAX.clear()
        h, mx = swiglu(gi, ui, signs)
        dg, du = torch.autograd.grad(h, [gi, ui], grad_outputs=d[:, :w].contiguous())
        hints = [linear._GRAD_AMAX[t.data_ptr()][1].clone() for t in (dg, du)]
        res.append((h[:, :cols], dg[:, :cols], du[:, :cols], mx, hints))
    linear._GRAD_AMAX.clear()
    (h0, dg0, du0, mx0, hint0), (h1, dg1, du1, mx1, hint1) = res
    assert torch.equal(h0, h1) and torch.equal(dg0, dg1) and torch.equal(du0, du1)
    assert torch.equal(_bits(mx0), _bits(mx1))
    assert all(torch.equal(_bits(a), _bits(b)) for a, b in zip(hint0, hint1))


@pytest.mark.parametrize("shape", [(16, 32), (512, 3072), (40, 64)])
def test_relu2_values_maxima_and_hint(Q, shape):
    from nvfp4_sm120_b200 import linear, quant
    from nvfp4_sm120_b200.swiglu import relu2
    from oracle import nvfp4_oracle as O
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(*shape, device="cuda", generator=gen).to(torch.bfloat16).requires_grad_(True)
    d = torch.randn(*shape, device="cuda", generator=gen).to(torch.bfloat16)
    signs = O.signs_from_seed(3).cuda()
    has_rht = shape[0] % 16 == 0
    linear._GRAD_AMAX.clear()
    a, mx = relu2(x, signs)
    (dx,) = torch.autograd.grad(a, [x], grad_outputs=d)
    xf = x.detach().float()
    assert torch.equal(a, (torch.relu(xf) ** 2).to(torch.bfloat16))                 # one rounding of an exact product
    assert torch.equal(dx, (2 * torch.relu(xf) * d.float()).to(torch.bfloat16))
    assert torch.equal(_bits(mx[0:1]), _bits(quant.tensor_amax(a)))
    plain, rht = linear._take_grad_amax(dx.reshape(-1, dx.shape[-1]), signs)
    assert torch.equal(_bits(plain), _bits(quant.tensor_amax(dx)))
    if has_rht:
        assert torch.equal(_bits(mx[1:2]), _bits(quant.tensor_amax(a, rht=True, signs=signs, transpose=True)))
        assert torch.equal(_bits(rht), _bits(quant.tensor_amax(dx, rht=True, signs=signs, transpose=True)))
    else:
        assert rht is None and float(mx[1]) == 0.0


def test_decoder_block_fused_activation_matches_torch_ops(Q):
    """The GPT block with the fused relu^2 against the same block with torch element-wise ops: same
    weights and stochastic-rounding seeds; relu^2 is exact in fp32, so only bf16-ulp effects remain."""
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.models import DecoderBlock, rotary_tables
    Q.set_amortize(False)
    torch.manual_seed(0)
    blk = DecoderBlock(256, 4, 4, 1024, True, "cuda")
    assert blk.fused_act
    x = torch.randn(2, 64, 256, device="cuda")
    cos, sin = rotary_tables(64, 64, "cuda")
    outs = []
    for fused in (True, False):
        blk.fused_act = fused
        quant._SEED[0] = 500
        xi = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = blk(xi, cos, sin)
        g = torch.autograd.grad(y.float().square().mean(), [xi] + list(blk.parameters()))
        outs.append((y, g))
    (ya, ga), (yb, gb) = outs
    rel = lambda p, q: ((p.float() - q.float()).norm() / (q.float().norm() + 1e-30)).item()
    assert rel(ya, yb) < 2e-2
    assert all(rel(p, q) < 0.15 for p, q in zip(ga, gb))


def test_hadamard_hint_is_dropped_for_another_sign_vector(Q):
    """A maximum taken after the Hadamard transform belongs to the sign vector it was computed with:
    a consumer that holds other signs gets the plain maximum only and recomputes the other; an equal
    vector in another buffer is accepted (compared once, then remembered)."""
    from nvfp4_sm120_b200 import linear
    from oracle import nvfp4_oracle as O
    g = torch.randn(64, 64, device="cuda").to(torch.bfloat16)
    mx = torch.tensor([1.0, 2.0], device="cuda")
    s3, s1 = O.signs_from_seed(3).cuda(), O.signs_from_seed(1).cuda()
    linear.hint_grad_amax(g, mx, True, s3)
    plain, rht = linear._take_grad_amax(g, s1)
    assert plain is not None and rht is None
    linear.hint_grad_amax(g, mx, True, s3)
    plain, rht = linear._take_grad_amax(g, s3.clone())
    assert plain is not None and rht is not None
    lin = Q.FP4Linear(64, 32)
    x = torch.randn(64, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    from nvfp4_sm120_b200 import quant
    amax = torch.stack([quant.tensor_amax(x.detach())[0], torch.zeros((), device="cuda")])      # a WRONG Hadamard maximum
    quant._SEED[0] = 77
    y1 = lin(x, amax=amax, amax_signs=s3)            # s3 is not the layer's vector: the wrong word is ignored
    y1.sum().backward()
    g1 = lin.weight.grad.clone()
    lin.weight.grad = None
    x.grad = None
    quant._SEED[0] = 77
    lin(x).sum().backward()
    assert torch.equal(lin.weight.grad, g1)


def test_packed_gate_up_kernels_match_the_split_ones(Q):
    """SwiGLU on a packed [tokens, 2H] gate|up tensor (the output of one fused projection) gives the
    bytes of the split form, forward and backward, and hints the maxima of the packed gradient."""
    from nvfp4_sm120_b200 import linear, quant
    from nvfp4_sm120_b200.swiglu import swiglu, swiglu_packed
    from oracle import nvfp4_oracle as O
    gen = torch.Generator(device="cuda").manual_seed(12)
    T, H = 256, 384
    gu = (torch.randn(T, 2 * H, device="cuda", generator=gen) * 1.5).to(torch.bfloat16).requires_grad_(True)
    dh = torch.randn(T, H, device="cuda", generator=gen).to(torch.bfloat16)
    signs = O.signs_from_seed(3).cuda()
    g = gu.detach()[:, :H].contiguous().requires_grad_(True)
    u = gu.detach()[:, H:].contiguous().requires_grad_(True)
    linear._GRAD_AMAX.clear()
    h1, m1 = swiglu(g, u, signs)
    dg, du = torch.autograd.grad(h1, [g, u], grad_outputs=dh)
    linear._GRAD_AMAX.clear()
    h2, m2 = swiglu_packed(gu, signs)
    (dgu,) = torch.autograd.grad(h2, [gu], grad_outputs=dh)
    assert torch.equal(h1, h2) and torch.equal(_bits(m1), _bits(m2))
    assert torch.equal(dgu[:, :H], dg) and torch.equal(dgu[:, H:], du)
    plain, rht = linear._take_grad_amax(dgu, signs)
    assert torch.equal(_bits(plain), _bits(quant.tensor_amax(dgu)))
    assert torch.equal(_bits(rht), _bits(quant.tensor_amax(dgu, rht=True, signs=signs, transpose=True)))


def test_ffn_with_fused_gate_up_projection(Q):
    """The FFN with gate and up as one [2h, d] projection: same initial weights as the three-linear
    form, output and gradients at the quantisation level of the exact block (the per-tensor scale of
    the fused weight spans both halves, so the bytes are not those of two separate linears)."""
    from nvfp4_sm120_b200.ffn import SwiGLUFFN
    d, h, T = 256, 512, 128
    a = SwiGLUFFN(d, h, use_fp4=True, seed=4)
    b = SwiGLUFFN(d, h, use_fp4=True, seed=4, fuse_gate_up=True)
    assert torch.equal(b.gate_up.weight[:h], a.gate.weight) and torch.equal(b.gate_up.weight[h:], a.up.weight)
    assert torch.equal(b.down.weight, a.down.weight)
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    y = b(x)
    gx, gw = torch.autograd.grad(y, [x, b.gate_up.weight], grad_outputs=gy)
    xe = x.detach().float().requires_grad_(True)
    wg, wu, wd = (t.detach().float().requires_grad_(True) for t in (a.gate.weight, a.up.weight, a.down.weight))
    ye = (F.silu(xe @ wg.t()) * (xe @ wu.t())) @ wd.t()
    ex, eg, eu = torch.autograd.grad(ye, [xe, wg, wu], grad_outputs=gy.float())
    rel = lambda p, q: ((p.float() - q).norm() / q.norm()).item()
    assert rel(y, ye) < 0.25 and rel(gx, ex) < 0.35
    assert rel(gw[:h], eg) < 0.35 and rel(gw[h:], eu) < 0.35
    assert Q.gemm_status() == 0
