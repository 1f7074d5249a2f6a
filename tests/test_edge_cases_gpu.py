"""Edge cases of the path on the GPU: degenerate and ragged shapes, extreme values, repeated use."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _same(q, o):
    return (torch.equal(q.qdata.cpu(), o.qdata) and torch.equal(q.scale.view(torch.uint8).cpu(), o.scale)
            and torch.equal(q.per_tensor_scale.cpu().reshape(()), o.per_tensor_scale))


def test_empty_and_bad_shapes_are_rejected(Q):
    from nvfp4_sm120_b200 import _lib
    with pytest.raises(_lib.NVFP4Error):
        Q.quant_nvfp4(torch.zeros(0, 32, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(AssertionError):
        Q.quant_nvfp4(torch.zeros(16, 8, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        Q.quant_nvfp4(torch.zeros(4, 16, 32, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("shape", [(1, 16), (1, 4096), (3, 48), (127, 16), (129, 80), (4097, 32)])
def test_tiny_and_ragged_shapes(Q, shape):
    x = O.synthetic_tensor(shape[0], shape[1], 41, outliers=False)
    s = O.signs_from_seed(3)
    assert _same(Q.quant_nvfp4(x.cuda()), O.quant_nvfp4(x))
    assert _same(Q.quant_nvfp4(x.cuda(), rht=True, signs=s.cuda()), O.quant_nvfp4(x, rht=True, signs=s, rht_impl="butterfly"))


def test_extreme_values(Q):
    """Largest finite bf16, tiny values, one huge outlier among zeros, all-equal blocks, negative zero."""
    big = torch.finfo(torch.bfloat16).max
    rows = [torch.full((64,), big), torch.full((64,), 1e-30), torch.zeros(64), -torch.zeros(64),
            torch.full((64,), -3.0), torch.linspace(-1e38, 1e38, 64)]
    x = torch.stack(rows).to(torch.bfloat16)
    x[2, 7] = 1.0
    assert _same(Q.quant_nvfp4(x.cuda()), O.quant_nvfp4(x))
    small = (torch.randn(32, 64) * 1e-20).to(torch.bfloat16)
    assert _same(Q.quant_nvfp4(small.cuda()), O.quant_nvfp4(small))
    z = torch.zeros(16, 32, dtype=torch.bfloat16)
    q = Q.quant_nvfp4(z.cuda(), rht=True, signs=-torch.ones(16, device="cuda"))
    assert int(q.qdata.max()) == 0                     # an all-zero block stays +0 under sign flips


def test_fp32_and_noncontiguous_inputs(Q):
    x = torch.randn(96, 256)
    assert _same(Q.quant_nvfp4(x.cuda()), O.quant_nvfp4(x.to(torch.bfloat16)))
    xt = O.synthetic_tensor(256, 96, 42)
    got = Q.quant_nvfp4(xt.cuda().t())                 # a transposed view: made contiguous internally
    assert _same(got, O.quant_nvfp4(xt.t().contiguous()))


def test_many_calls_reuse_workspace_without_leaking_state(Q):
    from nvfp4_sm120_b200 import quant
    xs = [O.synthetic_tensor(64 * (i + 1), 128, 50 + i) for i in range(6)]
    for rep in range(3):
        for x in xs:
            assert _same(Q.quant_nvfp4(x.cuda()), O.quant_nvfp4(x))
    # a large maximum followed by small ones, on grids of different sizes: a barrier slot that was not
    # cleared would carry the old maximum (or an old arrival count) into the next launch
    g = torch.Generator().manual_seed(77)
    big = (torch.randn(2048, 1024, generator=g) * 1000).to(torch.bfloat16)
    small = (torch.randn(48, 64, generator=g) * 1e-3).to(torch.bfloat16)
    mid = torch.randn(700, 512, generator=g).to(torch.bfloat16)
    want = {id(t): O.quant_nvfp4(t) for t in (big, small, mid)}
    for t in (big, small, small, mid, big, small, mid, mid, small):
        assert _same(Q.quant_nvfp4(t.cuda()), want[id(t)])
    assert quant.fused_error() == 0


def test_full_size_round_trip_properties(Q):
    """benchmark config 2 size without a CPU oracle run: dequantised values stay within half a grid
    step of the input (scaled), and quantising twice gives the same bytes (determinism)."""
    x = O.synthetic_tensor(8192, 4096, 1).cuda()
    a, b = Q.quant_nvfp4(x), Q.quant_nvfp4(x)
    assert torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))
    lv = torch.tensor(O.E2M1_LEVELS, device="cuda")
    rows = slice(0, 512)
    codes = torch.stack([a.qdata[rows] & 0xF, a.qdata[rows] >> 4], dim=-1).reshape(512, 4096)
    vals = lv[(codes & 7).long()] * torch.where((codes & 8) != 0, -1.0, 1.0)
    sc = O.unswizzle_scales(a.scale.view(torch.uint8).cpu(), 8192, 4096)[rows].view(torch.float8_e4m3fn).float().cuda()
    deq = (vals.reshape(512, 256, 16) * sc.unsqueeze(-1)).reshape(512, 4096) * a.per_tensor_scale
    err = (deq - x[rows].float()).abs()
    step = sc.repeat_interleave(16, dim=1) * a.per_tensor_scale          # grid spacing is <= 2 scale units
    assert bool((err <= step * 1.0001 + 1e-30).all())
