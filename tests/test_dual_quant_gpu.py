"""The dual-output activation quantizer (both layouts from one read) against the two separate
quantizations it replaces, bit for bit, and both against the CPU oracle."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _same(a, b):
    return (torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))
            and torch.equal(a.per_tensor_scale, b.per_tensor_scale))


@pytest.mark.parametrize("shape", [(256, 512), (48, 80), (1040, 272), (4096, 1024)])
@pytest.mark.parametrize("sr_rows,sr_cols", [(False, False), (True, True), (False, True), (True, False)])
def test_dual_equals_the_two_separate_quantizations(Q, shape, sr_rows, sr_cols):
    rows, cols = shape
    x = O.synthetic_tensor(rows, cols, 71).cuda()
    signs = O.signs_from_seed(3).cuda()
    H = Q.hadamard16("cuda")
    both = Q.tensor_amax_both(x, signs)
    assert float(both[0]) == float(Q.tensor_amax(x))
    assert float(both[1]) == float(Q.tensor_amax(x, True, signs, transpose=True))
    a_r = Q.quant_nvfp4(x, sr_rows, seed=11)
    a_c = Q.quant_nvfp4(x, sr_cols, True, H, signs, seed=12, transpose=True)
    d_r, d_c = Q.quant_dual_nvfp4(x, signs, stochastic_rows=sr_rows, stochastic_cols=sr_cols, seed_rows=11, seed_cols=12)
    assert _same(d_r, a_r) and _same(d_c, a_c)
    # maxima handed in (a fused producer knows them): same bytes
    e_r, e_c = Q.quant_dual_nvfp4(x, signs, both[0:1], both[1:2], sr_rows, sr_cols, 11, 12)
    assert _same(e_r, a_r) and _same(e_c, a_c)


def test_dual_against_the_oracle_and_seed_order(Q):
    from nvfp4_sm120_b200 import quant
    rows, cols = 272, 320
    x = O.synthetic_tensor(rows, cols, 72)
    signs = O.signs_from_seed(1)
    quant._SEED[0] = 300
    d_r, d_c = Q.quant_dual_nvfp4(x.cuda(), signs.cuda(), stochastic_rows=True, stochastic_cols=True)
    assert quant._SEED[0] == 302                       # rows drew seed 300, cols 301
    rb = O.philox_block_bits(rows * cols // 16, 300, 0)
    want_r = O.quant_nvfp4(x, stochastic=True, rbits=rb)
    rb = O.philox_block_bits(rows * cols // 16, 301, 0)
    want_c = O.quant_nvfp4(x.t().contiguous(), stochastic=True, rht=True, signs=signs, rbits=rb, rht_impl="butterfly")
    for got, want in ((d_r, want_r), (d_c, want_c)):
        assert torch.equal(got.qdata.cpu(), want.qdata)
        assert torch.equal(got.scale.view(torch.uint8).cpu(), want.scale.view(torch.uint8))
        assert float(got.per_tensor_scale) == float(want.per_tensor_scale)


def test_dual_with_shard_counters(Q):
    """A column shard of a gradient draws the bits of its place in the whole tensor in both layouts."""
    tokens, n, world = 256, 512, 2
    g = O.synthetic_tensor(tokens, n, 73).cuda()
    signs = O.signs_from_seed(1).cuda()
    H = Q.hadamard16("cuda")
    a_r = Q.quant_nvfp4(g, True, seed=21, amax=Q.tensor_amax(g))
    a_c = Q.quant_nvfp4(g, True, True, H, signs, seed=22, transpose=True, amax=Q.tensor_amax(g, True, signs, transpose=True))
    nl = n // world
    for rank in range(world):
        shard = g[:, rank * nl:(rank + 1) * nl].contiguous()
        ctr = (n // 16, rank * nl // 16, tokens // 16, rank * nl * (tokens // 16))
        d_r, d_c = Q.quant_dual_nvfp4(shard, signs, Q.tensor_amax(g), Q.tensor_amax(g, True, signs, transpose=True),
                                      True, True, 21, 22, counters=ctr)
        assert torch.equal(d_r.qdata, a_r.qdata[:, rank * nl // 2:(rank + 1) * nl // 2])
        assert torch.equal(d_c.qdata, a_c.qdata[rank * nl:(rank + 1) * nl])
