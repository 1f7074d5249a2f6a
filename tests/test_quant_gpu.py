"""Parity of the CUDA quantizer (through the C ABI) with the CPU oracle and the golden vectors."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

CASES = ["a_128x256", "b_130x192", "c_48x80", "d_260x320", "e_edges_32x64", "f_zeros_16x32"]


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _cmp(q, o, what=""):
    assert torch.equal(q.qdata.cpu(), o.qdata), f"{what}: packed nibbles differ"
    assert torch.equal(q.scale.view(torch.uint8).cpu(), o.scale), f"{what}: block scales differ"
    assert torch.equal(q.per_tensor_scale.cpu().reshape(()), o.per_tensor_scale), f"{what}: pts differs"


@pytest.mark.parametrize("name", CASES)
def test_golden_rne(Q, golden, name):
    x = golden[f"{name}.x"].cuda()
    q = Q.quant_nvfp4(x)
    assert torch.equal(q.qdata.cpu(), golden[f"{name}.rne.qdata"])
    assert torch.equal(q.scale.view(torch.uint8).cpu(), golden[f"{name}.rne.scale"])
    assert torch.equal(q.per_tensor_scale.cpu(), golden[f"{name}.rne.pts"])


@pytest.mark.parametrize("name", CASES)
def test_golden_rht(Q, golden, name):
    x = golden[f"{name}.x"].cuda()
    q = Q.quant_nvfp4(x, rht=True, H=Q.hadamard16("cuda"), signs=O.signs_from_seed(3).cuda())
    assert torch.equal(q.scale.view(torch.uint8).cpu(), golden[f"{name}.rht.scale"])
    assert torch.equal(q.per_tensor_scale.cpu(), golden[f"{name}.rht.pts"])
    mism = (q.qdata.cpu() != golden[f"{name}.rht.qdata"]).float().mean().item()
    assert mism <= 1e-5          # summation order of the 16-term sums; 0 on these cases


# shapes of the reference's own byte-match sweeps (tests/cuda_val.py:12, tests/nvfp4_fused_sweep.py:22-24)
@pytest.mark.parametrize("shape", [(256, 512), (1024, 1024), (5328, 768), (2048, 2048), (333 * 16, 512),
                                   (8192, 4096)])
def test_rne_reference_sweep_shapes(Q, shape):
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(*shape, generator=g) * 3).to(torch.bfloat16)
    _cmp(Q.quant_nvfp4(x.cuda()), O.quant_nvfp4(x), str(shape))


def test_config1_operands_bit_exact(Q):
    """benchmark config 1: A 2048x4096 and B 4096x1024 (quantised as B.t()), outliers x50."""
    A = O.synthetic_tensor(2048, 4096, 0)
    B = O.synthetic_tensor(4096, 1024, 100)
    _cmp(Q.quant_nvfp4(A.cuda()), O.quant_nvfp4(A), "A")
    bt = B.t().contiguous()
    _cmp(Q.quant_nvfp4(bt.cuda()), O.quant_nvfp4(bt), "B^T")
    _cmp(Q.quant_nvfp4(B.cuda(), transpose=True), O.quant_nvfp4(bt), "B via transposing kernel")


@pytest.mark.parametrize("shape", [(256, 512), (1040, 272), (48, 80), (2048, 1024)])
@pytest.mark.parametrize("rht", [False, True])
def test_transposing_variant(Q, shape, rht):
    x = O.synthetic_tensor(shape[0], shape[1], 21)
    s = O.signs_from_seed(1)
    o = O.quant_nvfp4(x.t().contiguous(), rht=rht, signs=s, rht_impl="butterfly")
    q = Q.quant_nvfp4(x.cuda(), rht=rht, signs=s.cuda(), transpose=True)
    _cmp(q, o, f"transpose {shape} rht={rht}")


@pytest.mark.parametrize("shape", [(512, 1024), (130, 192)])
def test_rht_butterfly_bit_exact_and_matmul_close(Q, shape):
    x = O.synthetic_tensor(shape[0], shape[1], 22)
    s = O.signs_from_seed(3)
    q = Q.quant_nvfp4(x.cuda(), rht=True, signs=s.cuda())
    _cmp(q, O.quant_nvfp4(x, rht=True, signs=s, rht_impl="butterfly"), "butterfly")
    om = O.quant_nvfp4(x, rht=True, H=O.hadamard16(), signs=s)
    assert torch.equal(q.scale.view(torch.uint8).cpu(), om.scale)
    assert (q.qdata.cpu() != om.qdata).float().mean().item() <= 1e-5


def test_amax_words(Q):
    x = O.synthetic_tensor(1024, 768, 23)
    s = O.signs_from_seed(3)
    assert Q.tensor_amax(x.cuda()).item() == x.float().abs().max().item()
    want = O.rht_butterfly(x.float(), s).abs().max().item()
    assert Q.tensor_amax(x.cuda(), rht=True, signs=s.cuda()).item() == want
    want_t = O.rht_butterfly(x.t().contiguous().float(), s).abs().max().item()
    assert Q.tensor_amax(x.cuda(), rht=True, signs=s.cuda(), transpose=True).item() == want_t


def test_strided_rows_input(Q):
    big = O.synthetic_tensor(256, 1024, 24)
    view = big[:, 256:768]                       # row stride 1024, 512 columns
    _cmp(Q.quant_nvfp4(big.cuda()[:, 256:768]), O.quant_nvfp4(view.contiguous()), "strided")


@pytest.mark.parametrize("rht", [False, True])
@pytest.mark.parametrize("transpose", [False, True])
def test_sr_bit_exact_given_same_random_bits(Q, rht, transpose):
    """Stochastic rounding equals the CPU bit model of the hardware conversion fed the same
    Philox words."""
    x = O.synthetic_tensor(272, 320, 25)
    s = O.signs_from_seed(3)
    xin = x.t().contiguous() if transpose else x
    seed, off = 7, 3
    rbits = O.philox_block_bits(xin.numel() // 16, seed, off)
    o = O.quant_nvfp4(xin, stochastic=True, rht=rht, signs=s, rbits=rbits, rht_impl="butterfly")
    q = Q.quant_nvfp4(x.cuda(), stochastic=True, rht=rht, signs=s.cuda(), seed=seed,
                      transpose=transpose, philox_offset=off)
    _cmp(q, o, f"SR rht={rht} transpose={transpose}")


def test_sr_matches_reference_rule_with_transformed_uniforms(Q):
    """The hardware rule is the reference's `u < p` rule (nvfp4_validate.py:44-45) for
    u = (65535 - dither) / 65536 whenever p has at most 16 fraction bits; on real data the two
    differ only where p is cut to 16 bits: about 2^-16 of the nibbles."""
    x = O.synthetic_tensor(256, 512, 26)
    seed = 11
    rb = O.philox_block_bits(x.numel() // 16, seed, 0)                       # [nblk, 4 words]
    u = torch.from_numpy(O.cvt_rs_equivalent_uniforms(rb).reshape(x.shape))  # [nblk, 4, 4] -> [M, K]
    o = O.quant_nvfp4(x, stochastic=True, u=u)
    q = Q.quant_nvfp4(x.cuda(), stochastic=True, seed=seed)
    assert torch.equal(q.scale.view(torch.uint8).cpu(), o.scale)
    nib_q, nib_o = O.unpack_nibbles(q.qdata.cpu()), O.unpack_nibbles(o.qdata)
    assert (nib_q != nib_o).float().mean().item() < 2e-4


def test_sr_unbiased_and_seeded(Q):
    """Mean of 32 stochastic draws is closer to x than round-to-nearest (the reference's
    unbiasedness check, tests/cuda_val.py:19-26, on the quantizer alone); equal seeds repeat."""
    x = O.synthetic_tensor(512, 1024, 27, outliers=False)
    xc = x.cuda()
    def deq(q):
        return O.dequant_parts(q.qdata, q.scale.view(torch.uint8), q.per_tensor_scale, 512, 1024)
    rne = deq(Q.quant_nvfp4(xc))
    acc = torch.zeros_like(rne)
    for i in range(32):
        acc += deq(Q.quant_nvfp4(xc, stochastic=True, seed=100 + i))
    xf = x.float()
    e_rne = ((rne - xf).norm() / xf.norm()).item()
    e_sr = ((acc / 32 - xf).norm() / xf.norm()).item()
    # oracle's own reduction with the reference's software SR on the same data
    acc_o = torch.zeros_like(rne)
    g = torch.Generator().manual_seed(1)
    for i in range(32):
        acc_o += O.dequant(O.quant_nvfp4(x, stochastic=True, u=torch.rand(x.shape, generator=g)))
    e_sr_ref = ((acc_o / 32 - xf).norm() / xf.norm()).item()
    assert e_sr < e_rne
    assert e_sr <= 1.5 * e_sr_ref
    a = Q.quant_nvfp4(xc, stochastic=True, seed=5)
    b = Q.quant_nvfp4(xc, stochastic=True, seed=5)
    c = Q.quant_nvfp4(xc, stochastic=True, seed=6)
    assert torch.equal(a.qdata, b.qdata) and not torch.equal(a.qdata, c.qdata)


def test_auto_seed_counter(Q):
    """seed=None takes a module counter that advances on stochastic calls only (nvfp4_cuda.py:160-162)."""
    from nvfp4_sm120_b200 import quant
    x = O.synthetic_tensor(64, 64, 28).cuda()
    s0 = quant._SEED[0]
    Q.quant_nvfp4(x)
    assert quant._SEED[0] == s0
    a = Q.quant_nvfp4(x, stochastic=True)
    assert quant._SEED[0] == s0 + 1
    b = Q.quant_nvfp4(x, stochastic=True, seed=s0)
    assert torch.equal(a.qdata, b.qdata)


def test_argument_errors(Q):
    from nvfp4_sm120_b200 import _lib
    x = torch.zeros(16, 24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):
        Q.quant_nvfp4(x)                                   # K % 16 != 0, as nvfp4_cuda.py:164
    with pytest.raises(_lib.NVFP4Error):
        Q.quant_nvfp4(torch.zeros(16, 32, dtype=torch.bfloat16))       # CPU tensor: no CPU path
    assert _lib.lib().nvfp4_quantize_bf16(None, 16, 32, 32, 0, 0, 0, None, None, 0, 0, None, None, None, None) == -1
    with pytest.raises(ValueError):
        Q.quant_nvfp4(torch.zeros(16, 32, dtype=torch.bfloat16, device="cuda"), rht=True,
                      H=torch.eye(16, device="cuda"), signs=torch.ones(16, device="cuda"))


def test_full_size_properties(Q):
    """benchmark config 2 size (8192x4096): properties that need no CPU oracle run.  Every scale
    byte is a finite E4M3 in [2^-6, 448]; the per-tensor scale is amax / 2688; a stochastic draw
    keeps the scales and moves no nibble by more than one level."""
    x = O.synthetic_tensor(8192, 4096, 1).cuda()
    q = Q.quant_nvfp4(x)
    sc = q.scale.view(torch.uint8)
    assert int(sc.max()) <= 0x7E and int(sc.min()) >= 0x08       # 0x08 = 2^-6, 0x7E = 448
    assert q.per_tensor_scale.item() == pytest.approx(x.float().abs().max().item() / 2688.0, rel=1e-6)
    lo, hi = q.qdata & 0xF, q.qdata >> 4
    lv = torch.tensor(O.E2M1_LEVELS, device="cuda")
    assert int((lo & 7).max()) == 7 or int((hi & 7).max()) == 7   # the amax element maps to +-6
    # SR draws differ from RNE in a sizeable fraction of nibbles but never by more than one level
    qs = Q.quant_nvfp4(x, stochastic=True, seed=7)
    assert torch.equal(qs.scale.view(torch.uint8), sc)
    d = (lv[(qs.qdata & 7).long()] - lv[(q.qdata & 7).long()]).abs()
    assert float(d.max()) <= 2.0 and 0.05 < float((d > 0).float().mean()) < 0.6


@pytest.mark.parametrize("shape", [(16, 32), (130, 192), (2048, 4096), (5328, 768), (8192, 4096), (1000, 7168)])
def test_single_launch_equals_two_launch(Q, shape):
    """The persistent cooperative kernel and the amax + quantize pair give the same bytes in all
    three modes, and the cooperative kernel leaves its workspace ready for the next launch."""
    from nvfp4_sm120_b200 import quant
    x = O.synthetic_tensor(shape[0], shape[1], 31).cuda()
    s = O.signs_from_seed(3).cuda()
    for kw in (dict(), dict(stochastic=True, seed=9), dict(stochastic=True, rht=True, signs=s, seed=9),
               dict(rht=True, signs=s)):
        a = Q.quant_nvfp4(x, fused=True, **kw)
        b = Q.quant_nvfp4(x, fused=False, **kw)
        assert torch.equal(a.qdata, b.qdata), kw
        assert torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8)), kw
        assert torch.equal(a.per_tensor_scale, b.per_tensor_scale), kw
    assert quant.fused_error() == 0
    ws = quant._workspace(x.device).cpu()       # words: amax[2], arrived[2], error, launch counter, stamps
    nxt = int(ws[5].item()) & 1                   # the slot the next launch will use is clean
    assert int(ws[0 + nxt].item()) == 0 and int(ws[2 + nxt].item()) == 0 and int(ws[4].item()) == 0


def test_single_launch_strided_input(Q):
    big = O.synthetic_tensor(512, 2048, 32).cuda()
    view = big[:, 512:1536]
    a = Q.quant_nvfp4(view, fused=True)
    b = Q.quant_nvfp4(view.contiguous(), fused=False)
    assert torch.equal(a.qdata, b.qdata) and torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8))


@pytest.mark.parametrize("rht", [False, True])
def test_shard_counters_reproduce_the_whole_tensor(Q, rht):
    """A column shard quantized with the whole tensor's amax and the shard's counter pitch / base
    (nvfp4_quantize_shard_bf16) gives the bytes of the corresponding part of the unsharded
    quantization, stochastic rounding included -- row-wise and transposed."""
    x = O.synthetic_tensor(256, 512, 61).cuda()
    s = O.signs_from_seed(1).cuda()
    c0, c1 = 128, 384
    shard = x[:, c0:c1]
    # row-wise (blocks along the columns): the Hadamard runs inside a block, so shards commute with it
    full = Q.quant_nvfp4(x, stochastic=True, rht=rht, signs=s, seed=5)
    amax = Q.tensor_amax(x, rht=rht, signs=s)
    part = Q.quant_nvfp4(shard, stochastic=True, rht=rht, signs=s, seed=5, amax=amax,
                         counter=(512 // 16, c0 // 16))
    assert torch.equal(part.qdata, full.qdata[:, c0 // 2:c1 // 2])
    full_sc = O.unswizzle_scales(full.scale.view(torch.uint8).cpu(), 256, 512)
    part_sc = O.unswizzle_scales(part.scale.view(torch.uint8).cpu(), 256, c1 - c0)
    assert torch.equal(part_sc, full_sc[:, c0 // 16:c1 // 16])
    # transposed (output rows = columns of x, blocks along the rows of x)
    full_t = Q.quant_nvfp4(x, stochastic=True, rht=rht, signs=s, seed=6, transpose=True)
    amax_t = Q.tensor_amax(x, rht=rht, signs=s, transpose=True)
    part_t = Q.quant_nvfp4(shard, stochastic=True, rht=rht, signs=s, seed=6, transpose=True, amax=amax_t,
                           counter=(256 // 16, c0 * (256 // 16)))
    assert torch.equal(part_t.qdata, full_t.qdata[c0:c1])
    full_tsc = O.unswizzle_scales(full_t.scale.view(torch.uint8).cpu(), 512, 256)
    part_tsc = O.unswizzle_scales(part_t.scale.view(torch.uint8).cpu(), c1 - c0, 256)
    assert torch.equal(part_tsc, full_tsc[c0:c1])
