"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py), and against torch's internal FP4 helpers."""
import sys
import types

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

CASES = ["a_128x256", "b_130x192", "c_48x80", "d_260x320", "e_edges_32x64", "f_zeros_16x32"]


def test_hadamard_and_signs(golden):
    assert torch.equal(O.hadamard16(), golden["hadamard16"])
    assert torch.equal(O.signs_from_seed(1), golden["signs_seed1"])
    assert torch.equal(O.signs_from_seed(3), golden["signs_seed3"])
    # the sign vector every FP4Linear carries (nvfp4_train.py:64-66)
    assert O.signs_from_seed(1).tolist() == [1, 1, -1, -1, 1, 1, 1, 1, 1, -1, -1, 1, -1, 1, 1, -1]


@pytest.mark.parametrize("name", CASES)
def test_rne_bit_exact(golden, name):
    x = golden[f"{name}.x"]
    q = O.quant_nvfp4(x)
    assert torch.equal(q.qdata, golden[f"{name}.rne.qdata"])
    assert torch.equal(q.scale, golden[f"{name}.rne.scale"])
    assert torch.equal(q.per_tensor_scale, golden[f"{name}.rne.pts"])


@pytest.mark.parametrize("name", CASES)
def test_rht_bit_exact(golden, name):
    x = golden[f"{name}.x"]
    H, s = O.hadamard16(), O.signs_from_seed(3)
    q = O.quant_nvfp4(x, rht=True, H=H, signs=s)
    assert torch.equal(q.qdata, golden[f"{name}.rht.qdata"])
    assert torch.equal(q.scale, golden[f"{name}.rht.scale"])
    assert torch.equal(q.per_tensor_scale, golden[f"{name}.rht.pts"])


@pytest.mark.parametrize("name", CASES)
def test_rht_butterfly_matches_matmul(golden, name):
    """The kernel's summation order gives the same bytes as the reference's matmul."""
    x = golden[f"{name}.x"]
    q = O.quant_nvfp4(x, rht=True, signs=O.signs_from_seed(3), rht_impl="butterfly")
    assert torch.equal(q.scale, golden[f"{name}.rht.scale"])
    mism = (q.qdata != golden[f"{name}.rht.qdata"]).float().mean().item()
    assert mism <= 1e-5


@pytest.mark.parametrize("name", ["a_128x256", "b_130x192"])
def test_sr_with_known_uniforms(golden, name):
    x, u = golden[f"{name}.x"], golden[f"{name}.u"]
    q = O.quant_nvfp4(x, stochastic=True, u=u)
    assert torch.equal(q.qdata, golden[f"{name}.sr.qdata"])
    assert torch.equal(q.scale, golden[f"{name}.sr.scale"])
    qr = O.quant_nvfp4(x, stochastic=True, rht=True, H=O.hadamard16(), signs=O.signs_from_seed(1), u=u)
    assert torch.equal(qr.qdata, golden[f"{name}.rht_sr.qdata"])
    assert torch.equal(qr.scale, golden[f"{name}.rht_sr.scale"])


def test_round_e2m1_reference(golden):
    g, u = golden["round.grid"], golden["round.u"]
    assert torch.equal(O.round_e2m1_reference(g, True, u), golden["round.sr"])
    assert torch.equal(O.round_e2m1_reference(g, False), golden["round.rn"])


def test_dequant_equals_simulator_off_ties(golden):
    """dequant(quant(x)) equals the simulator's fake-quant (nvfp4_validate.py:51-65)
    except where the scaled value is a tie or within an ulp of one (the simulator
    rounds ties down and divides where the real path multiplies by a reciprocal)."""
    x = golden["a_128x256.x"]
    q = O.quant_nvfp4(x, keep_scaled=True)
    dq = O.dequant(q)
    sim = golden["a_128x256.sim1d"]
    m = q.scaled.abs()
    tie = torch.zeros_like(m, dtype=torch.bool)
    for t in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        tie |= (m - t).abs() <= 4e-7 * t      # x*recip vs x/deq differ by an ulp near a tie
    assert torch.allclose(dq[~tie], sim[~tie], rtol=1e-6, atol=0)
    assert tie.float().mean() < 0.01


def test_rht_apply(golden):
    x = golden["a_128x256.x"].float()
    got = O.rht_matmul(x, O.hadamard16(), O.signs_from_seed(1))
    assert torch.equal(got, golden["a_128x256.rht_apply"])
    assert torch.allclose(O.rht_butterfly(x, O.signs_from_seed(1)), got, rtol=0, atol=1e-5)


def test_against_torch_internal_helpers():
    """E2M1 encode, nibble packing and scale swizzle against the twins torch ships."""
    sys.modules.setdefault("expecttest", types.ModuleType("expecttest"))
    if not hasattr(sys.modules["expecttest"], "TestCase"):
        sys.modules["expecttest"].TestCase = object
    cq = pytest.importorskip("torch.testing._internal.common_quantized")
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(4096, generator=g) * 3,
                   torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, 0.0, 7.0, -9.0, 1e-9, -1e-9])])
    x = torch.cat([x, -x])
    assert torch.equal(O.e2m1_encode_rne(x), cq._f32_to_floatx_unpacked(x, 2, 1))
    codes = O.e2m1_encode_rne(x[:4096].reshape(64, 64))
    assert torch.equal(O.pack_nibbles(codes), cq.pack_uint4(codes))
    assert torch.equal(O.unpack_nibbles(O.pack_nibbles(codes)), codes)
    assert torch.equal(O.e2m1_decode(codes), cq._floatx_unpacked_to_f32(codes, 2, 1))
    for (m, c) in [(128, 4), (130, 12), (48, 5), (300, 9)]:
        s = torch.randint(0, 255, (m, c), dtype=torch.uint8, generator=g)
        sw = O.swizzle_scales(s)
        assert torch.equal(sw.flatten(), cq.to_blocked(s).flatten())
        assert torch.equal(O.unswizzle_scales(sw, m, c * 16), s)
        for (r, cc) in [(0, 0), (m - 1, c - 1), (m // 2, c // 2), (33, 1)]:
            assert sw.flatten()[O.swizzled_scale_offset(r, cc, c * 16)] == s[r, cc]


def test_fp32_division_is_ieee():
    """The oracle's divisions are true fp32 divisions (what the CUDA kernel does
    with `/`), not reciprocal multiplies."""
    g = torch.Generator().manual_seed(3)
    a = torch.rand(100000, generator=g) * 100
    b = torch.rand((), generator=g) + 0.01
    want = torch.from_numpy(a.numpy() / np.float32(b.item()))
    assert torch.equal(a / b, want)
    assert torch.equal(a / 6.0, torch.from_numpy(a.numpy() / np.float32(6.0)))
    assert torch.equal(a / 2688.0, torch.from_numpy(a.numpy() / np.float32(2688.0)))
    assert torch.equal(1.0 / a, torch.from_numpy(np.float32(1.0) / a.numpy()))


def test_philox_known_answers():
    """Philox4x32-10 known-answer vectors (Random123 kat_vectors)."""
    z = np.zeros((1, 4), dtype=np.uint32)
    out = O.philox4x32_10(z, np.zeros(2, dtype=np.uint32))[0]
    assert [hex(v) for v in out] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    f = np.full((1, 4), 0xFFFFFFFF, dtype=np.uint32)
    out = O.philox4x32_10(f, np.full(2, 0xFFFFFFFF, dtype=np.uint32))[0]
    assert [hex(v) for v in out] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    c = np.array([[0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344]], dtype=np.uint32)
    out = O.philox4x32_10(c, np.array([0xA4093822, 0x299F31D0], dtype=np.uint32))[0]
    assert [hex(v) for v in out] == ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]


def test_config1_tolerance_statement():
    """benchmark config 1 on a slice: RNE quantise -> dequantise, fp32 matmul; the
    error against the unquantised product is the ~0.1 the reference reports."""
    A = O.synthetic_tensor(256, 512, 0)
    B = O.synthetic_tensor(512, 128, 1)
    ref = A.float() @ B.float()
    got = O.fp4_matmul_ref(A, B)
    rel = ((got - ref).norm() / ref.norm()).item()
    assert 0.05 < rel < 0.2


def test_cvt_rs_bit_model_against_recorded_hardware():
    """The CPU bit model of cvt.rs.satfinite.e2m1x4.f32 reproduces conversions recorded on a
    B200 (tests/golden/cvt_rs_probe.cu made them)."""
    import os
    d = np.load(os.path.join(os.path.dirname(__file__), "golden", "cvt_rs_hw_samples.npz"))
    x, rbits, out = d["x"], d["rbits"], d["out"].astype(np.int64)
    # the probe passes x[:, p] as the p-th source operand, which lands in nibble 3 - p
    got = O.cvt_rs_e2m1x4(x[:, ::-1], rbits).astype(np.int64)
    packed = got[:, 0] | (got[:, 1] << 4) | (got[:, 2] << 8) | (got[:, 3] << 12)
    assert np.array_equal(packed, out)
    assert out[0] == 0x1246          # sources (0.5, 1, 2, 4): first source in the highest nibble


def test_cvt_rs_model_matches_reference_rule():
    """With u = (65535 - dither) / 65536 the reference's `u < p` rule and the hardware model
    agree on values whose step fraction has at most 16 bits."""
    rng = np.random.default_rng(1)
    lv = np.array(O.E2M1_LEVELS, dtype=np.float32)
    iv = rng.integers(0, 7, size=(4096, 4))
    frac = rng.integers(0, 65536, size=(4096, 4)).astype(np.float64) / 65536.0
    x = (lv[iv] + (lv[iv + 1] - lv[iv]) * frac).astype(np.float32)
    x *= rng.choice([-1.0, 1.0], size=x.shape).astype(np.float32)
    rbits = rng.integers(0, 2 ** 32, size=4096, dtype=np.uint64).astype(np.uint32)
    hw = O.cvt_rs_e2m1x4(x, rbits)
    u = torch.from_numpy(O.cvt_rs_equivalent_uniforms(rbits))
    ref = O.e2m1_encode_rne(O.round_e2m1_reference(torch.from_numpy(x), True, u)).numpy()
    assert np.array_equal(hw, ref)


# ---------------------------------------------------------------------------------------------
# the reference's training recipe as a simulator (oracle/nvfp4_sim.py) against the reference's own
# quantize_nvfp4_1d / quantize_nvfp4_2d / apply_rht_lastdim / _NVFP4LinearFn
# ---------------------------------------------------------------------------------------------
def test_simulator_quantizers_match_reference(golden):
    from oracle import nvfp4_sim as S
    x = golden["a_128x256.x"].float()
    assert torch.equal(S.quantize_1d(x), golden["a_128x256.sim1d"])
    assert torch.equal(S.rht_lastdim(x, S.hadamard16("cpu"), O.signs_from_seed(1)), golden["a_128x256.rht_apply"])
    w2d = S.quantize_2d(golden["sim.w"])
    assert torch.equal(w2d, golden["sim.w2d"])
    # the point of the 16x16 scaling: the transposed weight quantizes to the transposed values
    assert torch.equal(S.quantize_2d(golden["sim.w"].t().contiguous()), w2d.t())
    grid, u = golden["round.grid"], golden["round.u"]
    assert torch.equal(S.snap_e2m1(grid, True, u), golden["round.sr"])
    assert torch.equal(S.snap_e2m1(grid, False), golden["round.rn"])


def test_simulator_linear_forward_backward_match_reference(golden, monkeypatch):
    """One forward + backward of the recipe (x 1-D RNE, w 2-D RNE, dY stochastic, wgrad through the
    Hadamard with 40 tokens padded to 48), fed the uniforms the reference run was fed."""
    from oracle import nvfp4_sim as S
    pool = {(40, 3, 16): golden["sim.u_dgrad"].reshape(40, 3, 16), (48, 3, 16): golden["sim.u_wgrad"].reshape(48, 3, 16)}
    monkeypatch.setattr(torch, "rand_like", lambda m: pool[tuple(m.shape)])
    x = golden["sim.x"].clone().requires_grad_(True)
    w = golden["sim.w"].clone().requires_grad_(True)
    y = S.SimLinearFn.apply(x, w, True, True, S.hadamard16("cpu"), O.signs_from_seed(1))
    y.backward(golden["sim.gy"])
    assert torch.equal(y.detach(), golden["sim.y"])
    assert torch.equal(x.grad, golden["sim.dx"])
    assert torch.equal(w.grad, golden["sim.dw"])


def test_simulator_tracks_the_real_fp4_recipe():
    """The simulator and the real-FP4 oracle describe the same quantizer up to their documented
    differences (tie direction, 2^-6 scale clamp): off ties their dequantised values agree to the
    last bit or two of the product of the two scales."""
    from oracle import nvfp4_sim as S
    x = O.synthetic_tensor(64, 256, 77, outliers=False).float()
    sim = S.quantize_1d(x)
    real = O.dequant(O.quant_nvfp4(x.to(torch.bfloat16)))
    assert (~torch.isclose(sim, real, rtol=1e-6, atol=0)).float().mean().item() < 5e-3


def test_weight_2d_scaling_oracle(golden):
    """The real-NVFP4 form of the simulator's 16 x 16 weight scaling: both layouts dequantize to the
    same matrix, which equals the simulator's fake-quant off ties (tie direction and the scale clamp
    are the documented differences)."""
    from oracle import nvfp4_sim as S
    w = golden["sim.w"]
    qr, qc = O.quant_nvfp4_weight_2d(w)
    assert torch.equal(O.dequant(qr), O.dequant(qc).t())
    sim = golden["sim.w2d"]
    assert (~torch.isclose(O.dequant(qr), sim, rtol=1e-6, atol=0)).float().mean().item() < 5e-3
    # a tile's sixteen row blocks carry the same scale byte
    assert torch.equal(qr.scale_rowmajor.reshape(3, 16, 4)[:, 0], qr.scale_rowmajor.reshape(3, 16, 4)[:, 15])
