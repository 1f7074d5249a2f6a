"""The tcgen05 block-scaled GEMM against the fp32 matmul of the dequantised operands (the oracle)."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3        # target: within 1e-3 relative error of an fp32 matmul of the dequantised operands


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _ref_from_gpu_quant(qa, qb, m, n, k):
    a = O.dequant_parts(qa.qdata, qa.scale.view(torch.uint8), qa.per_tensor_scale, m, k)
    b = O.dequant_parts(qb.qdata, qb.scale.view(torch.uint8), qb.per_tensor_scale, n, k)
    return (a.double() @ b.double().t()).float()


@pytest.mark.parametrize("mnk", [(128, 256, 256), (128, 256, 1024), (256, 512, 512), (384, 768, 2048),
                                 (130, 200, 320), (48, 80, 64), (1024, 1024, 4096), (128, 256, 96)])
def test_gemm_fp32_out_matches_dequant_matmul(Q, mnk):
    m, n, k = mnk
    A = O.synthetic_tensor(m, k, 2)
    Bt = O.synthetic_tensor(n, k, 3)
    qa, qb = Q.quant_nvfp4(A.cuda()), Q.quant_nvfp4(Bt.cuda())
    got = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32).cpu()
    assert Q.gemm_status() == 0
    ref = _ref_from_gpu_quant(qa, qb, m, n, k)
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel < REL_TOL, f"{mnk}: rel {rel}"
    assert torch.allclose(got, ref, rtol=2e-3, atol=2e-3 * ref.abs().max().item())


@pytest.mark.parametrize("mode", [2])
@pytest.mark.parametrize("mnk", [(256, 512, 512), (130, 200, 320), (384, 768, 2048), (48, 80, 64), (1024, 1024, 4096)])
def test_two_cta_kernel_matches(Q, mnk, mode):
    """The persistent cta_group::2 kernel (mode 2) gives the one-CTA kernel's result and meets the
    tolerance, in fp32 and in bf16."""
    from nvfp4_sm120_b200 import _lib
    m, n, k = mnk
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 12).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 13).cuda())
    try:
        _lib.lib().nvfp4_gemm_set_mode(1)
        one = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32).cpu()
        one_bf = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16).cpu()
        _lib.lib().nvfp4_gemm_set_mode(mode)
        two = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32).cpu()
        two_bf = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16).cpu()
    finally:
        _lib.lib().nvfp4_gemm_set_mode(0)
    assert Q.gemm_status() == 0
    ref = _ref_from_gpu_quant(qa, qb, m, n, k)
    assert ((two - ref).norm() / ref.norm()).item() < REL_TOL
    assert torch.allclose(one, two, rtol=1e-5, atol=1e-5 * ref.abs().max().item())
    assert torch.equal(two_bf, two.to(torch.bfloat16))              # same accumulation, rounded once
    # the one-CTA fp32 result may come from the split-K path (another summation order): one bf16 ulp
    assert torch.allclose(one_bf.float(), one, rtol=2.0 ** -7, atol=1e-5 * ref.abs().max().item())


@pytest.mark.parametrize("mode", [1, 2])
def test_many_tiles_per_cluster_and_strided_output(Q, mode):
    """More tiles than SM pairs (the persistent kernel loops), ragged M and N, and an output whose
    row pitch is larger than N (TMA-store epilogue with a pitch) or not a multiple of 16 bytes
    (direct stores)."""
    from nvfp4_sm120_b200 import _lib
    m, n, k = 2500, 2100, 512
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 21).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 22).cuda())
    ref = _ref_from_gpu_quant(qa, qb, m, n, k)
    try:
        _lib.lib().nvfp4_gemm_set_mode(mode)
        for dtype in (torch.float32, torch.bfloat16):
            for pitch in (n, n + 8, n + 3):
                buf = torch.full((m, pitch), 7.0, device="cuda", dtype=dtype)
                Q.nvfp4_mm(qa, qb.t(), out=buf[:, :n])
                got = buf[:, :n].float().cpu()
                tol = REL_TOL if dtype == torch.float32 else 4e-3
                assert ((got - ref).norm() / ref.norm()).item() < tol, (mode, dtype, pitch)
                if pitch > n:
                    assert bool((buf[:, n:] == 7.0).all()), "wrote past column N"
    finally:
        _lib.lib().nvfp4_gemm_set_mode(0)
    assert Q.gemm_status() == 0


@pytest.mark.parametrize("mnk", [(256, 256, 8192), (640, 512, 16384), (768, 3072, 4096)])
def test_split_k_small_output(Q, mnk):
    """Weight-gradient shapes (small fp32 output, long K): K is split over several CTAs per tile that
    add into the zeroed output; same tolerance, and the bf16 path (never split) agrees."""
    m, n, k = mnk
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 14).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 15).cuda())
    out = torch.full((m, n), 7.0, device="cuda")                 # stale contents must not leak in
    got = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32, out=out).cpu()
    assert Q.gemm_status() == 0
    ref = _ref_from_gpu_quant(qa, qb, m, n, k)
    assert ((got - ref).norm() / ref.norm()).item() < REL_TOL
    bf = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16).float().cpu()
    assert ((bf - ref).norm() / ref.norm()).item() < 5e-3


def test_gemm_bf16_out_is_rounded_fp32(Q):
    m, n, k = 256, 512, 1024
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 4).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 5).cuda())
    f32 = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32)
    bf = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16)
    assert torch.equal(bf, f32.to(torch.bfloat16))


def test_config1_end_to_end(Q):
    """benchmark config 1 through fp4_matmul: A 2048x4096, B 4096x1024 (outliers x50)."""
    A = O.synthetic_tensor(2048, 4096, 0)
    B = O.synthetic_tensor(4096, 1024, 100)
    got = Q.fp4_matmul(A.cuda(), B.cuda(), out_dtype=torch.float32).cpu()
    ref = O.fp4_matmul_ref(A, B)
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel < REL_TOL
    exact = A.float() @ B.float()
    q_err = ((got - exact).norm() / exact.norm()).item()
    assert 0.05 < q_err < 0.2          # the quantisation error itself (~0.1 on this input)


def test_fp4_matmul_rhs_layouts_and_preq(Q):
    """B given row-major [K, N] or as the .t() view of [N, K] gives the same bytes; fp4_mm_preqB with
    a cached quant(B.t()) equals fp4_matmul (nvfp4_cuda.py:196-200)."""
    A = O.synthetic_tensor(256, 512, 6).cuda()
    W = O.synthetic_tensor(768, 512, 7).cuda()          # [N, K]
    y1 = Q.fp4_matmul(A, W.t())
    y2 = Q.fp4_matmul(A, W.t().contiguous())
    assert torch.equal(y1, y2)
    wq = Q.quant_nvfp4(W)
    assert torch.equal(Q.fp4_mm_preqB(A, wq), y1)


def test_gemm_rht_cancels(Q):
    """The same random-sign Hadamard on both operands cancels in the product (nvfp4_train.py:53-54):
    the error stays at the quantisation level."""
    A = O.synthetic_tensor(512, 1024, 8, outliers=False).cuda()
    B = O.synthetic_tensor(1024, 256, 9, outliers=False).cuda()
    s = O.signs_from_seed(1).cuda()
    ref = A.float() @ B.float()
    plain = Q.fp4_matmul(A, B, out_dtype=torch.float32)
    rht = Q.fp4_matmul(A, B, rht=True, H=Q.hadamard16("cuda"), signs=s, out_dtype=torch.float32)
    e0 = ((plain - ref).norm() / ref.norm()).item()
    e1 = ((rht - ref).norm() / ref.norm()).item()
    assert e1 < 1.3 * e0 and e0 < 0.2


def test_gemm_sr_unbiased(Q):
    """tests/cuda_val.py:19-26: the mean of 32 stochastic products is closer to the exact product
    than the round-to-nearest one."""
    m, k, n = 512, 512, 512
    g = torch.Generator().manual_seed(0)
    A = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(k, n, generator=g).to(torch.bfloat16).cuda()
    ref = A.float() @ B.float()
    rne = ((Q.fp4_matmul(A, B, out_dtype=torch.float32) - ref).norm() / ref.norm()).item()
    acc = torch.zeros_like(ref)
    for i in range(32):
        acc += Q.fp4_matmul(A, B, sr_a=True, sr_b=True, seed=100 + i, out_dtype=torch.float32)
    sr = ((acc / 32 - ref).norm() / ref.norm()).item()
    assert sr < rne
    assert 0.08 < rne < 0.2


def test_gemm_argument_errors(Q):
    from nvfp4_sm120_b200 import _lib
    qa = Q.quant_nvfp4(torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda"))
    qb = Q.quant_nvfp4(torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        Q.nvfp4_mm(qa, qb.t())                       # contraction mismatch
    with pytest.raises(ValueError):
        Q.nvfp4_mm(qa, qa)                           # right operand must be the .t() view
    assert _lib.lib().nvfp4_gemm(None, None, None, None, None, None, None, 0, 1, 1, 32, 1, None, None) == -1


def test_standalone_c_driver_verifies():
    """The C driver (no Python, no torch above the ABI) quantizes, multiplies and verifies on the host,
    like the reference's CUTLASS executables (`--m --n --k --iterations --verify`, "Disposition: Passed")."""
    import os
    import subprocess
    cli = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nvfp4_sm120_b200", "nvfp4_gemm_cli")
    assert os.path.exists(cli), "build with `python -m nvfp4_sm120_b200.build`"
    for args in (["--m", "256", "--n", "512", "--k", "512"], ["--m", "1000", "--n", "776", "--k", "2048"]):
        res = subprocess.run([cli] + args + ["--iterations", "3", "--verify"], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "Disposition: Passed" in res.stdout


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("mnk", [(256, 512, 512), (130, 208, 320), (1024, 768, 2048)])
def test_fp4_output_epilogue_equals_quantizing_the_bf16_output(Q, mnk, mode):
    """The NVFP4-output epilogue (for chained GEMMs; the reference's CUTLASS example has the same
    E2M1 + scale-factor output, cutlass_gemm/nvfp4_gemm.cu:106-108) gives, bit for bit, the quantizer's
    result on the bf16 output with the same per-tensor maximum -- exact, a generous bound, or one that
    is too small (saturation)."""
    from nvfp4_sm120_b200 import _lib, quant
    m, n, k = mnk
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 31).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 32).cuda())
    try:
        _lib.lib().nvfp4_gemm_set_mode(mode)
        y = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16)
        exact = quant.tensor_amax(y)
        for factor in (1.0, 1.5, 0.25):
            amax = exact * factor
            got = Q.nvfp4_mm_fp4out(qa, qb.t(), amax)
            want = Q.quant_nvfp4(y, amax=amax)
            assert torch.equal(got.qdata, want.qdata), (mnk, mode, factor)
            assert torch.equal(got.scale.view(torch.uint8), want.scale.view(torch.uint8)), (mnk, mode, factor)
            assert torch.equal(got.per_tensor_scale, want.per_tensor_scale)
    finally:
        _lib.lib().nvfp4_gemm_set_mode(0)
    assert Q.gemm_status() == 0
    # and the quantized output feeds the next GEMM directly (whose contraction dim N must be a multiple of 32)
    if n % 32 == 0:
        w2 = Q.quant_nvfp4(O.synthetic_tensor(64, n, 33).cuda())
        z = Q.nvfp4_mm(got, w2.t(), out_dtype=torch.float32)
        z_ref = Q.nvfp4_mm(Q.quant_nvfp4(y, amax=amax), w2.t(), out_dtype=torch.float32)
        assert torch.equal(z, z_ref)


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("shape,dtype", [((512, 768, 512), torch.bfloat16), ((300, 200, 256), torch.bfloat16),
                                         ((130, 1000, 128), torch.float32), ((128, 264, 2048), torch.float32),
                                         ((100, 90, 64), torch.bfloat16)])
def test_epilogue_amax_equals_a_pass_over_the_output(Q, mode, shape, dtype):
    """nvfp4_gemm_amax: the word the epilogue leaves is max|D| of the stored output, bit for bit what a
    reduction over D finds (whole tiles, clipped tiles, a row pitch that rules the TMA store out, both
    output types and both kernels), and quantizing D with it equals the two-pass quantization."""
    from nvfp4_sm120_b200 import _lib
    from nvfp4_sm120_b200.gemm import nvfp4_mm
    m, n, k = shape
    qa = Q.quant_nvfp4(O.synthetic_tensor(m, k, 61).cuda())
    qb = Q.quant_nvfp4(O.synthetic_tensor(n, k, 62).cuda())
    word = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")   # the call zeroes it first
    try:
        _lib.lib().nvfp4_gemm_set_mode(mode)
        d = nvfp4_mm(qa, qb.t(), dtype, amax_out=word)
        plain = nvfp4_mm(qa, qb.t(), dtype)
    finally:
        _lib.lib().nvfp4_gemm_set_mode(0)
    if dtype == torch.float32 and k >= 2048 and mode != 2:
        # the plain call splits K over CTAs here (partial sums added by atomics); this one does not
        assert ((d - plain).norm() / plain.norm()).item() < 1e-5
    else:
        assert torch.equal(d, plain)
    assert float(word) == float(d.abs().max().float()) and float(word) > 0
    if dtype == torch.bfloat16 and n % 16 == 0:
        q1, q2 = Q.quant_nvfp4(d, amax=word), Q.quant_nvfp4(d)
        assert torch.equal(q1.qdata, q2.qdata) and torch.equal(q1.scale.view(torch.uint8), q2.scale.view(torch.uint8))
        assert torch.equal(q1.per_tensor_scale, q2.per_tensor_scale)
    assert Q.gemm_status() == 0
