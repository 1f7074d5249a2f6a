"""Parity at the sizes the benchmark numbers are quoted on.

* config 2 (bf16 8192 x 4096, seed 1, x50 outliers): the three quantizer modes bit for bit against
  the CPU oracle (round to nearest; stochastic rounding with Philox seed 7; Hadamard with sign seed 3
  + stochastic rounding), the relation of the reference's tests/cuda_val.py:9-16 at full size.
* config 3 (4096^3, 8192^3, 16384^3 and both readings of 16384 x 4096 x 14336): the GEMM with its
  automatic kernel choice against an fp64 matmul of the dequantised operands, on sampled output rows
  over all columns (first and last tile row, rasterization-group boundaries, the last cluster's
  tiles) and, for every tile at once, through the column sums of the whole output; the bf16 output
  must be the bf16 rounding of the fp32 one.  Relation of cutlass_gemm/nvfp4_gemm_bf16out.cu:396-421
  (host verification of the block-scaled product).
The operands are dequantised on the GPU with torch ops that restate the oracle's dequant_parts."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


@pytest.fixture(scope="module")
def Q():
    import nvfp4_sm120_b200 as pkg
    return pkg


def _eq(q, o, what):
    assert torch.equal(q.qdata.cpu(), o.qdata), f"{what}: packed nibbles differ"
    assert torch.equal(q.scale.view(torch.uint8).cpu(), o.scale), f"{what}: block scales differ"
    assert torch.equal(q.per_tensor_scale.cpu().reshape(()), o.per_tensor_scale), f"{what}: pts differs"


def test_config2_tensor_three_modes_bit_exact(Q):
    from nvfp4_sm120_b200 import quant
    x = O.synthetic_tensor(8192, 4096, 1)
    xc = x.cuda()
    signs = O.signs_from_seed(3)
    rb = O.philox_block_bits(x.numel() // 16, 7, 0)
    _eq(Q.quant_nvfp4(xc), O.quant_nvfp4(x), "RNE")
    _eq(Q.quant_nvfp4(xc, stochastic=True, seed=7), O.quant_nvfp4(x, stochastic=True, rbits=rb), "SR seed 7")
    _eq(Q.quant_nvfp4(xc, stochastic=True, rht=True, signs=signs.cuda(), seed=7),
        O.quant_nvfp4(x, stochastic=True, rht=True, signs=signs, rbits=rb, rht_impl="butterfly"), "RHT+SR")
    assert quant.fused_error() == 0


# ---------------------------------------------------------------------------------------------
def dequant_rows_gpu(q, rows=None):
    """fp64 [n, K] values of the given rows (all when None) of a row-major NVFP4Tensor on the GPU:
    code value x E4M3 block scale x per-tensor scale (oracle.dequant_parts with torch CUDA ops)."""
    m, k2 = q.qdata.shape
    k = 2 * k2
    dev = q.qdata.device
    if rows is None:
        rows = torch.arange(m, device=dev)
    qd = q.qdata[rows]
    codes = torch.stack([qd & 0xF, qd >> 4], dim=-1).reshape(len(rows), k).long()
    lv = torch.tensor(O.E2M1_LEVELS, dtype=torch.float64, device=dev)
    vals = lv[codes & 7] * (1.0 - 2.0 * (codes >> 3).double())
    c = torch.arange(k // 16, device=dev)
    col_tiles = (k // 16 + 3) // 4
    r = rows[:, None]
    off = ((r // 128) * col_tiles + c[None, :] // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c[None, :] % 4
    sc = q.scale.view(torch.uint8).reshape(-1)[off].view(torch.float8_e4m3fn).double()
    return (vals.reshape(len(rows), k // 16, 16) * sc[..., None]).reshape(len(rows), k) * q.per_tensor_scale.double()


def _sample_rows(m, n_rand=40, seed=0):
    fixed = [0, 1, 127, 128, 255, 256, 257, 511, m // 2 - 1, m // 2, m - 256, m - 129, m - 128, m - 1]
    fixed += [r for r in (4095, 4096, 8191, 8192, 12287, 12288) if r < m]      # 16-pair raster groups
    g = torch.Generator().manual_seed(seed)
    rnd = torch.randint(0, m, (n_rand,), generator=g).tolist()
    return torch.tensor(sorted(set(fixed + rnd)), dtype=torch.long)


SHAPES = [(4096, 4096, 4096), (8192, 8192, 8192), (16384, 4096, 14336), (16384, 14336, 4096), (16384, 16384, 16384)]


@pytest.mark.parametrize("mnk", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_config3_shapes_against_fp64_dequant_matmul(Q, mnk):
    m, n, k = mnk
    gen = torch.Generator(device="cuda").manual_seed(2)
    A = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, generator=gen)
    Bt = torch.randn(n, k, device="cuda", dtype=torch.bfloat16, generator=gen)
    qa, qb = Q.quant_nvfp4(A), Q.quant_nvfp4(Bt)
    del A, Bt
    d32 = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32)
    dbf = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.bfloat16)
    assert Q.gemm_status() == 0
    assert torch.equal(dbf, d32.to(torch.bfloat16)), "bf16 output is not the rounding of the fp32 output"
    del dbf

    b64 = dequant_rows_gpu(qb)                                   # [n, k] fp64
    rows = _sample_rows(m).cuda()
    assert len(rows) >= 48
    ref = dequant_rows_gpu(qa, rows) @ b64.t()                   # [rows, n] fp64
    got = d32[rows].double()
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel < REL_TOL, f"{mnk}: sampled rows rel {rel}"
    worst = ((got - ref).abs().max() / ref.abs().max()).item()
    assert worst < REL_TOL, f"{mnk}: worst element {worst}"

    # every tile at once: column sums of the whole output = (sum of the rows of A) @ B^T
    a_sum = torch.zeros(k, dtype=torch.float64, device="cuda")
    for r0 in range(0, m, 2048):
        a_sum += dequant_rows_gpu(qa, torch.arange(r0, min(m, r0 + 2048), device="cuda")).sum(0)
    col_ref = b64 @ a_sum
    col_got = d32.double().sum(0)
    # a wrong 256 x 256 tile moves 256 of these sums by about sqrt(256 / m) of their size
    assert ((col_got - col_ref).norm() / col_ref.norm()).item() < REL_TOL, f"{mnk}: column sums"
    # and the same over row sums, which localise a wrong tile to its 256 rows
    row_ref_sampled = ref.sum(1)
    assert ((got.sum(1) - row_ref_sampled).norm() / row_ref_sampled.norm()).item() < REL_TOL
