"""One FP4 decoder block, forward and backward, against the CPU oracle's recipe.

The block of nvfp4_train.py:101-123 (RMSNorm, rotary attention, squared-ReLU MLP; six linears) runs
twice from the same weights and input: once with FP4Linear on the sm_100a kernels (fused squared-ReLU
producer included), once with every linear replaced by an autograd function that evaluates the same
recipe on the CPU oracle -- fprop RNE, dgrad stochastic, wgrad Hadamard + stochastic
(nvfp4_train.py:19-55) -- drawing the same Philox seeds in the same order.  Everything else
(norms, attention, residuals) is the same torch code in both runs.

The two runs do not see bit-identical operands after the first GEMM (accumulation order, then bf16
rounding), so a rounding decision may flip downstream; the bound is the GEMM tolerance, 2e-3 relative
in the Frobenius norm, one to two orders of magnitude below the distance between the FP4 block and the
exact bf16 block (0.2 to 0.3 on the weight gradients), which the test also measures."""
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3


class _OracleLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, owner):
        x2 = x.reshape(-1, x.shape[-1]).detach().cpu().to(torch.bfloat16)
        wb = w.detach().cpu().to(torch.bfloat16)
        y = O.dequant(O.quant_nvfp4(x2)) @ O.dequant(O.quant_nvfp4(wb)).t()
        ctx.save_for_backward(x, w)
        ctx.owner = owner
        return y.to(torch.bfloat16).reshape(*x.shape[:-1], w.shape[0]).to(x.device).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        owner = ctx.owner
        x2 = x.reshape(-1, x.shape[-1]).detach().cpu().to(torch.bfloat16)
        wb = w.detach().cpu().to(torch.bfloat16)
        g2 = gy.reshape(-1, w.shape[0]).detach().cpu().to(torch.bfloat16)
        tokens, n = g2.shape
        signs = O.signs_from_seed(1)
        seed = owner.seeds[0]
        owner.seeds[0] += 2
        owner.order.append(owner.name)
        rb = O.philox_block_bits(tokens * n // 16, seed, 0)
        gq = O.dequant(O.quant_nvfp4(g2, stochastic=True, rbits=rb))
        dx = gq @ O.dequant(O.quant_nvfp4(wb.t().contiguous())).t()
        rb = O.philox_block_bits(tokens * n // 16, seed + 1, 0)
        gtq = O.dequant(O.quant_nvfp4(g2.t().contiguous(), stochastic=True, rht=True, signs=signs, rbits=rb,
                                      rht_impl="butterfly"))
        xtq = O.dequant(O.quant_nvfp4(x2.t().contiguous(), rht=True, signs=signs, rht_impl="butterfly"))
        dw = gtq @ xtq.t()
        return (dx.to(torch.bfloat16).reshape(x.shape).to(gy.device).to(gy.dtype),
                dw.to(w.device).to(w.dtype), None)


class _OracleLinear(torch.nn.Module):
    def __init__(self, cin, cout, shared):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty(cout, cin, device="cuda"))
        self.seeds, self.order = shared["seeds"], shared["order"]
        self.name = f"{cin}x{cout}#{len(shared['made'])}"
        shared["made"].append(self.name)

    def forward(self, x):
        if torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        return _OracleLinearFn.apply(x, self.weight, self)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("fused_norm,tol", [(False, TOL), (True, 5 * TOL)])
def test_decoder_block_forward_backward_match_oracle_recipe(fused_norm, tol):
    """fused_norm: the block's RMSNorms run as the fused kernel that hands the projections their maxima.
    Its output h is bf16, so the three gradients that meet at h (from q, k, v) are summed in bf16 where
    the torch norm of the oracle run sums them in fp32: a wider, still small, bound."""
    import nvfp4_sm120_b200 as Q
    from nvfp4_sm120_b200 import quant
    from nvfp4_sm120_b200.models import DecoderBlock, rotary_tables

    Q.set_amortize(False)
    dim, heads, hidden, B, T = 128, 4, 512, 2, 64
    torch.manual_seed(5)
    blk = DecoderBlock(dim, heads, heads, hidden, True, "cuda")
    assert blk.fused_act and blk.fused_norm
    blk.fused_norm = fused_norm
    shared = {"seeds": [4000], "order": [], "made": []}
    ref = DecoderBlock(dim, heads, heads, hidden, True, "cuda",
                       linear_factory=lambda cin, cout: _OracleLinear(cin, cout, shared))
    dense = DecoderBlock(dim, heads, heads, hidden, False, "cuda")
    names = ["q", "k", "v", "o", "up", "down"]
    with torch.no_grad():
        blk.norm_attn.weight.uniform_(0.5, 1.5)
        blk.norm_mlp.weight.uniform_(0.5, 1.5)
        for other in (ref, dense):
            other.norm_attn.weight.copy_(blk.norm_attn.weight)
            other.norm_mlp.weight.copy_(blk.norm_mlp.weight)
            for n in names:
                getattr(other, n).weight.copy_(getattr(blk, n).weight)
    g = torch.Generator(device="cuda").manual_seed(6)
    x0 = torch.randn(B, T, dim, device="cuda", generator=g)
    gy = torch.randn(B, T, dim, device="cuda", generator=g)
    cos, sin = rotary_tables(T, dim // heads, "cuda")

    def run(block):
        x = x0.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = block(x, cos, sin)
        y.backward(gy)
        grads = {n: getattr(block, n).weight.grad for n in names}
        grads["norm_attn"], grads["norm_mlp"] = block.norm_attn.weight.grad, block.norm_mlp.weight.grad
        return y.detach(), x.grad, grads

    quant._SEED[0] = 4000
    y_fp4, dx_fp4, gr_fp4 = run(blk)
    assert quant._SEED[0] == 4000 + 12            # six linears, two stochastic quantizations each
    y_ref, dx_ref, gr_ref = run(ref)
    assert shared["seeds"][0] == 4000 + 12
    # the oracle run's backward visited the linears in the order the real one draws its seeds in:
    # down, up, o, then the three attention projections
    kinds = [s.split("#")[0] for s in shared["order"]]
    assert kinds[:3] == [f"{hidden}x{dim}", f"{dim}x{hidden}", f"{dim}x{dim}"] and len(kinds) == 6
    y_bf, dx_bf, gr_bf = run(dense)

    report = {"y": (_rel(y_fp4, y_ref), _rel(y_fp4, y_bf)), "dx": (_rel(dx_fp4, dx_ref), _rel(dx_fp4, dx_bf))}
    for n in gr_fp4:
        report["d" + n] = (_rel(gr_fp4[n], gr_ref[n]), _rel(gr_fp4[n], gr_bf[n]))
    print("relative distance (to the oracle recipe, to the bf16 block):",
          {k: (float(f"{a:.2e}"), round(b, 4)) for k, (a, b) in report.items()})
    for k, (to_ref, to_bf16) in report.items():
        assert to_ref < tol, (k, to_ref)
        assert to_ref < 0.1 * to_bf16, (k, to_ref, to_bf16)
    assert Q.gemm_status() == 0
