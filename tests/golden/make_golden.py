"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own
code on the CPU.  Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

What runs: the reference's `nvfp4_gemm.quant_nvfp4`, `nvfp4_gemm.hadamard16`,
`nvfp4_validate._round_e2m1`, `nvfp4_validate.quantize_nvfp4_1d`, `quantize_nvfp4_2d`,
`apply_rht_lastdim` and the simulator autograd `_NVFP4LinearFn` (forward and backward),
unmodified, imported from that path.
`nvfp4_gemm` imports four helpers from the third-party package torchao, which is
not installed; they are stood in by the twins torch itself ships for its own
tests (`torch.testing._internal.common_quantized`: `_f32_to_floatx_unpacked`,
`pack_uint4`, `to_blocked`) and by a plain record type for `NVFP4Tensor`.  The
FP4 GEMM dispatch is never called here.

Output: one `golden_quant.pt` (a dict of small tensors) written beside this
script.  Nothing at test time reads the reference checkout.
"""
import os
import sys
import types
from collections import namedtuple

import torch


def _install_torchao_standins():
    sys.modules.setdefault("expecttest", types.ModuleType("expecttest"))
    sys.modules["expecttest"].TestCase = object
    import torch.testing._internal.common_quantized as cq

    rec = namedtuple("NVFP4Tensor", "qdata scale block_size orig_dtype per_tensor_scale "
                     "act_per_tensor_scale is_swizzled_scales use_triton_kernel act_quant_kwargs")

    def dims(m, k):
        return ((m + 127) // 128) * 128, ((k // 16 + 3) // 4) * 4

    def _no_gemm(*a, **k):
        raise RuntimeError("the FP4 GEMM dispatch is not part of the golden generator")

    pkg = types.ModuleType("torchao")
    proto = types.ModuleType("torchao.prototype")
    mx = types.ModuleType("torchao.prototype.mx_formats")
    kern = types.ModuleType("torchao.prototype.mx_formats.kernels")
    kern.f32_to_f4_unpacked = lambda x: cq._f32_to_floatx_unpacked(x, 2, 1)
    kern.pack_uint4 = cq.pack_uint4
    utils = types.ModuleType("torchao.prototype.mx_formats.utils")
    utils.to_blocked = cq.to_blocked
    nvt = types.ModuleType("torchao.prototype.mx_formats.nvfp4_tensor")
    nvt.NVFP4Tensor = rec
    nvt.hp_data_dims_to_swizzled_scale_dims_nvfp4 = dims
    nvt._addmm_nvfp4_dispatch = _no_gemm
    for name, mod in [("torchao", pkg), ("torchao.prototype", proto),
                      ("torchao.prototype.mx_formats", mx),
                      ("torchao.prototype.mx_formats.kernels", kern),
                      ("torchao.prototype.mx_formats.utils", utils),
                      ("torchao.prototype.mx_formats.nvfp4_tensor", nvt)]:
        sys.modules[name] = mod


def _input(rows, cols, seed, scale=1.0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * scale
    if outliers:
        n = x.numel()
        pos = torch.randperm(n, generator=g)[: max(1, n // 1000)]
        x.view(-1)[pos] *= 50.0
    return x.to(torch.bfloat16)


def main(ref_path):
    sys.path.insert(0, ref_path)
    import nvfp4_validate as V          # import before torch.testing internals touch backends
    _install_torchao_standins()
    import nvfp4_gemm as G

    out = {}
    H = G.hadamard16("cpu")
    out["hadamard16"] = H.clone()
    # sign vector exactly as FP4Linear draws it (nvfp4_train.py:64-66)
    g1 = torch.Generator().manual_seed(1)
    signs1 = torch.randint(0, 2, (16,), generator=g1).float() * 2 - 1
    g3 = torch.Generator().manual_seed(3)
    signs3 = torch.randint(0, 2, (16,), generator=g3).float() * 2 - 1
    out["signs_seed1"], out["signs_seed3"] = signs1, signs3

    cases = {
        "a_128x256": _input(128, 256, 10, 3.0, outliers=False),
        "b_130x192": _input(130, 192, 11),                 # ragged rows, 12 scale columns
        "c_48x80": _input(48, 80, 12),                     # 5 scale columns -> column padding
        "d_260x320": _input(260, 320, 13),
    }
    # hand-made edge rows: zeros, exact ties, an outlier block, tiny values, negative zero
    e = torch.zeros(32, 64)
    e[1, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                              -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    e[2, 16:32] = 1e-3
    e[3, 32:48] = -1e-6
    e[4, 48:64] = torch.linspace(-6, 6, 16)
    e[5, :16] = 448.0 * 6.0
    e[6, :] = torch.arange(64).float() / 8
    e[7, 5] = -0.0
    cases["e_edges_32x64"] = e.to(torch.bfloat16)
    cases["f_zeros_16x32"] = torch.zeros(16, 32, dtype=torch.bfloat16)

    for name, x in cases.items():
        out[f"{name}.x"] = x
        q = G.quant_nvfp4(x)
        out[f"{name}.rne.qdata"] = q.qdata
        out[f"{name}.rne.scale"] = q.scale.view(torch.uint8)
        out[f"{name}.rne.pts"] = q.per_tensor_scale.reshape(())
        qr = G.quant_nvfp4(x, rht=True, H=H, signs=signs3)
        out[f"{name}.rht.qdata"] = qr.qdata
        out[f"{name}.rht.scale"] = qr.scale.view(torch.uint8)
        out[f"{name}.rht.pts"] = qr.per_tensor_scale.reshape(())

    # stochastic rounding with known uniforms: patch the reference's RNG draw
    real_rand_like = torch.rand_like
    for name in ("a_128x256", "b_130x192"):
        x = cases[name]
        gu = torch.Generator().manual_seed(99)
        u = torch.rand(x.shape, generator=gu)
        torch.rand_like = lambda m, _u=u: _u
        try:
            q = G.quant_nvfp4(x, stochastic=True)
            qr = G.quant_nvfp4(x, stochastic=True, rht=True, H=H, signs=signs1)
        finally:
            torch.rand_like = real_rand_like
        out[f"{name}.u"] = u
        out[f"{name}.sr.qdata"] = q.qdata
        out[f"{name}.sr.scale"] = q.scale.view(torch.uint8)
        out[f"{name}.rht_sr.qdata"] = qr.qdata
        out[f"{name}.rht_sr.scale"] = qr.scale.view(torch.uint8)

    # _round_e2m1 on a dense grid, both branches
    grid = torch.linspace(-6.5, 6.5, 833)
    gu = torch.Generator().manual_seed(5)
    ug = torch.rand(grid.shape, generator=gu)
    torch.rand_like = lambda m, _u=ug: _u
    try:
        out["round.grid"], out["round.u"] = grid, ug
        out["round.sr"] = V._round_e2m1(grid, True)
        out["round.rn"] = V._round_e2m1(grid, False)
    finally:
        torch.rand_like = real_rand_like

    # the simulator's fake-quant of one case (quant -> dequant) and its RHT
    x = cases["a_128x256"]
    out["a_128x256.sim1d"] = V.quantize_nvfp4_1d(x.float())
    out["a_128x256.rht_apply"] = V.apply_rht_lastdim(x.float(), V._hadamard16("cpu", torch.float32), signs1)

    # the simulator's 16x16 weight scaling, and one forward + backward of its linear (the "reference
    # recipe": x 1-D RNE, w 2-D RNE, dY stochastic, wgrad through the Hadamard with the token dim
    # padded from 40 to 48) with the two uniform draws of the backward pass fixed
    gw = torch.Generator().manual_seed(21)
    w = torch.randn(48, 64, generator=gw) * 0.02
    out["sim.w"] = w
    out["sim.w2d"] = V.quantize_nvfp4_2d(w)
    xs = torch.randn(40, 64, generator=gw)
    gys = torch.randn(40, 48, generator=gw) * 1e-2
    u_dgrad = torch.rand(40, 48, generator=gw)            # drawn for quantize_nvfp4_1d(gy): blocks [40, 3, 16]
    u_wgrad = torch.rand(48, 48, generator=gw)            # drawn for quantize_nvfp4_1d(gy^T padded): [48, 3, 16]
    pool = {(40, 3, 16): u_dgrad.reshape(40, 3, 16), (48, 3, 16): u_wgrad.reshape(48, 3, 16)}
    torch.rand_like = lambda m: pool[tuple(m.shape)]
    try:
        cfg = {"sr": True, "rht": True}
        xr, wr = xs.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = V._NVFP4LinearFn.apply(xr, wr, cfg, V._hadamard16("cpu", torch.float32), signs1)
        y.backward(gys)
    finally:
        torch.rand_like = real_rand_like
    out["sim.x"], out["sim.gy"], out["sim.u_dgrad"], out["sim.u_wgrad"] = xs, gys, u_dgrad, u_wgrad
    out["sim.y"], out["sim.dx"], out["sim.dw"] = y.detach(), xr.grad.clone(), wr.grad.clone()

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_quant.pt")
    torch.save(out, dst)
    print(f"wrote {dst}: {len(out)} tensors, {os.path.getsize(dst) / 1e6:.2f} MB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
