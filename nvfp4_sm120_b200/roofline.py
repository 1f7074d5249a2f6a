"""Applicable roofline of an NVFP4 GEMM shape on B200, and the six training shapes of the
reference's study (cutlass_gemm/roofline.py, DEVLOG.md:168-208) measured against it.

    python -m nvfp4_sm120_b200.roofline              # arithmetic only, no GPU
    python -m nvfp4_sm120_b200.roofline --measure    # also times nvfp4_gemm on each shape

Traffic model (the reference's): A and B at 0.5 byte per element plus one E4M3 scale per 16
elements, bf16 output at 2 bytes per element.  A shape is compute-bound when its arithmetic
intensity exceeds peak / bandwidth; otherwise its ceiling is intensity x bandwidth."""
from __future__ import annotations

import argparse

PEAK_FP4_TFLOPS = 9000.0        # dense NVFP4, datasheet
HBM_GBS = 7700.0                # HBM3e, datasheet (HGX B200)

TRAINING_SHAPES = [             # (M, N, K, produced by) -- DEVLOG.md:171-178
    (16384, 512, 512, "q/k/v/o fprop+dgrad"),
    (16384, 512, 2048, "down.fprop, up.dgrad"),
    (16384, 2048, 512, "up.fprop, down.dgrad"),
    (512, 512, 16384, "q/k/v/o wgrad"),
    (512, 2048, 16384, "down.wgrad"),
    (2048, 512, 16384, "up.wgrad"),
]


def gemm_roofline(m, n, k, peak_tflops=PEAK_FP4_TFLOPS, bw_gbs=HBM_GBS):
    flops = 2.0 * m * n * k
    nbytes = (m * k + n * k) * (0.5 + 1.0 / 16.0) + 2.0 * m * n
    intensity = flops / nbytes
    ridge = peak_tflops * 1e12 / (bw_gbs * 1e9)
    compute_bound = intensity >= ridge
    ceiling = peak_tflops if compute_bound else intensity * bw_gbs * 1e9 / 1e12
    return {"flops": flops, "bytes": nbytes, "intensity": intensity, "ridge": ridge,
            "bound": "compute" if compute_bound else "hbm", "ceiling_tflops": ceiling}


def measure(m, n, k, iters=20, out_dtype=None):
    import torch
    import nvfp4_sm120_b200 as Q
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    qa = Q.quant_nvfp4(torch.randn(m, k, device=dev, dtype=torch.bfloat16, generator=g))
    qb = Q.quant_nvfp4(torch.randn(n, k, device=dev, dtype=torch.bfloat16, generator=g))
    out_dtype = out_dtype or torch.bfloat16
    d = torch.empty(m, n, device=dev, dtype=out_dtype)
    for _ in range(3):
        Q.nvfp4_mm(qa, qb.t(), out_dtype=out_dtype, out=d)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        Q.nvfp4_mm(qa, qb.t(), out_dtype=out_dtype, out=d)
    e1.record()
    torch.cuda.synchronize()
    return 2.0 * m * n * k / (e0.elapsed_time(e1) / iters) / 1e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--measure", action="store_true")
    ap.add_argument("--peak", type=float, default=PEAK_FP4_TFLOPS)
    ap.add_argument("--bw", type=float, default=HBM_GBS)
    a = ap.parse_args()
    print(f"B200: dense NVFP4 {a.peak:.0f} TFLOP/s, HBM {a.bw:.0f} GB/s, ridge {a.peak * 1e3 / a.bw:.0f} FLOP/byte")
    print(f"{'M':>6} {'N':>6} {'K':>6}  {'GFLOP':>8} {'MB':>7} {'FLOP/B':>7} {'bound':>8} {'ceiling':>8}"
          + ("  measured  % of ceiling" if a.measure else "") + "  produced by")
    for (m, n, k, who) in TRAINING_SHAPES:
        r = gemm_roofline(m, n, k, a.peak, a.bw)
        line = (f"{m:>6} {n:>6} {k:>6}  {r['flops'] / 1e9:>8.1f} {r['bytes'] / 1e6:>7.1f} {r['intensity']:>7.0f} "
                f"{r['bound']:>8} {r['ceiling_tflops']:>8.0f}")
        if a.measure:
            import torch
            # weight gradients are produced in fp32 (master weights), where K may be split over CTAs
            t = measure(m, n, k, out_dtype=torch.float32 if "wgrad" in who else torch.bfloat16)
            line += f"  {t:>8.0f}  {100 * t / r['ceiling_tflops']:>11.1f}%"
        print(line + f"  {who}")


if __name__ == "__main__":
    main()
