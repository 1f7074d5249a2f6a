"""Small fixed cases of the hot-path kernels, for profilers (ncu) and quick timing.

    python -m nvfp4_sm120_b200.profile_case quant --rows 16384 --cols 8192 --mode rht_sr --iters 3
    python -m nvfp4_sm120_b200.profile_case gemm --m 4096 --n 4096 --k 4096 --iters 3
    python -m nvfp4_sm120_b200.profile_case block --d 768 --heads 12 --tokens 16384 --iters 3

Prints the CUDA-event time per iteration.  Inputs are random bf16 from a device generator."""
import argparse

import torch

import nvfp4_sm120_b200 as Q


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["quant", "gemm", "ffn", "block"])
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--mode", default="rne", choices=["rne", "sr", "rht_sr"])
    ap.add_argument("--transpose", action="store_true")
    ap.add_argument("--rotate", type=int, default=1, help="quant: number of input tensors taken in turn (more than "
                    "L2 / tensor size of them make every launch read HBM)")
    ap.add_argument("--known-amax", action="store_true", help="quant: hand the quantizer the maximum (one-pass form)")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--h", type=int, default=14336)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--heads", type=int, default=12, help="block: attention heads (sequence length 1024)")
    ap.add_argument("--bf16", action="store_true", help="ffn: bf16 nn.Linear comparator instead of FP4Linear")
    ap.add_argument("--fuse-gate-up", action="store_true", help="ffn: one [2h, d] gate|up projection")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--gemm-mode", type=int, default=0, help="0 auto, 1 one-CTA kernel, 2 persistent two-CTA kernel")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    from nvfp4_sm120_b200 import _lib
    _lib.lib().nvfp4_gemm_set_mode(a.gemm_mode)
    g = torch.Generator(device=dev).manual_seed(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.case == "ffn":
        from nvfp4_sm120_b200.ffn import SwiGLUFFN, ffn_flops
        Q.set_amortize(True)
        m = SwiGLUFFN(a.d, a.h, use_fp4=not a.bf16, device=dev, seed=4, fuse_gate_up=a.fuse_gate_up)
        if a.bf16:
            m = m.to(torch.bfloat16)
        xs = [torch.randn(a.tokens, a.d, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
              for _ in range(a.micro)]
        gys = [torch.randn(a.tokens, a.d, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(2)]

        def step():
            Q.mark_step()
            for i, x in enumerate(xs):
                y = m(x)
                torch.autograd.grad(y, [x] + list(m.parameters()), grad_outputs=gys[i % 2])
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        fl = a.micro * ffn_flops(a.tokens, a.d, a.h)
        print(f"ffn {'bf16' if a.bf16 else 'fp4'} d={a.d} h={a.h} tokens={a.tokens} x {a.micro}: {ms:.2f} ms/step, "
              f"{fl / ms / 1e9:.0f} TFLOP/s")
        return
    if a.case == "block":
        # one decoder block of the GPT model (attention + squared-ReLU MLP), forward + backward
        from nvfp4_sm120_b200.models import DecoderBlock, rotary_tables
        Q.set_amortize(True)
        torch.manual_seed(0)
        blk = DecoderBlock(a.d, a.heads, a.heads, 4 * a.d, not a.bf16, dev)
        seq = 1024
        x = torch.randn(a.tokens // seq, seq, a.d, device=dev, dtype=torch.float32, generator=g).requires_grad_(True)
        cos, sin = rotary_tables(seq, a.d // a.heads, dev)

        def step():
            Q.mark_step()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = blk(x, cos, sin)
            y.float().square().mean().backward()
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        print(f"block {'bf16' if a.bf16 else 'fp4'} d={a.d} heads={a.heads} tokens={a.tokens}: "
              f"{e0.elapsed_time(e1) / a.iters:.3f} ms per forward+backward")
        return
    if a.case == "quant":
        xs = [torch.randn(a.rows, a.cols, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(max(1, a.rotate))]
        x = xs[0]
        signs = torch.ones(16, device=dev)
        kw = dict(stochastic=a.mode != "rne", rht=a.mode == "rht_sr", signs=signs, seed=7, transpose=a.transpose)
        if a.known_amax:                 # the same tensor values in every input: one maximum serves all
            xs = [x] + [x.clone() for _ in xs[1:]]
            kw["amax"] = Q.tensor_amax(x, kw["rht"], signs, a.transpose)
        for xi in xs:
            Q.quant_nvfp4(xi, **kw)
        torch.cuda.synchronize()
        e0.record()
        for i in range(a.iters):
            Q.quant_nvfp4(xs[i % len(xs)], **kw)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        nbytes = a.rows * a.cols * (2 + 0.5 + 1 / 16)
        print(f"quant {a.rows}x{a.cols} {a.mode} transpose={a.transpose}: {ms * 1e3:.1f} us/iter, "
              f"{nbytes / ms / 1e6:.0f} GB/s algorithmic")
        if not a.transpose and not a.known_amax:
            from nvfp4_sm120_b200 import quant
            ws = quant._workspace(dev).cpu()         # start (u64 at byte 24), four u32 offsets, last end (u64)
            start, last_end = int(ws.view(torch.int64)[3]), int(ws.view(torch.int64)[6])
            t = [0] + [int(v) & 0xffffffff for v in ws[8:12].tolist()]
            print("CTA 0 phases (us): streamed amax %.1f, stashed amax %.1f, barrier %.1f, quantize %.1f; "
                  "first CTA start to last CTA end %.1f" %
                  (tuple((t[i + 1] - t[i]) / 1e3 for i in range(4)) + ((last_end - start) / 1e3,)))
    else:
        A = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16, generator=g)
        Bt = torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16, generator=g)
        qa, qb = Q.quant_nvfp4(A), Q.quant_nvfp4(Bt)
        d = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        Q.nvfp4_mm(qa, qb.t(), out=d)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            Q.nvfp4_mm(qa, qb.t(), out=d)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        print(f"gemm {a.m}x{a.n}x{a.k}: {ms * 1e3:.1f} us/iter, {2.0 * a.m * a.n * a.k / ms / 1e9:.0f} TFLOP/s, "
              f"status {Q.gemm_status()}")


if __name__ == "__main__":
    main()
