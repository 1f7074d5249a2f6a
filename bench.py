"""Benchmark of the NVFP4 hot path on B200.

Headline line (one JSON object on stdout, rank 0): the fused quantizer on benchmark config 2 --
a bf16 8192 x 4096 tensor (N(0,1) seed 1 + 0.1 % x50 outliers) quantized in three modes per step:
round-to-nearest, stochastic rounding (Philox seed 7), and stochastic rounding after the 16-point
random-sign Hadamard (sign seed 3).  metric = algorithmic HBM GB/s, bytes = M*K*(2 + 1/2 + 1/16)
per mode (the reference's own traffic model, tests/cuda_val.py:31).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

N > 1 (launched under torchrun) runs N independent replicas: this workload does not shard.
--impl reference times the CPU restatement of the reference's pure-torch quantizer (the oracle
port; the reference itself needs torchao and a GPU and cannot be installed offline) on the host
cores, on a bounded row sample of the same tensor.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 4096
BYTES_PER_MODE = ROWS * COLS * 2 + ROWS * COLS // 2 + ROWS * COLS // 16      # 85 983 232
MODES = ("rne", "sr", "rht_sr")
N_BUF = 6                                   # 6 x 64 MiB inputs = 384 MiB, three times the 126 MB L2
SR_SEED, SIGN_SEED, DATA_SEED = 7, 3, 1
METRIC = "quantizer HBM GB/s @8192x4096"
# one description of the workload for both arms (the GPU arm and --impl reference)
CONFIG = {"workload": "quantizer sweep bf16 8192x4096: RNE, SR (Philox seed 7), RHT (sign seed 3)+SR",
          "bytes_per_mode": BYTES_PER_MODE, "modes_per_step": 3,
          "l2": f"GPU arm: inputs rotate over {N_BUF} tensors of 64 MiB (384 MiB, larger than the 126 MB L2); "
                "reference arm: host run",
          "launch": "GPU arm: one CUDA graph per input tensor, replayed", "multi_gpu": "replicas only"}


def measured_traffic():
    """DRAM read + write bytes per launch of the single-launch quantizer from the tracked ncu summary
    of the same kernel and size (a line `traffic_bytes_per_launch: N`), or None when it is absent."""
    import re
    p = os.path.join(ROOT, "profiles", "quant_fused_8192x4096.md")
    try:
        with open(p) as f:
            m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", f.read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def synthetic(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    n = x.numel()
    pos = torch.randperm(n, generator=g)[: n // 1000]
    x.view(-1)[pos] *= 50.0
    return x.to(torch.bfloat16)


def signs_from_seed(seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 2, (16,), generator=g).float() * 2 - 1


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's pure-torch quantizer
# ----------------------------------------------------------------------------------------------
def cpu_step(O, x, signs, H, step):
    """One pass of the three modes on the host (the reference's algorithm, nvfp4_gemm.py:30-48)."""
    g = torch.Generator().manual_seed(SR_SEED + step)
    O.quant_nvfp4(x)
    O.quant_nvfp4(x, stochastic=True, u=torch.rand(x.shape, generator=g))
    O.quant_nvfp4(x, stochastic=True, rht=True, H=H, signs=signs, u=torch.rand(x.shape, generator=g))


def cpu_sample_rows(O, x_full, signs, H, budget_s):
    """Rows of the tensor one CPU step can process in about budget_s seconds."""
    probe = x_full[:256]
    t0 = time.perf_counter()
    cpu_step(O, probe, signs, H, 0)
    per_row = (time.perf_counter() - t0) / 256
    rows = int(budget_s / per_row) // 128 * 128
    return max(128, min(ROWS, rows))


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    from oracle import nvfp4_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x_full = synthetic(ROWS, COLS, DATA_SEED)
    signs, H = signs_from_seed(SIGN_SEED), O.hadamard16()
    total_steps = args.steps + args.warmup
    rows = cpu_sample_rows(O, x_full, signs, H, min(2.0, 150.0 / max(1, total_steps)))
    x = x_full[:rows].contiguous()
    for i in range(args.warmup):
        cpu_step(O, x, signs, H, i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        cpu_step(O, x, signs, H, args.warmup + i)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = 3 * (rows * COLS * (2 + 0.5 + 1 / 16)) / dt / 1e9
    sample = f"{rows} of {ROWS} rows x {COLS} cols per step, three modes (RNE, SR, RHT+SR)"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def time_events(fn, iters, stream):
    """fn(i) launched iters times; device time between two events on `stream`, in ms per call."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(iters):
        fn(i)
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def run_gpu_arm(args, rank, world, local_rank):
    import nvfp4_sm120_b200 as Q
    from nvfp4_sm120_b200 import _lib

    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        import datetime
        # a rank that fails inside an extra must not leave the others waiting for the default 10 minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=240))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.lib()
    stream = torch.cuda.current_stream()

    x_host = synthetic(ROWS, COLS, DATA_SEED + rank)
    xs = [x_host.to(dev)]
    for i in range(1, N_BUF):                      # distinct contents per buffer, same distribution
        xs.append(torch.roll(xs[0], shifts=i * 37, dims=0).contiguous())
    signs = signs_from_seed(SIGN_SEED).to(dev)

    def quant_mode(x, mode, seed):
        if mode == "rne":
            return Q.quant_nvfp4(x)
        if mode == "sr":
            return Q.quant_nvfp4(x, stochastic=True, seed=seed)
        return Q.quant_nvfp4(x, stochastic=True, rht=True, signs=signs, seed=seed)

    def step(i):
        x = xs[i % N_BUF]
        return [quant_mode(x, m, SR_SEED) for m in MODES]

    # ---- warm-up, then capture one CUDA graph per input buffer (the step is launch-bound from Python)
    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    graphs, keep = [], []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for b in range(N_BUF):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                keep.append(step(b))
            graphs.append(g)
    torch.cuda.synchronize()
    for i in range(max(3, args.warmup)):
        graphs[i % N_BUF].replay()
    torch.cuda.synchronize()

    # ---- timed region: K steps, barrier + synchronize on both sides, max over ranks
    # (the clock sampler runs from here to the end of the per-kernel pass below: the timed region
    # alone lasts a few milliseconds, shorter than one nvidia-smi sample)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(200):
        graphs[i % N_BUF].replay()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = time_events(lambda i: graphs[i % N_BUF].replay(), args.steps, torch.cuda.current_stream())
    torch.cuda.synchronize()
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    value = world * 3 * BYTES_PER_MODE / (ms * 1e-3) / 1e9

    # ---- per-kernel durations (roofline): events around every launch of a step.  The product path
    # is ONE cooperative launch per mode; the two-launch pair (amax, quantize) is timed beside it.
    amax_buf = torch.empty(1, device=dev, dtype=torch.float32)
    from nvfp4_sm120_b200.tensor import swizzled_scale_dims
    from nvfp4_sm120_b200 import quant as quant_mod
    sm, sk = swizzled_scale_dims(ROWS, COLS)
    qd = torch.empty(ROWS, COLS // 2, dtype=torch.uint8, device=dev)
    sc = torch.empty(sm, sk, dtype=torch.uint8, device=dev)
    pts = torch.empty((), dtype=torch.float32, device=dev)
    kern = {}

    def graph_time(launch, reps=20):
        """Average device time of one launch: a CUDA graph of N_BUF launches (one per input tensor),
        replayed; launches issued one by one from Python would measure the host instead."""
        side2 = torch.cuda.Stream()
        with torch.cuda.stream(side2):
            for b in range(N_BUF):
                launch(xs[b], side2.cuda_stream)
            side2.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side2):
                for b in range(N_BUF):
                    launch(xs[b], torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        return time_events(lambda i: g.replay(), reps, torch.cuda.current_stream()) / N_BUF

    for mode in MODES:
        rht, sr = int(mode == "rht_sr"), int(mode != "rne")

        def fused(x, sp_):
            lib.nvfp4_quantize_fused_bf16(x.data_ptr(), ROWS, COLS, COLS, sr, rht, signs.data_ptr(), SR_SEED, 0,
                                          qd.data_ptr(), sc.data_ptr(), pts.data_ptr(), ws2.data_ptr(), 64, sp_)

        def amax_only(x, sp_):
            lib.nvfp4_amax_bf16(x.data_ptr(), ROWS, COLS, COLS, rht, 0, signs.data_ptr(), amax_buf.data_ptr(), 1, sp_)

        def quant_only(x, sp_):
            lib.nvfp4_quantize_bf16(x.data_ptr(), ROWS, COLS, COLS, 0, sr, rht, signs.data_ptr(), amax_buf.data_ptr(),
                                    SR_SEED, 0, qd.data_ptr(), sc.data_ptr(), pts.data_ptr(), sp_)

        ws2 = torch.zeros(16, dtype=torch.int32, device=dev)
        t_fused, t_amax, t_quant = graph_time(fused), graph_time(amax_only), graph_time(quant_only)
        kern[mode] = {"fused_us": t_fused * 1e3, "gbs": BYTES_PER_MODE / (t_fused * 1e-3) / 1e9,
                      "two_launch": {"amax_us": t_amax * 1e3, "quant_us": t_quant * 1e3,
                                     "gbs": BYTES_PER_MODE / ((t_amax + t_quant) * 1e-3) / 1e9}}
    for i in range(400):
        graphs[i % N_BUF].replay()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    t_all = sum(k["fused_us"] for k in kern.values()) * 1e-6
    achieved = 3 * BYTES_PER_MODE / t_all / 1e9

    # ---- end to end through the public API with HOST buffers (pinned), copies inside the timed region
    # Double-buffered over three streams (PCIe is full duplex): the copy-in of step i+1 and the copy-out
    # of step i-1 run beside the kernels of step i.  Every step still moves its own input and all of
    # its results; the timed region spans pipeline fill and drain.
    x_pin = x_host.pin_memory()
    NSLOT = 2
    outs_host = [[(torch.empty(ROWS, COLS // 2, dtype=torch.uint8).pin_memory(),
                   torch.empty(sm, sk, dtype=torch.uint8).pin_memory(),
                   torch.empty((), dtype=torch.float32).pin_memory()) for _ in MODES] for _ in range(NSLOT)]
    x_devs = [torch.empty_like(xs[0]) for _ in range(NSLOT)]
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(NSLOT)]       # input of the slot is on the device
    ev_cmp = [torch.cuda.Event() for _ in range(NSLOT)]      # results of the slot are computed (input free)
    ev_out = [torch.cuda.Event() for _ in range(NSLOT)]      # results of the slot are on the host
    hold = [None] * NSLOT                                    # keeps a slot's device results alive until copied

    def e2e_step(i):
        k = i % NSLOT
        s_in.wait_event(ev_cmp[k])                           # the kernels that read this input buffer are done
        with torch.cuda.stream(s_in):
            x_devs[k].copy_(x_pin, non_blocking=True)
            ev_in[k].record(s_in)
        s_cmp.wait_event(ev_in[k])
        s_cmp.wait_event(ev_out[k])                          # the slot's previous results have left the device
        with torch.cuda.stream(s_cmp):
            hold[k] = [quant_mode(x_devs[k], m, SR_SEED + i) for m in MODES]
            ev_cmp[k].record(s_cmp)
        s_out.wait_event(ev_cmp[k])
        with torch.cuda.stream(s_out):
            for q, (hq, hs, hp) in zip(hold[k], outs_host[k]):
                hq.copy_(q.qdata, non_blocking=True)
                hs.copy_(q.scale.view(torch.uint8), non_blocking=True)
                hp.copy_(q.per_tensor_scale, non_blocking=True)
            ev_out[k].record(s_out)

    def e2e_run(n):
        """n pipelined steps; device time from before the first copy-in to after the last copy-out."""
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_in)
        for i in range(n):
            e2e_step(i)
        s_out.wait_stream(s_in)
        s_out.wait_stream(s_cmp)
        e1.record(s_out)
        e1.synchronize()
        return e0.elapsed_time(e1) / n

    e2e_run(3)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_iters = max(5, min(args.steps, 20))
    e2e_ms = e2e_run(e2e_iters)
    torch.cuda.synchronize()
    e2e_ok = all(bool(torch.equal(hq, q.qdata.cpu())) for q, (hq, _, _) in zip(hold[(e2e_iters - 1) % NSLOT],
                                                                           outs_host[(e2e_iters - 1) % NSLOT]))
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_val = world * 3 * BYTES_PER_MODE / (e2e_ms * 1e-3) / 1e9
    h2d = ROWS * COLS * 2
    d2h = 3 * (ROWS * COLS // 2 + sm * sk + 4)

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "clocks": clocks,
        "gpu_launches": 3 * args.steps,
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "results_on_host_match_device": e2e_ok,
                "note": "pinned host input -> device, three quantizations, all results -> pinned host; double-buffered "
                        "over three streams so that copy-in, kernels and copy-out of neighbouring steps overlap; "
                        "timed from before the first copy-in to after the last copy-out"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": measured_traffic(), "peak_kind": peak_kind,
                     "traffic_note": "dram read + write bytes per launch from an ncu capture of the same kernel and "
                                     "size (the tracked summary of that capture), mean of the three modes",
                     "kernel": "quant_fused_kernel, one launch per mode (algorithmic bytes of the three modes / summed event time)"},
        "modes": kern,
        "quantizer_error_word": quant_mod.fused_error(dev),
    }

    if rank == 0 and world == 1:
        from oracle import nvfp4_oracle as O
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        Hc, sg = O.hadamard16(), signs_from_seed(SIGN_SEED)
        rows = cpu_sample_rows(O, x_host, sg, Hc, 6.0)
        xc = x_host[:rows].contiguous()
        cpu_step(O, xc[:128], sg, Hc, 0)
        best = 1e30
        for r in range(2):
            t0 = time.perf_counter()
            cpu_step(O, xc, sg, Hc, r)
            best = min(best, time.perf_counter() - t0)
        line["cpu_baseline"] = {"value": 3 * rows * COLS * (2 + 0.5 + 1 / 16) / best / 1e9, "unit": "GB/s",
                                "cores": cores, "kind": "port",
                                "sample": f"{rows} of {ROWS} rows x {COLS} cols, three modes, best of 2"}
        if not args.no_extras:
            try:                                   # what stands beside the headline must not take it down
                line["extras"] = extras(Q, dev, bf16_peak, peak_kind)
            except Exception as exc:
                line["extras"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            try:
                line["extras"]["dp_gpt124m"] = extras_data_parallel(Q, dev, 0, 1, None)
            except Exception as exc:
                line["extras"]["dp_gpt124m"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if world > 1 and not args.no_extras:
        try:
            tp = extras_tensor_parallel(Q, dev, rank, world, dist)
        except Exception as exc:
            tp = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        try:
            tp_fused = extras_tensor_parallel(Q, dev, rank, world, dist, fuse_gate_up=True)
        except Exception as exc:
            tp_fused = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        try:
            dp = extras_data_parallel(Q, dev, rank, world, dist, backends=("fp4",))
        except Exception as exc:
            dp = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        if rank == 0:
            line["extras"] = {"ffn_tensor_parallel": tp, "ffn_tensor_parallel_fused_gate_up": tp_fused, "dp_gpt124m": dp}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def extras_data_parallel(Q, dev, rank, world, dist, backends=("fp4", "bf16")):
    """benchmark config 5 on `world` GPUs: GPT 12 layers / d 768 / 12 heads / MLP 4x / vocab 50257,
    seq 1024, 256 sequences per optimizer step split over the ranks (strong scaling), every linear of
    every block an FP4Linear, AdamW, synthetic Zipf(1.1) token ids; bf16 gradient all-reduce over NCCL
    overlapped with the last backward pass.  One warm-up step, two timed steps, device time, max over
    ranks; tokens/s = 262 144 tokens / step time."""
    from nvfp4_sm120_b200.train import Trainer
    res = {}
    for backend in backends:
        tr = Trainer(dev, rank, world, backend=backend, all_fp4=True, total_steps=300)
        tr.step(20)                                   # warm-up at a mid-schedule learning rate
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n = 2
        for i in range(n):
            loss = tr.step(21 + i)
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        res[backend] = {"ms_per_step": ms, "tokens_per_s": tr.global_batch * tr.seq / (ms * 1e-3),
                        "loss_after_3_steps": float(loss), "fp4_linears": len(tr.model.fp4_linears()),
                        "microbatches_per_rank": tr.accum}
        if tr.reducer is not None:
            res[backend]["gradient_buckets"] = len(tr.reducer.buckets)
            tr.reducer.remove()
        del tr
        torch.cuda.empty_cache()
    Q.set_amortize(False)
    res["config"] = ("GPT-124M, 256 x 1024 tokens per step over all ranks, all 72 block linears FP4, AdamW, bf16 "
                     "gradient all-reduce overlapped with backward; scaling: strong")
    res["dp"] = world
    return res


def extras_tensor_parallel(Q, dev, rank, world, dist, fuse_gate_up=False):
    """benchmark config 4 over `world` GPUs: SwiGLU d 4096 / h 14336 split column- (gate, up) and row-wise
    (down), 8 microbatches x 4096 tokens, forward + backward, amortized weight quantization; NCCL
    all-reduce of the amax words and of the row-parallel output / column-parallel input gradient.
    Strong scaling: the same total work on more GPUs.  Timed on the device, max over ranks."""
    from nvfp4_sm120_b200 import parallel as P
    from nvfp4_sm120_b200.ffn import ffn_flops
    d_model, hidden, tokens, micro = 4096, 14336, 4096, 8
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    bd, bh = 1.0 / d_model ** 0.5, 1.0 / hidden ** 0.5
    hs = hidden // world
    mk = lambda r, c, b: (torch.rand(r, c, device=dev, generator=g) * 2 - 1) * b
    ffn = P.TensorParallelSwiGLU(mk(hs, d_model, bd), mk(hs, d_model, bd), mk(d_model, hs, bh), device=dev,
                                 fuse_gate_up=fuse_gate_up)
    gx = torch.Generator(device=dev).manual_seed(40)              # activations are replicated
    xs = [torch.randn(tokens, d_model, device=dev, dtype=torch.bfloat16, generator=gx).requires_grad_(True)
          for _ in range(micro)]
    gy = torch.randn(tokens, d_model, device=dev, dtype=torch.bfloat16, generator=gx)
    Q.set_amortize(True)

    def step():
        Q.mark_step()
        for x in xs:
            y = ffn(x)
            torch.autograd.grad(y, [x] + list(ffn.parameters()), grad_outputs=gy)
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    # The sharded step is host-bound when launched kernel by kernel (hundreds of launches and small
    # collectives for a few milliseconds of device work), so it is captured once into a CUDA graph --
    # kernels, autograd and NCCL collectives alike -- and replayed.  Eager timing is kept beside it.
    def timed(fn, reps=3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / reps
    eager_ms = timed(step)
    graph_ms, graph_note = None, "captured"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()                                   # allocations of the capture stream's first use
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        graph_ms = timed(graph.replay)
    except Exception as exc:                         # capture is an optimisation: report and keep the eager number
        graph_note = f"capture failed: {type(exc).__name__}: {str(exc)[:120]}"
        torch.cuda.synchronize()
    best = eager_ms if graph_ms is None else min(eager_ms, graph_ms)
    t = torch.tensor([best, eager_ms, -1.0 if graph_ms is None else graph_ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    Q.set_amortize(False)
    ms, eager_ms = float(t[0]), float(t[1])
    return {"ms_per_step": ms, "tflops_all_gpus": micro * ffn_flops(tokens, d_model, hidden) / ms / 1e9,
            "eager_ms_per_step": eager_ms, "graph_ms_per_step": None if float(t[2]) < 0 else float(t[2]),
            "graph": graph_note, "scaling": "strong", "tp": world, "gemm_status": Q.gemm_status(),
            "config": "SwiGLU d4096 h14336, 8 microbatches x 4096 tokens, fwd+bwd, TP over NCCL" +
                      (", gate|up as one column-parallel projection, dX all-reduce beside the wgrad GEMM" if fuse_gate_up else "")}


def library_fp4_mm(qa, qb):
    """The library comparator, bench-side only: cuBLASLt's block-scaled NVFP4 GEMM reached through
    torch's scaled matmul on the SAME quantized operands (what the reference's fp4_matmul dispatches
    to through torchao, nvfp4_gemm.py:57).  Returns (callable(out) or None, description)."""
    import torch.nn.functional as F
    a4 = qa.qdata.view(torch.float4_e2m1fn_x2)
    b4 = qb.qdata.view(torch.float4_e2m1fn_x2).t()
    sa, sb = qa.scale.reshape(-1), qb.scale.reshape(-1)
    ga, gb = qa.per_tensor_scale.reshape(1), qb.per_tensor_scale.reshape(1)
    tried = []
    if hasattr(F, "scaled_mm") and hasattr(F, "ScalingType"):
        ST, SW = F.ScalingType, F.SwizzleType
        def two_level():
            return F.scaled_mm(a4, b4, [sa, ga], [ST.BlockWise1x16, ST.TensorWise], [sb, gb],
                               [ST.BlockWise1x16, ST.TensorWise], [SW.SWIZZLE_32_4_4, SW.NO_SWIZZLE],
                               [SW.SWIZZLE_32_4_4, SW.NO_SWIZZLE], output_dtype=torch.bfloat16)
        def one_level():
            return F.scaled_mm(a4, b4, sa, ST.BlockWise1x16, sb, ST.BlockWise1x16, SW.SWIZZLE_32_4_4,
                               SW.SWIZZLE_32_4_4, output_dtype=torch.bfloat16)
        for name, fn in (("F.scaled_mm block 1x16 + per-tensor scale", two_level),
                         ("F.scaled_mm block 1x16 scales only (per-tensor scales left out of the timed call)", one_level)):
            try:
                fn()
                torch.cuda.synchronize()
                return fn, name
            except Exception as exc:                 # try the next spelling
                tried.append(f"{name}: {type(exc).__name__}: {str(exc)[:80]}")
    try:
        fn = lambda: torch._scaled_mm(a4, b4, sa, sb, out_dtype=torch.bfloat16)
        fn()
        torch.cuda.synchronize()
        return fn, "torch._scaled_mm block scales only (per-tensor scales left out of the timed call)"
    except Exception as exc:
        tried.append(f"torch._scaled_mm: {type(exc).__name__}: {str(exc)[:80]}")
    return None, "unavailable: " + " | ".join(tried)


def extras(Q, dev, bf16_peak, peak_kind):
    """Beside the headline: FP4 GEMM throughput on benchmark config 3 shapes with the library's FP4
    GEMM (cuBLASLt through torch, same quantized operands) and bf16 torch.matmul alongside, each as a
    burst figure (single launches, L2 flushed, after a pause) and a sustained one (back to back for
    about a second); then the SwiGLU FFN of config 4 (d 4096, h 14336, 8 x 4096 tokens)
    forward+backward in FP4 (amortized weight quantization) against the same block in bf16."""
    out = {"gemm": []}
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for (m, n, k) in [(4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (16384, 4096, 14336)]:
        g = torch.Generator(device=dev).manual_seed(2)
        A = torch.randn(m, k, device=dev, dtype=torch.bfloat16, generator=g)
        Bt = torch.randn(n, k, device=dev, dtype=torch.bfloat16, generator=g)
        qa, qb = Q.quant_nvfp4(A), Q.quant_nvfp4(Bt)
        d = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        lib_fn, lib_note = library_fp4_mm(qa, qb)
        fns = {"fp4": lambda: Q.nvfp4_mm(qa, qb.t(), out=d), "bf16": lambda: torch.matmul(A, Bt.t(), out=d)}
        lib_check = None
        if lib_fn is not None:
            fns["cublaslt_fp4"] = lib_fn
            ours = Q.nvfp4_mm(qa, qb.t(), out_dtype=torch.float32)
            theirs = lib_fn().float()
            if "only" in lib_note:
                theirs = theirs * (qa.per_tensor_scale * qb.per_tensor_scale)
            lib_check = float((theirs - ours).norm() / ours.norm())       # the comparator computes the same product
            del ours, theirs
        flops = 2.0 * m * n * k
        rec = {"m": m, "n": n, "k": k, "library": lib_note, "library_vs_ours_rel_diff": lib_check}
        for name, fn in fns.items():
            # burst: single launches; let the previous seconds of dense GEMMs drain out of the
            # power/thermal state first (a shape read 30 % low right after the 16384^3 runs)
            torch.cuda.synchronize()
            time.sleep(1.0)
            for _ in range(3):
                fn()
            ts = []
            for _ in range(10):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); e1.synchronize()
                ts.append(e0.elapsed_time(e1))
            burst_ms = statistics.median(ts)
            # sustained: back to back for about a second, under the power cap
            reps = max(5, min(4000, int(1000.0 / burst_ms)))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record(); e1.synchronize()
            rec[f"{name}_tflops"] = flops / (burst_ms * 1e-3) / 1e12
            rec[f"{name}_tflops_sustained"] = flops / (e0.elapsed_time(e1) / reps * 1e-3) / 1e12
        rec["frac_of_4x_bf16_peak"] = rec["fp4_tflops"] / (4 * bf16_peak)
        rec["frac_of_9pf_datasheet"] = rec["fp4_tflops"] / 9000.0
        out["gemm"].append(rec)
        del A, Bt, qa, qb, d, fns, lib_fn
    out["gemm_peak_kind"] = f"4 x {peak_kind} bf16 burst ({bf16_peak} TF/s)"
    del flush
    torch.cuda.empty_cache()

    from nvfp4_sm120_b200.ffn import SwiGLUFFN, ffn_flops
    d_model, hidden, tokens, micro = 4096, 14336, 4096, 8
    g = torch.Generator(device=dev).manual_seed(4)
    xs = [torch.randn(tokens, d_model, device=dev, dtype=torch.bfloat16, generator=g).requires_grad_(True)
          for _ in range(micro)]
    gy = torch.randn(tokens, d_model, device=dev, dtype=torch.bfloat16, generator=g)
    ffn = {}
    Q.set_amortize(True)
    for name in ("fp4", "fp4_fused_gate_up", "bf16"):
        # "fp4": three FP4Linear as the benchmark config words it; "fp4_fused_gate_up": the same block
        # with gate and up kept as one [2h, d] projection (one quantization of x per layout, one dgrad GEMM)
        m = SwiGLUFFN(d_model, hidden, use_fp4=(name != "bf16"), device=dev, seed=4,
                      fuse_gate_up=(name == "fp4_fused_gate_up"))
        if name == "bf16":
            m = m.to(torch.bfloat16)

        def step():
            Q.mark_step()
            for x in xs:
                y = m(x)
                torch.autograd.grad(y, [x] + list(m.parameters()), grad_outputs=gy)
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            step()
        e1.record()
        e1.synchronize()
        ms = e0.elapsed_time(e1) / 3
        ffn[name] = {"ms_per_step": ms, "tflops": micro * ffn_flops(tokens, d_model, hidden) / ms / 1e9}
        del m
        torch.cuda.empty_cache()
    Q.set_amortize(False)
    ffn["speedup_vs_bf16"] = ffn["bf16"]["ms_per_step"] / ffn["fp4"]["ms_per_step"]
    ffn["speedup_vs_bf16_fused_gate_up"] = ffn["bf16"]["ms_per_step"] / ffn["fp4_fused_gate_up"]["ms_per_step"]
    ffn["config"] = "SwiGLU d4096 h14336, 8 microbatches x 4096 tokens, fprop RNE / dgrad SR / wgrad RHT+SR, 1 GPU"
    out["ffn_fwd_bwd"] = ffn
    out["gemm_status"] = Q.gemm_status()
    return out


def gemm_case(which, m, n, k, launches=3):
    """A few launches of one GEMM for a profiler: `ours` = nvfp4_mm, `library` = the cuBLASLt comparator
    of the extras, both on the same quantized operands (config 3's generator)."""
    import nvfp4_sm120_b200 as Q
    from nvfp4_sm120_b200.gemm import nvfp4_mm
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    qa = Q.quant_nvfp4(torch.randn(m, k, device=dev, dtype=torch.bfloat16, generator=g))
    qb = Q.quant_nvfp4(torch.randn(n, k, device=dev, dtype=torch.bfloat16, generator=g))
    if which == "library":
        fn, note = library_fp4_mm(qa, qb)
        if fn is None:
            raise SystemExit("no library FP4 GEMM in this torch: " + note)
    else:
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        fn, note = (lambda: nvfp4_mm(qa, qb.t(), out=out)), "nvfp4_mm"
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / launches * 1e3
    print(f"{which} ({note}) {m}x{n}x{k}: {us:.1f} us per launch, {2.0 * m * n * k / us / 1e6:.0f} TFLOP/s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--gemm-case", choices=["ours", "library"], default=None,
                    help="profiling aid: run a few launches of one FP4 GEMM (this build's kernel, or the library "
                         "comparator on the same quantized operands), print the time and exit")
    ap.add_argument("--mnk", type=int, nargs=3, default=[8192, 8192, 8192])
    args = ap.parse_args()
    if args.gemm_case is not None:
        gemm_case(args.gemm_case, *args.mnk)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); the CPU arm is --impl reference")
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
