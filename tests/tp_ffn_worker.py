"""Worker for test_parallel_gpu.py (launched with torch.distributed.run, one rank per GPU).
Checks the tensor-parallel FP4 SwiGLU against the single-GPU FP4 SwiGLU built from the same weights,
and the data-parallel gradient exchange, over NCCL."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import nvfp4_sm120_b200 as Q
    from nvfp4_sm120_b200 import parallel as P, quant
    from nvfp4_sm120_b200.ffn import SwiGLUFFN

    dev = torch.device("cuda", local)
    d, h, T = 512, 2048, 256
    g = torch.Generator().manual_seed(4)
    bound_d, bound_h = 1.0 / d ** 0.5, 1.0 / h ** 0.5
    gate = (torch.rand(h, d, generator=g) * 2 - 1) * bound_d
    up = (torch.rand(h, d, generator=g) * 2 - 1) * bound_d
    down = (torch.rand(d, h, generator=g) * 2 - 1) * bound_h
    x = torch.randn(T, d, generator=g).to(torch.bfloat16)
    gy = torch.randn(T, d, generator=g).to(torch.bfloat16)

    for amort in (False, True):
        Q.set_amortize(amort)
        Q.mark_step()
        # single-GPU reference on every rank
        ref = SwiGLUFFN(d, h, use_fp4=True, device=dev)
        with torch.no_grad():
            ref.gate.weight.copy_(gate); ref.up.weight.copy_(up); ref.down.weight.copy_(down)
        xr = x.to(dev).requires_grad_(True)
        quant._SEED[0] = 100
        yr = ref(xr)
        yr.backward(gy.to(dev))
        # tensor parallel
        tp = P.TensorParallelSwiGLU.from_full(gate, up, down, device=dev)
        xt = x.to(dev).requires_grad_(True)
        quant._SEED[0] = 100
        yt = tp(xt)
        yt.backward(gy.to(dev))
        torch.cuda.synchronize()
        # forward: round-to-nearest with group-reduced amax -> same quantized operands as one GPU;
        # only the bf16 partial-sum order of the row-parallel output differs
        e_y = rel(yt, yr)
        e_dx = rel(xt.grad, xr.grad)
        e_gw = rel(tp.gate.weight.grad, P.shard_rows(ref.gate.weight.grad, rank, world))
        e_dw = rel(tp.down.weight.grad, P.shard_cols(ref.down.weight.grad, rank, world))
        exact = torch.nn.functional.silu(x.float() @ gate.t()) * (x.float() @ up.t()) @ down.t()
        e_q = rel(yr.cpu(), exact)
        print(f"rank {rank} amortize={amort}: y {e_y:.4f} dx {e_dx:.4f} dW_gate {e_gw:.4f} dW_down {e_dw:.4f} "
              f"(1-GPU quantization error vs exact {e_q:.4f})", flush=True)
        assert e_y < 0.02, e_y                       # bf16 reduction order only
        # A shard draws the stochastic-rounding bits of its place in the whole tensor and uses the
        # group-reduced maxima, so its quantized operands are those of the 1-GPU run: the weight
        # gradients (no reduction across ranks) agree to the GEMM tolerance, the input gradient to the
        # bf16 order of summation of the all-reduce
        assert e_dx < 0.02, e_dx
        assert e_gw < 2e-3 and e_dw < 2e-3, (e_gw, e_dw)
        assert Q.gemm_status() == 0
    Q.set_amortize(False)

    # data parallel: broadcast + bucketed bf16 gradient average over NCCL
    lin = Q.FP4Linear(256, 128, device=dev)
    P.broadcast_parameters(lin)
    P.seed_stochastic_rounding(7, rank)
    xb = torch.randn(64, 256, device=dev, dtype=torch.bfloat16) * (rank + 1)
    lin(xb).float().square().mean().backward()
    local_grad = lin.weight.grad.clone()
    gathered = [torch.empty_like(local_grad) for _ in range(world)]
    dist.all_gather(gathered, local_grad)
    P.all_reduce_gradients([lin.weight])
    want = torch.stack(gathered).float().mean(0)
    assert rel(lin.weight.grad, want) < 0.02          # bf16 on the wire
    dist.barrier()
    if rank == 0:
        print("TP_DP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
