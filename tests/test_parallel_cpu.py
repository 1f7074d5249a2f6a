"""Host logic of the tensor-parallel FFN and the data-parallel gradient exchange, on two CPU ranks
(gloo).  The local linear is a plain fp32 matmul that also exercises the amax reduction hook, so
the test checks the collectives and the sharding, not the FP4 kernels (those are GPU tests)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _ScaledLinear(torch.autograd.Function):
    """y = x w^T, with every operand first "fake-scaled" by its (possibly group-reduced) amax, the
    way the quantizer uses it: wrong amax reduction shows up as a wrong result."""

    @staticmethod
    def forward(ctx, x, w, amax_reduce, sharded):
        def scaled(t, reduce_it):
            a = t.abs().max().reshape(1).clone()
            if reduce_it:
                amax_reduce(a)
            return torch.round(t / a * 1000.0) * a / 1000.0       # depends on the GLOBAL amax
        xs = scaled(x, sharded[0])
        ws = scaled(w, True)
        ctx.save_for_backward(xs, ws)
        return xs @ ws.t()

    @staticmethod
    def backward(ctx, gy):
        xs, ws = ctx.saved_tensors
        return gy @ ws, gy.t() @ xs, None, None


def _linear_fn(x, w, H, signs, wq_K, wq_N, amax_reduce, sharded):
    return _ScaledLinear.apply(x, w, amax_reduce, sharded)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, ROOT)
    from nvfp4_sm120_b200 import parallel as P
    torch.manual_seed(0)
    d, h, T = 32, 64, 16
    gate, up, down = torch.randn(h, d), torch.randn(h, d), torch.randn(d, h)
    x = torch.randn(T, d, requires_grad=True)
    ffn = P.TensorParallelSwiGLU.from_full(gate, up, down, linear_fn=_linear_fn, device="cpu")
    y = ffn(x)
    y.square().sum().backward()
    # unsharded reference with the same fake scaling and no group
    xr = x.detach().clone().requires_grad_(True)
    g_, u_, d_ = (t.clone().requires_grad_(True) for t in (gate, up, down))
    ident = lambda a: a
    hid = torch.nn.functional.silu(_ScaledLinear.apply(xr, g_, ident, (False, True))) * \
        _ScaledLinear.apply(xr, u_, ident, (False, True))
    yr = _ScaledLinear.apply(hid, d_, ident, (True, False))
    yr.square().sum().backward()
    ok = torch.allclose(y, yr, rtol=1e-4, atol=1e-4)
    ok &= torch.allclose(x.grad, xr.grad, rtol=1e-3, atol=1e-3)
    ok &= torch.allclose(ffn.gate.weight.grad, P.shard_rows(g_.grad, rank, world), rtol=1e-3, atol=1e-3)
    ok &= torch.allclose(ffn.down.weight.grad, P.shard_cols(d_.grad, rank, world), rtol=1e-3, atol=1e-3)
    # amax reducer
    a = torch.tensor([float(rank + 1)])
    P.amax_max_reducer()(a)
    ok &= a.item() == float(world)
    # data parallel: broadcast, then bucketed averaged gradients (bf16 on the wire)
    lin = torch.nn.Linear(8, 8)
    P.broadcast_parameters(lin)
    w0 = lin.weight.detach().clone()
    gathered = [torch.empty_like(w0) for _ in range(world)]
    dist.all_gather(gathered, w0)
    ok &= all(torch.equal(g, gathered[0]) for g in gathered)
    lin.weight.grad = torch.full_like(lin.weight, float(rank + 1))
    lin.bias.grad = torch.full_like(lin.bias, float(2 * rank))
    P.all_reduce_gradients(list(lin.parameters()), bucket_bytes=64)
    ok &= torch.allclose(lin.weight.grad, torch.full_like(lin.weight, (1 + world) / 2))
    ok &= torch.allclose(lin.bias.grad, torch.full_like(lin.bias, float(world - 1)))
    # the same averages from the reducer that overlaps the exchange with the backward pass: hooks fire
    # as gradients are accumulated, buckets go out as they fill, finish() stores the means
    torch.manual_seed(3)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    P.broadcast_parameters(net)
    red = P.GradientReducer(list(net.parameters()), bucket_bytes=64)
    ok &= len(red.buckets) >= 2
    xin = torch.full((5, 8), float(rank + 1))
    net(xin).sum().backward()                    # not armed: a microbatch before the last, nothing is sent
    ok &= red._inflight == {}
    red.arm()
    net(xin).sum().backward()
    local = [p.grad.clone() for p in net.parameters()]
    red.finish()
    for p, g in zip(net.parameters(), local):
        both = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(both, g)
        ok &= torch.allclose(p.grad, torch.stack(both).mean(0), rtol=2e-2, atol=1e-3)      # bf16 on the wire
    red.remove()
    # a whole optimizer step of the trainer on two ranks: replicas stay identical
    from nvfp4_sm120_b200.train import Trainer
    tr = Trainer(torch.device("cpu"), rank, world, backend="bf16", vocab=61, dim=32, layers=2, heads=2, seq=8,
                 global_batch=8, micro_batch=2, total_steps=4)
    for st in range(1, 4):
        tr.step(st)
    w = tr.model.blocks[1].up.weight.detach().clone()
    both = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(both, w)
    ok &= torch.equal(both[0], both[1]) and bool(torch.isfinite(w).all())
    results[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_tensor_and_data_parallel_logic_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_shard_helpers():
    from nvfp4_sm120_b200 import parallel as P
    w = torch.arange(24.0).reshape(4, 6)
    assert torch.equal(torch.cat([P.shard_rows(w, r, 2) for r in range(2)], 0), w)
    assert torch.equal(torch.cat([P.shard_cols(w, r, 3) for r in range(3)], 1), w)
