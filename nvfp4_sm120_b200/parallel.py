"""Multi-GPU forms of the FP4 path on one 8 x B200 box (one process per GPU, torch.distributed).

The reference is single-GPU (it has no collective anywhere); these are the two shardings its
path admits, each with exactly one exchange step:

* tensor-parallel SwiGLU FFN: gate/up column-parallel (weight [h/p, d] per rank), down
  row-parallel (weight [d, h/p]).  The per-tensor amax of every tensor that is split across
  ranks (the weights, the hidden activation and its gradient) is max-reduced over the group
  BEFORE quantizing, so every rank uses the global scale amax/2688 a single GPU would use and
  the round-to-nearest bytes of a shard equal the corresponding slice of the 1-GPU result.  The
  row-parallel output and the column-parallel input gradient are summed with an all-reduce.
* data-parallel training: replicas, bucketed bf16 gradient all-reduce, per-rank Philox seed offset
  so that the stochastic-rounding dither of different ranks is independent.

The local linear is injected (`linear_fn`), which lets the collective logic run on CPU ranks
(gloo) with a plain matmul; on GPUs it is FP4LinearFn."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------
# collectives as autograd functions
# ------------------------------------------------------------------------------------------
class _CopyToGroup(torch.autograd.Function):
    """Identity forward, all-reduce(SUM) backward: the input of a column-parallel linear."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    """All-reduce(SUM) forward, identity backward: the output of a row-parallel linear."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def amax_max_reducer(group=None):
    """Callable that max-reduces a 1-element fp32 amax tensor over `group`, in place."""
    def reduce_(amax):
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
        return amax
    return reduce_


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows [rank*n/world, (rank+1)*n/world) of w (the column-parallel shard of a [out, in] weight)."""
    n = w.shape[0]
    assert n % world == 0
    return w[rank * (n // world):(rank + 1) * (n // world)].contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Columns slice of w (the row-parallel shard of a [out, in] weight)."""
    n = w.shape[1]
    assert n % world == 0
    return w[:, rank * (n // world):(rank + 1) * (n // world)].contiguous()


def _fp4_linear_fn(x, w, H, signs, wq_K, wq_N, amax_reduce, sharded):
    from .linear import FP4LinearFn
    return FP4LinearFn.apply(x, w, H, signs, wq_K, wq_N, amax_reduce, sharded, None)


# ------------------------------------------------------------------------------------------
# tensor-parallel layers
# ------------------------------------------------------------------------------------------
class _ParallelLinearBase(nn.Module):
    def __init__(self, weight_shard, group, linear_fn, device):
        super().__init__()
        self.group = group
        self.weight = nn.Parameter(weight_shard.to(device))
        self.linear_fn = linear_fn or _fp4_linear_fn
        self.amax_reduce = amax_max_reducer(group)
        if linear_fn is None:
            from .linear import WeightQuantCache
            from .quant import hadamard16
            self._cache = WeightQuantCache()
            self.register_buffer("H", hadamard16(device))
            g = torch.Generator().manual_seed(1)
            self.register_buffer("signs", (torch.randint(0, 2, (16,), generator=g).float() * 2 - 1).to(device))
        else:
            self._cache = None
            self.H = self.signs = None

    def _call(self, x, sharded, x_amax=None, x_amax_signs=None, dx_reduce=None):
        """x_amax: this rank's maxima of x from a fused producer (swiglu.SwiGLUFn), FP4 path only;
        x_amax_signs: the sign vector its Hadamard maximum was computed with; dx_reduce: see FP4LinearFn."""
        wq_K = wq_N = None
        if self._cache is not None:
            wq_K, wq_N = self._cache.get(self.weight, self.amax_reduce)
        if (x_amax is not None or dx_reduce is not None) and self.linear_fn is _fp4_linear_fn:
            from .linear import FP4LinearFn, _same_signs
            rht_ok = x_amax_signs is None or _same_signs(x_amax_signs, self.signs)
            return FP4LinearFn.apply(x, self.weight, self.H, self.signs, wq_K, wq_N, self.amax_reduce, sharded, x_amax,
                                     rht_ok, dx_reduce)
        return self.linear_fn(x, self.weight, self.H, self.signs, wq_K, wq_N, self.amax_reduce, sharded)


class ColumnParallelFP4Linear(_ParallelLinearBase):
    """y_local[*, out/p] = x @ W_local^T.  x is replicated; the output and its gradient are split
    along the feature dim, so their amax is reduced; dX is summed over the group."""

    def forward(self, x, copied=False, overlap_dx=False, contiguous_shard=True):
        """copied: x already went through the group's copy (the caller feeds several column-parallel
        layers from one copy so that their input gradients are summed locally and all-reduced once).
        overlap_dx (FP4 path): no copy node; the layer itself starts the all-reduce of its input
        gradient right after its dgrad GEMM and waits for it after its wgrad GEMM.
        contiguous_shard: the shard is rows [rank n/p, (rank+1) n/p) of the whole weight, so its output
        gradient can draw the whole tensor's stochastic-rounding bits (False for packed gate|up shards)."""
        place = None
        if contiguous_shard and dist.is_available() and dist.is_initialized():
            place = (dist.get_rank(self.group), dist.get_world_size(self.group))
        if overlap_dx and self.linear_fn is _fp4_linear_fn:
            group = self.group

            def start_sum(dx):
                return dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group, async_op=True)
            return self._call(x, (False, True, place), dx_reduce=start_sum)
        if not copied:
            x = _CopyToGroup.apply(x, self.group)
        return self._call(x, (False, True, place))


class RowParallelFP4Linear(_ParallelLinearBase):
    """y[*, out] = sum over ranks of x_local @ W_local^T.  The input is split along the feature dim
    (its amax is reduced); the output is summed over the group and is then replicated."""

    def forward(self, x_local, amax=None, amax_signs=None):
        y = self._call(x_local, (True, False), amax, amax_signs)
        return _ReduceFromGroup.apply(y, self.group)


class TensorParallelSwiGLU(nn.Module):
    """SwiGLU FFN y = down(silu(gate(x)) * up(x)) with d_model d and hidden h, sharded over `group`
    (benchmark config 4: d 4096, h 14336).  Built from this rank's shards: gate/up [h/p, d], down [d, h/p];
    `from_full` slices them out of the unsharded [h, d], [h, d], [d, h] weights."""

    def __init__(self, gate_shard, up_shard, down_shard, group=None, linear_fn=None, device="cuda", fuse_gate_up=False):
        """fuse_gate_up (FP4 path): this rank's gate and up shards as ONE [2 h/p, d] projection: x is
        quantized once per layout, one dgrad GEMM over K = 2 h/p whose all-reduce runs beside the
        wgrad GEMM, and the SwiGLU kernels work on the packed [tokens, 2 h/p] tensors in place."""
        super().__init__()
        self.fuse_gate_up = bool(fuse_gate_up and linear_fn is None)
        if self.fuse_gate_up:
            self.gate_up = ColumnParallelFP4Linear(torch.cat([gate_shard, up_shard], 0), group, linear_fn, device)
        else:
            self.gate = ColumnParallelFP4Linear(gate_shard, group, linear_fn, device)
            self.up = ColumnParallelFP4Linear(up_shard, group, linear_fn, device)
        self.down = RowParallelFP4Linear(down_shard, group, linear_fn, device)

    @classmethod
    def from_full(cls, full_gate, full_up, full_down, group=None, linear_fn=None, device="cuda", fuse_gate_up=False):
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        return cls(shard_rows(full_gate, rank, world), shard_rows(full_up, rank, world),
                   shard_cols(full_down, rank, world), group, linear_fn, device, fuse_gate_up)

    def forward(self, x):
        if self.fuse_gate_up:
            from .swiglu import swiglu_packed
            gu = self.gate_up(x, overlap_dx=True, contiguous_shard=False)
            tokens = gu.numel() // gu.shape[-1]
            h, h_max = swiglu_packed(gu, self.gate_up.signs if tokens % 16 == 0 else None)
            return self.down(h, amax=h_max, amax_signs=self.gate_up.signs)
        # one copy-to-group for both projections: autograd adds gate's and up's input gradients
        # locally and the sum crosses the links once
        xc = _CopyToGroup.apply(x, self.gate.group)
        g, u = self.gate(xc, copied=True), self.up(xc, copied=True)
        if self.gate.linear_fn is _fp4_linear_fn and g.is_cuda and g.dtype == torch.bfloat16:
            # fused SwiGLU: the maxima it leaves are this rank's; the linears reduce them over the group
            from .swiglu import swiglu
            tokens = g.numel() // g.shape[-1]
            h, h_max = swiglu(g, u, self.gate.signs if tokens % 16 == 0 else None)
            return self.down(h, amax=h_max, amax_signs=self.gate.signs)
        return self.down(F.silu(g) * u)


# ------------------------------------------------------------------------------------------
# data parallel
# ------------------------------------------------------------------------------------------
def broadcast_parameters(module: nn.Module, src: int = 0, group=None):
    """Make every replica start from rank src's parameters and buffers."""
    with torch.no_grad():
        for t in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(t, src=src, group=group)


def all_reduce_gradients(params, group=None, bucket_bytes: int = 64 << 20, wire_dtype=torch.bfloat16):
    """Average the gradients of `params` over the group: gradients are packed into buckets of about
    bucket_bytes in `wire_dtype` (bf16 on the wire, as the data-parallel config asks), summed with
    one all-reduce per bucket, divided by the group size and copied back in their own dtype."""
    world = dist.get_world_size(group)
    grads = [p.grad for p in params if p.grad is not None]
    esize = torch.empty((), dtype=wire_dtype).element_size()
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        flat = torch.cat([g.reshape(-1).to(wire_dtype) for g in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat = flat.float().div_(world)
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n
        bucket, size = [], 0

    for g in grads:
        bucket.append(g)
        size += g.numel() * esize
        if size >= bucket_bytes:
            flush()
    flush()


class GradientReducer:
    """Data-parallel gradient averaging overlapped with the backward pass.

    The parameters are cut into buckets of about `bucket_bytes` in the order the backward pass
    finishes them (reverse registration order).  Every parameter gets a post-accumulate hook; once
    `arm()` has been called (before the backward of the LAST microbatch of a step) the hook counts
    the bucket down, and the bucket whose last gradient has just been accumulated is packed into one
    `wire_dtype` buffer (bf16 on the wire, as the data-parallel benchmark config asks) and all-reduced
    asynchronously: NCCL runs it on its own stream while the main stream goes on with the rest of the
    backward.  `finish()` launches what is left (parameters that received no gradient are skipped),
    waits, divides by the group size and writes the averages back in the gradients' own dtype."""

    def __init__(self, params, group=None, bucket_bytes: int = 32 << 20, wire_dtype=torch.bfloat16):
        self.group, self.wire_dtype = group, wire_dtype
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        esize = torch.empty((), dtype=wire_dtype).element_size()
        self.buckets, cur, size = [], [], 0
        seen = set()
        for p in reversed([p for p in params if p.requires_grad]):
            if id(p) in seen:                      # a tied parameter appears once
                continue
            seen.add(id(p))
            cur.append(p)
            size += p.numel() * esize
            if size >= bucket_bytes:
                self.buckets.append(cur)
                cur, size = [], 0
        if cur:
            self.buckets.append(cur)
        self._bucket_of = {id(p): i for i, b in enumerate(self.buckets) for p in b}
        self._pending, self._inflight, self._armed = [], {}, False
        self._handles = [p.register_post_accumulate_grad_hook(self._on_grad) for b in self.buckets for p in b]

    def arm(self):
        """Call before the backward pass whose gradients are final (the last microbatch)."""
        self._pending = [len(b) for b in self.buckets]
        self._inflight = {}
        self._armed = True

    def _on_grad(self, p):
        if not self._armed:
            return
        i = self._bucket_of[id(p)]
        self._pending[i] -= 1
        if self._pending[i] == 0:
            self._launch(i)

    def _launch(self, i):
        ps = [p for p in self.buckets[i] if p.grad is not None]
        if not ps:
            return
        flat = torch.cat([p.grad.reshape(-1).to(self.wire_dtype) for p in ps])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True) if self.world > 1 else None
        self._inflight[i] = (ps, flat, work)

    def finish(self):
        """Wait for every bucket and store the averaged gradients."""
        if not self._armed:
            raise RuntimeError("GradientReducer.finish() without arm()")
        self._armed = False
        for i in range(len(self.buckets)):
            if i not in self._inflight:
                self._launch(i)                    # a bucket some gradient never reached
        for i in sorted(self._inflight):
            ps, flat, work = self._inflight[i]
            if work is not None:
                work.wait()
            off = 0
            for p in ps:
                n = p.numel()
                p.grad.copy_(flat[off:off + n].view_as(p.grad).to(p.grad.dtype).div_(self.world))
                off += n
        self._inflight = {}

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []


def seed_stochastic_rounding(base_seed: int, rank: int):
    """Give each data-parallel rank its own Philox seed range (seeds advance by one per stochastic
    quantization, nvfp4_cuda.py:160-162; ranks are 2^40 apart)."""
    from . import quant
    quant._SEED[0] = int(base_seed) + (int(rank) << 40)
