"""Training loop for the GPT of benchmark config 5 on synthetic tokens, single GPU or data parallel.

    python -m nvfp4_sm120_b200.train --steps 300 --backend fp4            # one GPU
    torchrun --nproc-per-node 8 -m nvfp4_sm120_b200.train --backend fp4   # data parallel over NCCL

Model: 12 layers, d_model 768, 12 heads, MLP 4x, RMSNorm, RoPE, vocab 50257, seq 1024, 256
sequences per optimizer step, AdamW lr 6e-4 with warm-up and cosine decay (the schedule of
scaling/train_text.py:145-149).  Token ids are drawn Zipf(s = 1.1) over the vocabulary from seed 5:
the OpenWebText slice the reference trained on is not available offline, so this is a stand-in with
the same vocabulary and sequence format; the loss floor is the entropy of that distribution.
Every rank prints nothing; rank 0 prints one JSON line per logged step and a final summary."""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch

from . import linear, parallel
from .models import GPT, GPTConfig


def zipf_sampler(vocab, s, seed, device):
    """Sampler of token ids with P(rank r) ~ r^-s over a fixed random permutation of the vocabulary."""
    g = torch.Generator().manual_seed(seed)
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
    p = ranks.pow(-s)
    p /= p.sum()
    perm = torch.randperm(vocab, generator=g)
    probs = torch.empty(vocab, dtype=torch.float64)
    probs[perm] = p
    probs = probs.float().to(device)
    gen = torch.Generator(device=device).manual_seed(seed)

    def sample(n_seq, seq_len):
        flat = torch.multinomial(probs, n_seq * (seq_len + 1), replacement=True, generator=gen)
        t = flat.view(n_seq, seq_len + 1)
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()
    entropy = float(-(p * p.log()).sum())
    return sample, entropy


def lr_at(step, base, warmup, total):
    if step < warmup:
        return base * step / warmup
    t = (step - warmup) / max(1, total - warmup)
    return base * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * t)))


class Trainer:
    """One data-parallel replica of the config-5 training job: model, AdamW, synthetic sampler and
    the optimizer step (gradient accumulation over microbatches, gradient averaging over the group
    overlapped with the last backward, clipping, AdamW, weight-quant cache refresh)."""

    def __init__(self, dev, rank=0, world=1, backend="fp4", vocab=50257, dim=768, layers=12, heads=12, seq=1024,
                 global_batch=256, micro_batch=16, lr=6e-4, warmup=15, total_steps=300, all_fp4=False,
                 overlap=True, group=None):
        self.dev, self.rank, self.world, self.seq = dev, rank, world, seq
        self.lr, self.warmup, self.total_steps, self.global_batch = lr, warmup, total_steps, global_batch
        linear.set_amortize(True)                      # weights are quantized once per optimizer step
        torch.manual_seed(0)
        # all_fp4: every linear of every block (benchmark config 5 as written, 72 linears at 12 layers);
        # otherwise the reference's placement rule: block 0 and the last block stay dense
        cfg = GPTConfig(vocab=vocab, dim=dim, n_layers=layers, n_heads=heads, n_kv_heads=heads,
                        use_fp4=backend == "fp4", hp_tail=0 if all_fp4 else 1, dense_first=not all_fp4)
        self.model = GPT(cfg, device=dev)
        if world > 1:
            parallel.broadcast_parameters(self.model)
        parallel.seed_stochastic_rounding(1234, rank)
        self.params = [p for p in self.model.parameters()]
        self.opt = torch.optim.AdamW(self.params, lr=lr, betas=(0.9, 0.95), weight_decay=0.1, fused=dev.type == "cuda")
        self.sample, self.entropy = zipf_sampler(vocab, 1.1, 5 + rank, dev)
        per_rank = global_batch // world
        assert per_rank % micro_batch == 0 and per_rank * world == global_batch
        self.micro_batch, self.accum = micro_batch, per_rank // micro_batch
        self.reducer = parallel.GradientReducer(self.params, group) if (world > 1 and overlap) else None
        self.group = group

    def step(self, step):
        """Optimizer step number `step` (1-based); returns this rank's mean microbatch loss (a tensor)."""
        for pg in self.opt.param_groups:
            pg["lr"] = lr_at(step, self.lr, self.warmup, self.total_steps)
        self.opt.zero_grad(set_to_none=True)
        loss_sum = torch.zeros((), device=self.dev)
        for i in range(self.accum):
            x, y = self.sample(self.micro_batch, self.seq)
            with torch.autocast(self.dev.type, dtype=torch.bfloat16):
                _, loss = self.model(x, y)
            if self.reducer is not None and i == self.accum - 1:
                self.reducer.arm()                     # these gradients are final: reduce them as they appear
            (loss / self.accum).backward()
            loss_sum += loss.detach() / self.accum
        if self.reducer is not None:
            self.reducer.finish()
        elif self.world > 1:
            parallel.all_reduce_gradients(self.params, self.group)
        torch.nn.utils.clip_grad_norm_(self.params, 1.0)
        self.opt.step()
        linear.mark_step()
        return loss_sum


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="fp4", choices=["fp4", "bf16"])
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--global-batch", type=int, default=256, help="sequences per optimizer step, all ranks")
    ap.add_argument("--micro-batch", type=int, default=16, help="sequences per forward/backward")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--dim", type=int, default=768)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--warmup", type=int, default=15)
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--all-fp4", action="store_true",
                    help="every linear of every block in FP4 (default: block 0 and the last block stay dense)")
    ap.add_argument("--no-overlap", action="store_true", help="reduce the gradients after the backward pass")
    ap.add_argument("--out", default=None, help="append the JSON lines to this file too")
    a = ap.parse_args()

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    tr = Trainer(dev, rank, world, a.backend, a.vocab, a.dim, a.layers, a.heads, a.seq, a.global_batch, a.micro_batch,
                 a.lr, a.warmup, a.steps, a.all_fp4, not a.no_overlap)

    def emit(rec):
        if rank == 0:
            line = json.dumps(rec)
            print(line, flush=True)
            if a.out:
                with open(a.out, "a") as f:
                    f.write(line + "\n")

    emit({"event": "start", "backend": a.backend, "params_non_embedding": tr.model.num_params(), "world": world,
          "tokens_per_step": a.global_batch * a.seq, "fp4_linears": len(tr.model.fp4_linears()),
          "zipf_entropy_nats": tr.entropy})
    t_start = None
    loss_sum = torch.zeros((), device=dev)
    for step in range(1, a.steps + 1):
        if step == 3:
            torch.cuda.synchronize()
            t_start = time.perf_counter()
        loss_sum = tr.step(step)
        if step % a.log_every == 0 or step == a.steps or step == 1:
            if world > 1:
                dist.all_reduce(loss_sum)
                loss_sum /= world
            emit({"event": "step", "step": step, "loss": round(float(loss_sum), 4), "lr": lr_at(step, a.lr, a.warmup, a.steps)})
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_start if t_start else float("nan")
    steps_timed = max(1, a.steps - 2)
    emit({"event": "done", "backend": a.backend, "world": world, "steps": a.steps,
          "ms_per_step": dt / steps_timed * 1e3, "tokens_per_s": a.global_batch * a.seq * steps_timed / dt,
          "final_loss": round(float(loss_sum), 4)})
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
