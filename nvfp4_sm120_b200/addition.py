"""The reference's convergence check: 3-digit addition as a character LM with held-out pairs
(data: nvfp4_validate.py:239-282; trainer: nvfp4_train.py:143-200), on this build's FP4Linear.

    python -m nvfp4_sm120_b200.addition --steps 1500

Sequences are "DDD+DDD=DDDD\\n" (13 characters, vocabulary "0123456789+=\\n"); 900 000 of the 10^6
(a, b) pairs train, 100 000 are held out (permutation from a CPU generator with seed 0, as the
reference splits them); accuracy = all five answer characters right on held-out pairs.  The
reference reports bf16 100 %, NVFP4 with the full recipe 100 %, NVFP4 without SR+RHT 1.9 %."""
from __future__ import annotations

import argparse
import json
import time

import torch
import torch.nn.functional as F

from . import linear
from .models import LM

VOCAB = "0123456789+=\n"
SEQ = 13
ANSWER = slice(7, 12)          # the answer "DDDD\n" inside the 12 target positions


def encode(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[n] operands -> [n, 13] token ids of "aaa+bbb=cccc\\n"."""
    c = a + b
    digit = lambda v, p: (v // p) % 10
    cols = [digit(a, 100), digit(a, 10), digit(a, 1), torch.full_like(a, 10),
            digit(b, 100), digit(b, 10), digit(b, 1), torch.full_like(a, 11),
            digit(c, 1000), digit(c, 100), digit(c, 10), digit(c, 1), torch.full_like(a, 12)]
    return torch.stack(cols, dim=1)


def split_pairs():
    """Train / held-out pair indices (pair p = (p // 1000, p % 1000)), the reference's split."""
    perm = torch.randperm(1_000_000, generator=torch.Generator().manual_seed(0))
    return perm[100_000:], perm[:100_000]


_PAIR_LISTS = {}


def pair_tuples(idx):
    """Pair indices -> the reference's form, a list of (a, b) tuples (nvfp4_validate.py:247-255);
    the list is remembered so that as_pair_indices finds its tensor again without a conversion."""
    out = list(zip((idx // 1000).tolist(), (idx % 1000).tolist()))
    _PAIR_LISTS[id(out)] = (out, idx)
    return out


def as_pair_indices(pairs):
    """A tensor of pair indices 1000 a + b, or a list of (a, b) tuples -> the index tensor."""
    if isinstance(pairs, torch.Tensor):
        return pairs
    hit = _PAIR_LISTS.get(id(pairs))
    if hit is not None and hit[0] is pairs:
        return hit[1]
    t = torch.tensor(pairs, dtype=torch.long)
    idx = t[:, 0] * 1000 + t[:, 1]
    _PAIR_LISTS[id(pairs)] = (pairs, idx)
    return idx


def make_batch(pairs, batch, gen, device):
    pairs = as_pair_indices(pairs)
    pick = pairs[torch.randint(0, len(pairs), (batch,), generator=gen)]
    tok = encode(pick // 1000, pick % 1000).to(device)
    return tok[:, :-1], tok[:, 1:]


@torch.no_grad()
def evaluate(model, held_out, gen, device, batches=8, batch=512):
    model.eval()
    loss_sum, right, seen = 0.0, 0, 0
    for _ in range(batches):
        x, y = make_batch(held_out, batch, gen, device)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = model(x)
        loss_sum += F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), y.reshape(-1)).item()
        right += (logits[:, ANSWER].argmax(-1) == y[:, ANSWER]).all(dim=1).sum().item()
        seen += batch
    model.train()
    return loss_sum / batches, right / seen


def run(tag, steps, use_fp4, hp_tail=0, seed=0, device="cuda", log=print, linear_factory=None, eval_every=None):
    """One training run with the reference's hyper-parameters (nvfp4_train.py:159-185).
    linear_factory: build the low-precision linears with this callable instead of FP4Linear (see
    models.DecoderBlock); eval_every: held-out evaluation period in steps (default: six per run).
    The returned record carries every evaluation in `history`."""
    torch.manual_seed(seed)
    model = LM(len(VOCAB), 256, 6, 4, 2, 64, 768, use_fp4, hp_tail, device=device, linear_factory=linear_factory)
    train, held_out = split_pairs()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    sched = torch.optim.lr_scheduler.OneCycleLR(opt, max_lr=1e-3, total_steps=steps, pct_start=0.05)
    gen = torch.Generator().manual_seed(seed + 7)
    t0, last, diverged, history = time.time(), {}, False, []
    period = eval_every or max(1, steps // 6)
    for step in range(1, steps + 1):
        x, y = make_batch(train, 512, gen, device)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = model(x)
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), y.reshape(-1))
        if not torch.isfinite(loss):
            diverged = True
            break
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        linear.mark_step()
        if step % period == 0 or step == steps:
            val, acc = evaluate(model, held_out, gen, device)
            last = {"step": step, "train": round(loss.item(), 4), "val": round(val, 4), "acc": round(acc, 4)}
            history.append(last)
            log(json.dumps({"tag": tag, **last}))
    out = {"tag": tag, "diverged": diverged, "seconds": round(time.time() - t0, 1), **last, "history": history}
    log(json.dumps(out))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1500)
    ap.add_argument("--only", default=None, choices=[None, "bf16", "fp4"])
    a = ap.parse_args()
    linear.set_amortize(True)
    res = []
    if a.only in (None, "bf16"):
        res.append(run("bf16", a.steps, use_fp4=False))
    if a.only in (None, "fp4"):
        res.append(run("fp4-all", a.steps, use_fp4=True, hp_tail=0))
    print(json.dumps({"summary": res}))


if __name__ == "__main__":
    main()
