"""The data half of the reference's nvfp4_validate module (nvfp4_validate.py:239-264), which its
trainer imports as `D`: the 3-digit addition dataset.  The fake-quant simulator of that file is the
reference's own oracle and is not re-provided here."""
import torch

from nvfp4_sm120_b200 import addition as _a

DEV = "cuda"
VOCAB = list(_a.VOCAB)
STOI = {c: i for i, c in enumerate(VOCAB)}
SEQ = _a.SEQ
ANS_SLICE = _a.ANSWER


def encode_pair(a, b):
    return _a.encode(torch.tensor([a]), torch.tensor([b]))[0].tolist()


def build_dataset():
    """(train, held-out) as tensors of pair indices p = 1000 * a + b (the reference returns lists of
    (a, b) tuples; make_batch below takes these tensors)."""
    return _a.split_pairs()


def make_batch(pairs, bs, g):
    return _a.make_batch(pairs, bs, g, DEV)
