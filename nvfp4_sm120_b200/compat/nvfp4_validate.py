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
    """(train, val): two lists of (a, b) tuples, the held-out 100 000 first in the seed-0
    permutation, exactly what nvfp4_validate.py:247-255 returns."""
    train, held = _a.split_pairs()
    return _a.pair_tuples(train), _a.pair_tuples(held)


def make_batch(pairs, bs, g):
    """(input, target) token ids [bs, 12] on the device, drawn like nvfp4_validate.py:257-261;
    `pairs` is a list from build_dataset or a tensor of pair indices."""
    return _a.make_batch(pairs, bs, g, DEV)
