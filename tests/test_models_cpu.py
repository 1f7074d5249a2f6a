"""Callers of the hot path that do not need a GPU: the addition dataset, the model wiring in bf16
mode and the learning-rate schedule."""
import torch

from nvfp4_sm120_b200 import addition
from nvfp4_sm120_b200.models import GPT, GPTConfig, LM
from nvfp4_sm120_b200.train import lr_at, zipf_sampler


def test_addition_encoding_and_split():
    tok = addition.encode(torch.tensor([7, 999]), torch.tensor([456, 999]))
    text = ["".join(addition.VOCAB[i] for i in row) for row in tok.tolist()]
    assert text == ["007+456=0463\n", "999+999=1998\n"]           # nvfp4_validate.py:243-245 format
    train, held = addition.split_pairs()
    assert len(train) == 900_000 and len(held) == 100_000
    assert len(set(train[:1000].tolist()) & set(held.tolist())) == 0
    x, y = addition.make_batch(held, 8, torch.Generator().manual_seed(0), "cpu")
    assert x.shape == (8, 12) and torch.equal(x[:, 1:], y[:, :-1])
    assert y[:, addition.ANSWER].shape == (8, 5) and (y[:, -1] == 12).all()


def test_models_forward_backward_dense_on_cpu():
    m = LM(13, 64, 3, 4, 2, 16, 128, use_fp4=False, hp_tail=0, device="cpu")
    idx = torch.randint(0, 13, (4, 12))
    out = m(idx)
    assert out.shape == (4, 12, 13)
    out.sum().backward()
    g = GPT(GPTConfig(vocab=101, dim=64, n_layers=2, n_heads=4, n_kv_heads=4, use_fp4=False), device="cpu")
    logits, loss = g(torch.randint(0, 101, (2, 16)), torch.randint(0, 101, (2, 16)))
    assert logits.shape == (2, 16, 101) and loss.ndim == 0
    assert g.head.weight is g.emb.weight and g.fp4_linears() == []
    assert g.num_params() == sum(p.numel() for p in g.parameters()) - 101 * 64


def test_fp4_placement_rule():
    """First block and the last hp_tail blocks stay dense (scaling/train_text.py:66-67)."""
    cfg = GPTConfig(vocab=32, dim=64, n_layers=5, n_heads=4, n_kv_heads=4, use_fp4=True, hp_tail=1)
    fp4_at = [cfg.use_fp4 and not (i == 0 or i >= cfg.n_layers - cfg.hp_tail) for i in range(cfg.n_layers)]
    assert fp4_at == [False, True, True, True, False]


def test_schedule_and_sampler():
    assert lr_at(0, 6e-4, 15, 300) == 0.0 and abs(lr_at(15, 6e-4, 15, 300) - 6e-4) < 1e-12
    assert abs(lr_at(300, 6e-4, 15, 300) - 6e-5) < 1e-9          # decays to 10 %
    sample, entropy = zipf_sampler(1000, 1.1, 5, "cpu")
    x, y = sample(4, 32)
    assert x.shape == (4, 32) and torch.equal(x[:, 1:], y[:, :-1]) and 3.0 < entropy < 7.0
