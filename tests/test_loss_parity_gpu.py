"""Loss parity with the reference recipe on the reference's own convergence task.

The addition task of nvfp4_validate.py:239-282 / nvfp4_train.py:159-185 (same model, data split,
optimizer and schedule) is trained three ways from the same seed:
  * real FP4: every block linear an FP4Linear on the sm_100a kernels (hp_tail 0),
  * reference recipe: the same model with the reference's fake-quant simulator
    (`_NVFP4LinearFn`, nvfp4_validate.py:104-140, restated in oracle/nvfp4_sim.py and pinned to
    golden vectors) in place of the FP4 linears, run with torch ops on the GPU,
  * bf16.
Held-out loss is compared at matched steps; the bound is the benchmark's: |difference| <= 0.02, asserted
from step 200 on (the last three evaluations and their mean).  Before that the task itself is
noisier than the bound: GPU training is not bit-reproducible (atomics in attention backward), and two
bf16 runs of this very script read 1.4004 and 1.4507 at step 150 while the loss still falls by about
0.01 per step, so the earlier evaluations only get a loose bound.  Measured on a B200 (real FP4 /
reference recipe / bf16): step 50 1.5764 / 1.5696 / 1.5790, step 100 1.4770 / 1.4978 / 1.4430, step 150
1.4011 / 1.4159 / 1.4507, step 200 1.3822 / 1.3916 / 1.3748, step 250 1.3688 / 1.3717 / 1.3645, step 300
1.3630 / 1.3682 / 1.3610."""
import pytest
import torch

pytestmark = pytest.mark.gpu

STEPS, EVERY = 300, 50
TOL = 0.02
FIRST_TIGHT_STEP = 200


def test_fp4_loss_tracks_the_reference_recipe_and_bf16():
    import nvfp4_sm120_b200 as Q
    from nvfp4_sm120_b200 import addition
    from oracle import nvfp4_sim as S

    Q.set_amortize(True)
    try:
        quiet = lambda *_: None
        fp4 = addition.run("fp4-all", STEPS, use_fp4=True, hp_tail=0, log=quiet, eval_every=EVERY)
        sim = addition.run("reference-recipe", STEPS, use_fp4=True, hp_tail=0, log=quiet, eval_every=EVERY,
                           linear_factory=lambda cin, cout: S.SimLinear(cin, cout, sr=True, rht=True, device="cuda"))
        bf16 = addition.run("bf16", STEPS, use_fp4=False, log=quiet, eval_every=EVERY)
    finally:
        Q.set_amortize(False)
    assert not fp4["diverged"] and not sim["diverged"] and not bf16["diverged"]
    assert [h["step"] for h in fp4["history"]] == [h["step"] for h in sim["history"]] == list(range(EVERY, STEPS + 1, EVERY))
    rows = []
    for a, b, c in zip(fp4["history"], sim["history"], bf16["history"]):
        rows.append((a["step"], a["val"], b["val"], c["val"]))
    print("step, val loss real FP4 / reference recipe / bf16:", rows)
    for step, v_fp4, v_sim, v_bf16 in rows:
        tol = TOL if step >= FIRST_TIGHT_STEP else 4 * TOL
        assert abs(v_fp4 - v_sim) <= tol, (step, v_fp4, v_sim)
        assert abs(v_fp4 - v_bf16) <= tol, (step, v_fp4, v_bf16)
    tail = [r for r in rows if r[0] >= FIRST_TIGHT_STEP]
    mean = lambda i: sum(r[i] for r in tail) / len(tail)
    assert abs(mean(1) - mean(2)) <= TOL and abs(mean(1) - mean(3)) <= TOL
    assert Q.gemm_status() == 0
