"""Swin step on the GPU against the CPU oracle (oracle/swin_oracle.py: torchvision SwinTransformer + AdamW).
bf16 kernels with fp32 accumulation: rel 2e-2 on losses and parameter tensors (L2), as stated for the bf16 mode."""
import json
import pathlib

import numpy as np
import pytest
import torch

from oracle import swin_oracle as O
from sirius_b200 import ops
from sirius_b200.swin_step import GET_GRAD, SwinStep

pytestmark = pytest.mark.gpu
TINY = dict(image=224, patch=4, embed=32, depths=(2, 2, 2, 2), heads=(2, 4, 8, 16), window=7, num_classes=40)


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def test_forward_logits_and_first_step_gradients_match_the_oracle():
    B = 2
    model = O.build_model(**TINY, seed=0)
    batch = O.make_batches(B, 1, TINY["image"], TINY["num_classes"])[0]
    step = SwinStep(**TINY, max_batch=B)
    step.load_state_dict(O.state_arrays(model))
    step.upload_batch(batch[0].contiguous(), batch[1].contiguous())
    step.forward_only()
    ref = O.forward_logits(model, batch[0])
    assert rel(step.logits(), ref) < 3e-2, rel(step.logits(), ref)
    loss_ref, grads = O.first_step_gradients(model, batch)
    step.forward_backward()
    assert abs(step.loss() - loss_ref) < 2e-2 * abs(loss_ref)
    top = max(float(np.linalg.norm(g)) for g in grads.values())
    bad = [(round(rel(step.get(n, GET_GRAD), g), 4), n) for n, g in grads.items()
           if np.linalg.norm(g) > 1e-3 * top and rel(step.get(n, GET_GRAD), g) >= 6e-2]
    assert not bad, sorted(bad)[-8:]
    assert ops.tc_status() == 0
    step.close()


def test_three_adamw_steps_track_the_oracle_and_repeat_bit_for_bit():
    B = 2
    model = O.build_model(**TINY, seed=0)
    batches = O.make_batches(B, 3, TINY["image"], TINY["num_classes"])
    losses_ref, final = O.train_steps(model, batches)

    def run():
        step = SwinStep(**TINY, max_batch=B)
        step.load_state_dict(O.state_arrays(model))
        losses = [step.train_step(im.contiguous(), lb.contiguous()) for im, lb in batches]
        out = losses, {n: step.get(n) for n in final}
        step.close()
        return out

    losses, params = run()
    for a, b in zip(losses, losses_ref):
        assert abs(a - b) < 2e-2 * abs(b), (losses, losses_ref)
    lr, steps = 1e-3, len(batches)
    for n, v in final.items():
        if rel(params[n], v) < 2e-2:
            continue
        # AdamW turns a near-zero gradient's rounding noise into +-lr; such entries are bounded by 2*lr*steps
        assert np.abs(params[n] - v).max() <= 2 * lr * steps * 1.01, (n, rel(params[n], v), np.abs(params[n] - v).max())
    losses2, params2 = run()
    assert losses2 == losses and all(np.array_equal(params2[n], params[n]) for n in params)
    assert ops.tc_status() == 0


@pytest.mark.parametrize("case", ["swin_tiny", "swin_b_c3"])
def test_against_the_committed_golden_fixture(case):
    """Seeded weights and inputs against the digests the CPU oracle wrote (tests/golden/*.json): first-step loss,
    every first-step gradient tensor by norm, sampled entries and sketch distance (direction, not only size), the
    loss of every step, the AdamW update by direction and norm, the final parameters. swin_b_c3 is Swin-B at 32
    images of 224 x 224."""
    from parity import check_gradient_digests, check_update_digests
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / f"{case}.json").read_text())
    cfg = {k: tuple(v) if isinstance(v, list) else v for k, v in doc["config"].items()}
    B, steps, ref = doc["batch"], doc["steps"], doc["fp32"]
    model = O.build_model(**cfg, seed=doc["seed"])
    batches = O.make_batches(B, steps, cfg["image"], cfg["num_classes"], seed=doc["seed"])
    step = SwinStep(**cfg, max_batch=B)
    init = O.state_arrays(model)
    step.load_state_dict(init)
    del model
    losses = []
    for i, (im, lb) in enumerate(batches):
        step.upload_batch(im.contiguous(), lb.contiguous())
        step.forward_backward()
        if i == 0:
            assert abs(step.loss() - ref["loss0"]) < 2e-2 * abs(ref["loss0"])
            check_gradient_digests(lambda n: step.get(n, GET_GRAD), ref["grad0"], tol=6e-2, what=case)
        step.optimizer_step()
        losses.append(step.loss())
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (losses, ref["losses"])
    check_update_digests(step.get, init, ref["delta"], ref["final"], doc["optimizer"]["lr"], steps, what=case)
    assert ops.tc_status() == 0
    step.close()


def test_partial_batch_on_a_larger_step_object():
    """A micro-batch smaller than max_batch (what the dynamic batch manager hands out after an adjust)."""
    B = 1
    model = O.build_model(**TINY, seed=0)
    batch = O.make_batches(B, 1, TINY["image"], TINY["num_classes"], seed=7)[0]
    step = SwinStep(**TINY, max_batch=3)
    step.load_state_dict(O.state_arrays(model))
    step.upload_batch(batch[0].contiguous(), batch[1].contiguous())
    step.forward_only()
    assert rel(step.logits(), O.forward_logits(model, batch[0])) < 3e-2
    loss_ref, grads = O.first_step_gradients(model, batch)
    step.forward_backward()
    assert abs(step.loss() - loss_ref) < 2e-2 * abs(loss_ref)
    top = max(float(np.linalg.norm(g)) for g in grads.values())
    bad = [(round(rel(step.get(n, GET_GRAD), g), 4), n) for n, g in grads.items()
           if np.linalg.norm(g) > 1e-3 * top and rel(step.get(n, GET_GRAD), g) >= 6e-2]
    assert not bad, sorted(bad)[-8:]
    assert ops.tc_status() == 0
    step.close()
