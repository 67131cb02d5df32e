"""Qwen2 step on the GPU against the CPU oracle (oracle/qwen2_oracle.py: transformers Qwen2ForCausalLM + AdamW).
bf16 kernels with fp32 accumulation: rel 2e-2 on losses and parameter tensors (L2), as stated for the bf16 mode."""
import ctypes as C
import json
import pathlib

import numpy as np
import pytest
import torch

from oracle import qwen2_oracle as O
from sirius_b200 import ops
from sirius_b200._lib import call
from sirius_b200.gpt2_step import BgemmDescC
from sirius_b200.qwen2_step import GET_GRAD, Qwen2Step

pytestmark = pytest.mark.gpu
TINY = dict(n_layer=2, n_head=4, n_kv_head=2, hidden=128, intermediate=256, vocab=500)


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def test_forward_logits_and_first_step_gradients_match_the_oracle():
    B, S = 2, 128
    model = O.build_model(**TINY, seed=0)
    ids = O.make_tokens(B, S, TINY["vocab"], 1)[0]
    step = Qwen2Step(**TINY, max_batch=B, seq=S)
    step.load_state_dict(O.state_arrays(model))
    step.upload_tokens(ids)
    step.forward_only()
    assert rel(step.logits(), O.forward_logits(model, ids).reshape(B * S, -1)) < 2e-2
    loss_ref, grads = O.first_step_gradients(model, ids)
    step.forward_backward()
    assert abs(step.loss() - loss_ref) < 2e-2 * abs(loss_ref)
    top = max(float(np.linalg.norm(g)) for g in grads.values())
    bad = [(round(rel(step.get(n, GET_GRAD), g), 4), n) for n, g in grads.items()
           if np.linalg.norm(g) > 1e-3 * top and rel(step.get(n, GET_GRAD), g) >= 5e-2]
    assert not bad, sorted(bad)[-8:]
    assert ops.tc_status() == 0
    step.close()


def test_three_adamw_steps_track_the_oracle_and_repeat_bit_for_bit():
    B, S = 2, 128
    model = O.build_model(**TINY, seed=0)
    batches = O.make_tokens(B, S, TINY["vocab"], 3)
    losses_ref, final = O.train_steps(model, batches)

    def run():
        step = Qwen2Step(**TINY, max_batch=B, seq=S)
        step.load_state_dict(O.state_arrays(model))
        losses = [step.train_step(ids) for ids in batches]
        out = losses, {n: step.get(n) for n in final}
        step.close()
        return out

    losses, params = run()
    for a, b in zip(losses, losses_ref):
        assert abs(a - b) < 2e-2 * abs(b), (losses, losses_ref)
    lr, steps = 3e-4, len(batches)
    for n, v in final.items():
        if rel(params[n], v) < 2e-2:
            continue
        # AdamW turns a near-zero gradient's rounding noise into +-lr (the key bias has no true gradient)
        assert n.endswith(".bias"), (n, rel(params[n], v))
        assert np.abs(params[n] - v).max() <= 2 * lr * steps * 1.01, (n, np.abs(params[n] - v).max())
    losses2, params2 = run()
    assert losses2 == losses and all(np.array_equal(params2[n], params[n]) for n in params)
    assert ops.tc_status() == 0


@pytest.mark.parametrize("case", ["qwen2_tiny", "qwen2_05b_b4_s2048"])
def test_against_the_committed_golden_fixture(case):
    """Seeded weights and token ids against the digests the CPU oracle wrote (tests/golden/*.json): first-step
    loss, every first-step gradient tensor by norm, sampled entries and sketch distance (direction, not only
    size), the loss of every step, the AdamW update by direction and norm, the final parameters.
    qwen2_05b_b4_s2048 is the 0.5B shape (24 layers, hidden 896, 14/2 heads, vocabulary 151 936) at four
    sequences of 2048 tokens, the per-GPU batch of the benchmark configuration."""
    from parity import check_gradient_digests, check_update_digests
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / f"{case}.json").read_text())
    cfg, B, S, steps, ref = doc["config"], doc["batch"], doc["seq"], doc["steps"], doc["fp32"]
    model = O.build_model(**cfg, seed=doc["seed"])
    batches = O.make_tokens(B, S, cfg["vocab"], steps, seed=doc["seed"])
    step = Qwen2Step(**cfg, max_batch=B, seq=S)
    init = O.state_arrays(model)
    step.load_state_dict(init)
    del model
    losses = []
    for i, ids in enumerate(batches):
        step.upload_tokens(ids)
        step.forward_backward()
        if i == 0:
            assert abs(step.loss() - ref["loss0"]) < 2e-2 * abs(ref["loss0"])
            check_gradient_digests(lambda n: step.get(n, GET_GRAD), ref["grad0"], what=case)
        step.optimizer_step()
        losses.append(step.loss())
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (losses, ref["losses"])
    check_update_digests(step.get, init, ref["delta"], ref["final"], doc["optimizer"]["lr"], steps, what=case)
    assert ops.tc_status() == 0
    step.close()
