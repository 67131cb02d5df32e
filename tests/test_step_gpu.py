"""Whole-step parity on the GPU: the CUDA training step, driven through the C ABI, against the
CPU oracle (stock torchvision + PyTorch; fp32 = the reference's path, fp64 = exact anchor) on
identical seeded weights and inputs, and against the committed golden fixtures.

Tolerances: the forward loss of the first step is compared directly (rel 1e-4 in fp32 mode, 2e-2 in
bf16 mode). Everything that depends on gradients uses the fp64-anchored criterion of
tests/parity.py, because the reference's fp32 path is itself only that close to exact."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import resnet_oracle as O
from parity import anchored_scalar, check_digest, check_tensors, rel_l2
from sirius_b200 import ops
from sirius_b200.step import GET_GRAD, ResNetStep

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gold(name):
    with open(os.path.join(GOLD, name + ".json")) as f:
        return json.load(f)


def _new_step(arch, batch, image, dtype):
    model = O.build_model(arch, 0)
    step = ResNetStep(layers=O.LAYERS[arch], max_batch=batch, image=image, dtype=dtype)
    step.load_state_dict(O.state_arrays(model))
    return step


def _run_steps(step, batches, batch, micro=1):
    losses = []
    for images, labels in batches:
        total = 0.0
        for im, lb in zip(images.chunk(micro), labels.chunk(micro)):
            b = step.upload_batch(im.contiguous(), lb.contiguous())
            step.forward_backward(b, batch)
            if micro > 1:
                step.accumulate()
            total += step.loss()
        step.optimizer_step()
        losses.append(total)
    step.synchronize()
    assert ops.tc_status() == 0
    return losses


def _oracle(arch, batch, image, steps, micro=1):
    torch.set_num_threads(os.cpu_count() or 1)
    out = {}
    for key, dbl in (("fp32", False), ("fp64", True)):
        model = O.build_model(arch, 0, double=dbl)
        batches = O.make_batches(batch, steps, image, double=dbl)
        loss0, grads = O.first_step_gradients(model, batches[0])
        losses = O.train_steps(model, batches, micro_batches=micro)
        out[key] = {"loss0": loss0, "grads": grads, "losses": losses, "final": O.state_arrays(model)}
    return out


@pytest.mark.parametrize("arch,batch,image", [("resnet14", 8, 64), ("resnet50", 4, 64)])
def test_fp32_step_matches_oracle(arch, batch, image):
    steps = 2
    ref = _oracle(arch, batch, image, steps)
    step = _new_step(arch, batch, image, "f32")
    batches = O.make_batches(batch, steps, image)
    # first step: forward loss (direct) and gradients (anchored)
    step.upload_batch(*batches[0])
    step.forward_backward(batch, batch)
    loss0 = step.loss()
    assert abs(loss0 - ref["fp32"]["loss0"]) <= 1e-4 * abs(ref["fp32"]["loss0"])
    check_tensors(lambda k: step.get(k, GET_GRAD), ref["fp32"]["grads"], ref["fp64"]["grads"],
                  what=f"{arch} first-step gradients")
    # full trajectory from a fresh object
    step = _new_step(arch, batch, image, "f32")
    losses = _run_steps(step, batches, batch)
    print("losses", losses, "oracle fp32", ref["fp32"]["losses"], "fp64", ref["fp64"]["losses"])
    for a, b32, b64 in zip(losses, ref["fp32"]["losses"], ref["fp64"]["losses"]):
        assert anchored_scalar(a, b32, b64)
    check_tensors(step.get, ref["fp32"]["final"], ref["fp64"]["final"], what=f"{arch} final parameters")
    g = _gold(f"{arch}_small")
    check_digest(step.get, g["fp32"]["final"], g["fp64"]["final"], what=f"{arch} vs golden digest")


def test_fp32_micro_batches_follow_scale_loss_semantics():
    """Two accumulated micro-batches, losses scaled by micro/global, one optimizer step."""
    arch, batch, image = "resnet14", 8, 64
    ref = _oracle(arch, batch, image, 1, micro=2)
    step = _new_step(arch, batch, image, "f32")
    losses = _run_steps(step, O.make_batches(batch, 1, image), batch, micro=2)
    assert anchored_scalar(losses[0], ref["fp32"]["losses"][0], ref["fp64"]["losses"][0])
    check_tensors(step.get, ref["fp32"]["final"], ref["fp64"]["final"], what="micro-batch final parameters")


@pytest.mark.parametrize("arch,batch,image", [("resnet14", 8, 64), ("resnet50", 4, 64)])
def test_bf16_step_tracks_oracle(arch, batch, image):
    ref = _oracle(arch, batch, image, 1)
    step = _new_step(arch, batch, image, "bf16")
    batches = O.make_batches(batch, 1, image)
    step.upload_batch(*batches[0])
    step.forward_backward(batch, batch)
    loss0 = step.loss()
    print("bf16 loss0", loss0, "oracle", ref["fp32"]["loss0"])
    assert abs(loss0 - ref["fp32"]["loss0"]) <= 2e-2 * abs(ref["fp32"]["loss0"])
    errs = {k: rel_l2(step.get(k, GET_GRAD), v) for k, v in ref["fp64"]["grads"].items()}
    worst = max(errs, key=errs.get)
    med = float(np.median(list(errs.values())))
    print(f"bf16 gradient rel-L2 to fp64: median {med:.3e}, worst {errs[worst]:.3e} at {worst}")
    # bf16 operands carry 2^-9 relative rounding per element and flip more ReLU masks than fp32
    # does; the bound is the task's 2e-2 or three times the reference's own distance from exact.
    ref_err = {k: rel_l2(ref["fp32"]["grads"][k], v) for k, v in ref["fp64"]["grads"].items()}
    assert med <= max(2e-2, 3 * float(np.median(list(ref_err.values()))))
    step.optimizer_step()
    step.synchronize()
    assert ops.tc_status() == 0
    all_ours = np.concatenate([step.get(k).ravel() for k in ref["fp64"]["final"]])
    all_ref = np.concatenate([np.asarray(v).ravel() for v in ref["fp64"]["final"].values()])
    e = rel_l2(all_ours, all_ref)
    print("bf16 parameters after one step, rel-L2 over the whole model:", e)
    assert e <= 2e-2


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_resnet152_c1_against_golden(dtype):
    """BASELINE config 1: ResNet-152, batch 16, 224x224, 3 SGD steps, against the fixture."""
    arch, batch, image, steps = "resnet152", 16, 224, 3
    g = _gold("resnet152_c1")
    step = _new_step(arch, batch, image, dtype)
    losses = _run_steps(step, O.make_batches(batch, steps, image), batch)
    print(f"C1 {dtype} losses", losses, "oracle fp32", g["fp32"]["losses"], "fp64", g["fp64"]["losses"])
    tol0 = 1e-4 if dtype == "f32" else 2e-2
    assert abs(losses[0] - g["fp32"]["losses"][0]) <= tol0 * abs(g["fp32"]["losses"][0])
    if dtype == "f32":
        for a, b32, b64 in zip(losses, g["fp32"]["losses"], g["fp64"]["losses"]):
            assert anchored_scalar(a, b32, b64)
        check_digest(step.get, g["fp32"]["final"], g["fp64"]["final"], what="C1 fp32 vs golden digest")
    else:
        l2_ours = np.sqrt(sum(float((step.get(k).astype(np.float64) ** 2).sum()) for k in g["fp64"]["final"]))
        l2_ref = np.sqrt(sum(d["l2"] ** 2 for d in g["fp64"]["final"].values()))
        print("C1 bf16 whole-model parameter norm", l2_ours, "fp64 oracle", l2_ref)
        assert abs(l2_ours - l2_ref) <= 2e-2 * l2_ref
        assert all(np.isfinite(losses))
