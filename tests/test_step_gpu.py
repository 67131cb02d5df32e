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
    """bf16 mode. The forward loss is compared directly (rel 2e-2). Gradients in reduced precision are
    far noisier than 2e-2 for any implementation (PyTorch's own bf16 autocast on CPU is 0.3-1.3 away
    from fp64 in per-tensor rel-L2 on these networks), so they are anchored: our distance to the fp64
    gradients may not exceed 1.5x that of PyTorch's bf16-autocast run of the same model, plus 2e-2."""
    ref = _oracle(arch, batch, image, 1)
    batches = O.make_batches(batch, 1, image)
    _, g_ac = O.first_step_gradients(O.build_model(arch, 0), batches[0], autocast_bf16=True)
    step = _new_step(arch, batch, image, "bf16")
    step.upload_batch(*batches[0])
    step.forward_backward(batch, batch)
    loss0 = step.loss()
    print("bf16 loss0", loss0, "oracle", ref["fp32"]["loss0"])
    assert abs(loss0 - ref["fp32"]["loss0"]) <= 2e-2 * abs(ref["fp32"]["loss0"])
    g64 = ref["fp64"]["grads"]
    ours = np.array([rel_l2(step.get(k, GET_GRAD), v) for k, v in g64.items()])
    auto = np.array([rel_l2(g_ac[k], v) for k, v in g64.items()])
    rms = lambda v: float(np.sqrt(np.mean(np.square(v))))
    print(f"bf16 gradient rel-L2 to fp64, rms over tensors: ours {rms(ours):.3e}, torch bf16 autocast {rms(auto):.3e}")
    assert rms(ours) <= 1.5 * rms(auto) + 2e-2
    step.optimizer_step()
    step.synchronize()
    assert ops.tc_status() == 0
    m_ac = O.build_model(arch, 0)
    O.train_steps(m_ac, batches, autocast_bf16=True)
    ac_final = O.state_arrays(m_ac)
    cat = lambda get: np.concatenate([np.asarray(get(k), np.float64).ravel() for k in ref["fp64"]["final"]])
    all_ref = cat(lambda k: ref["fp64"]["final"][k])
    e, e_ac = rel_l2(cat(step.get), all_ref), rel_l2(cat(lambda k: ac_final[k]), all_ref)
    print(f"bf16 parameters after one step, rel-L2 over the whole model: ours {e:.3e}, torch bf16 autocast {e_ac:.3e}")
    assert e <= 1.5 * e_ac + 2e-2


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_resnet152_c1_against_golden(dtype):
    """The reference's CPU-runnable case: ResNet-152, batch 16, 224x224, 3 SGD steps, against the fixture."""
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
        # three steps at lr 0.1 from random init diverge chaotically (the fixture's fp32 and fp64 runs
        # end 10% apart in loss), so beyond the first loss the bf16 run is held to the anchored bound
        # and the reduced-precision reference is PyTorch's bf16-autocast run recorded in the fixture
        ac = g["bf16_autocast"]
        l2_ours = np.sqrt(sum(float((step.get(k).astype(np.float64) ** 2).sum()) for k in g["fp64"]["final"]))
        l2_64 = np.sqrt(sum(d["l2"] ** 2 for d in g["fp64"]["final"].values()))
        l2_ac = np.sqrt(sum(d["l2"] ** 2 for d in ac["final"].values()))
        print("C1 bf16 whole-model parameter norm", l2_ours, "torch bf16 autocast", l2_ac, "fp64", l2_64)
        assert anchored_scalar(l2_ours, l2_ac, l2_64, factor=1.5, floor=5e-2)
        print("C1 torch bf16 autocast losses", ac["losses"])
        for a, bac, b64 in zip(losses, ac["losses"], g["fp64"]["losses"]):
            assert anchored_scalar(a, bac, b64, factor=1.5, floor=5e-2)


_TF_CACHE = {}


def _teacher_forced_oracle():
    """Three oracle SGD steps of ResNet-152 (batch 16, 224 x 224, the seeds of the committed fixture) on the
    host, with the state before and after every step."""
    if "rec" not in _TF_CACHE:
        torch.set_num_threads(os.cpu_count() or 1)
        model = O.build_model("resnet152", 0)
        _TF_CACHE["batches"] = O.make_batches(16, 3, 224)
        _TF_CACHE["rec"] = O.train_steps_recording_states(model, _TF_CACHE["batches"])
    return _TF_CACHE["rec"], _TF_CACHE["batches"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_resnet152_single_steps_from_the_oracles_state(dtype):
    """Teacher-forced steps 2 and 3 of the ResNet-152 fp32 configuration (batch 16, lr 0.1: a trajectory whose
    loss climbs 7 -> 15 -> 22 and amplifies any rounding difference of an earlier step). The step object is
    loaded with the oracle's parameters, BatchNorm buffers and SGD momentum before step k, runs that one step on
    the same batch, and is compared DIRECTLY (no anchoring on a third run) wherever the quantity is a continuous
    function of the inputs: the loss (1e-4 fp32, 2e-2 bf16), every BatchNorm running mean and variance after the
    step, and the update of the classifier (its gradient is softmax minus one-hot times the pooled features: no
    ReLU derivative in it). The rest of the update contains ReLU masks that flip on rounding noise in any
    implementation (the fixture's fp32 and fp64 oracles are 9e-2 apart per tensor in gradient), so all other
    parameters after the step are held to 5e-3 (fp32; measured 1.9e-3 and 6e-5 for the two steps) and 5e-2 (bf16)
    in relative L2 over the whole model."""
    rec, batches = _teacher_forced_oracle()
    loss_tol, tol = (1e-4, 1e-4) if dtype == "f32" else (2e-2, 2e-2)
    step = ResNetStep(arch="resnet152", max_batch=16, image=224, dtype=dtype)
    for k in (1, 2):
        r = rec[k]
        step.load_state_dict(r["before"])
        step.load_momentum(r["momentum"])
        step.upload_batch(*batches[k])
        step.forward_backward(16, 16)
        loss = step.loss()
        print(f"step {k} {dtype}: loss {loss:.6f}, oracle {r['loss']:.6f}")
        assert abs(loss - r["loss"]) <= loss_tol * abs(r["loss"]), (k, loss, r["loss"])
        step.optimizer_step()
        step.synchronize()
        # running mean: deviation relative to the layer's data scale (its running standard deviation; a mean can
        # be arbitrarily close to zero); running variance: relative deviation
        def stat_err(n, v):
            got = step.get(n).astype(np.float64)
            if n.endswith("running_var"):
                return rel_l2(got, v)
            std = np.sqrt(r["after"][n[:-len("running_mean")] + "running_var"].astype(np.float64))
            return float(np.linalg.norm(got - v) / max(np.linalg.norm(std), np.linalg.norm(v)))
        worst = max((stat_err(n, v), n) for n, v in r["after"].items()
                    if n.endswith("running_mean") or n.endswith("running_var"))
        print(f"step {k} {dtype}: worst BatchNorm running statistic deviation {worst}")
        assert worst[0] <= tol * (1 if dtype == "f32" else 1.5), worst
        for n in ("fc.weight", "fc.bias"):
            d_ref = r["after"][n].astype(np.float64) - r["before"][n]
            d_got = step.get(n).astype(np.float64) - r["before"][n]
            e = rel_l2(d_got, d_ref)
            print(f"step {k} {dtype}: {n} update rel-L2 {e:.3e}")
            # bf16: the logits of this diverging run have magnitude ~30, so their bf16 rounding (2^-8 relative,
            # ~0.1 absolute) moves the softmax probabilities, and with them this gradient, by ~10 %
            assert e <= (2e-4 if dtype == "f32" else 0.25), (k, n, e)
        names = [n for n in r["after"] if not n.startswith("fc.") and "running" not in n]
        cat = lambda get: np.concatenate([np.asarray(get(n), np.float64).ravel() for n in names])
        e_all = rel_l2(cat(step.get), cat(lambda n: r["after"][n]))
        e_upd = rel_l2(cat(step.get) - cat(lambda n: r["before"][n]), cat(lambda n: r["after"][n]) - cat(lambda n: r["before"][n]))
        print(f"step {k} {dtype}: all other parameters after the step rel-L2 {e_all:.3e} (their update {e_upd:.3e})")
        assert e_all <= (5e-3 if dtype == "f32" else 5e-2)
    assert ops.tc_status() == 0
    step.close()


def test_backward_overlap_is_bit_identical_and_repeatable():
    """The filter-gradient kernels run on a second stream beside the rest of backward, the filter
    transposes beside the next forward, and short kernels are launched early (programmatic dependent
    launch). None of that may change a bit: several optimizer steps with the overlap on, on again, and
    off give identical losses, weights and gradients."""
    arch, batch, image, steps = "resnet50", 16, 128, 4
    model = O.build_model(arch, 0)
    (im, lb), = O.make_batches(batch, 1, image)
    names = ("conv1.weight", "layer1.0.conv1.weight", "layer2.0.downsample.0.weight", "layer3.4.conv2.weight",
             "layer4.2.conv3.weight", "layer3.5.bn2.weight", "fc.weight", "fc.bias")

    def run(overlap):
        step = ResNetStep(layers=O.LAYERS[arch], max_batch=batch, image=image, dtype="bf16")
        step.load_state_dict(O.state_arrays(model))
        step.overlap_wgrad(overlap)
        step.upload_batch(im, lb)
        losses = []
        for _ in range(steps):
            step.forward_backward(batch, batch)
            step.optimizer_step()
            losses.append(step.loss())
        step.synchronize()
        out = (losses, [step.get(n).copy() for n in names], [step.get(n, GET_GRAD).copy() for n in names])
        step.close()
        return out

    ref = run(True)
    assert all(np.isfinite(ref[0]))
    for overlap in (True, False):
        got = run(overlap)
        assert got[0] == ref[0]
        for a, b in zip(got[1] + got[2], ref[1] + ref[2]):
            assert np.array_equal(a, b)
    assert ops.tc_status() == 0


def test_gradient_buckets_tile_the_buffer_and_fire_when_final():
    """The buckets cover the flat gradient buffer exactly once, last layers first, and a stream that waits
    for a bucket's event sees that bucket's final values (it copies them while backward is still running)."""
    arch, batch, image = "resnet50", 16, 128
    model = O.build_model(arch, 0)
    (im, lb), = O.make_batches(batch, 1, image)
    step = ResNetStep(layers=O.LAYERS[arch], max_batch=batch, image=image, dtype="bf16")
    step.load_state_dict(O.state_arrays(model))
    ptr, n = step.grad_buffer()
    buckets = step.grad_buckets()
    assert len(buckets) >= 2
    assert buckets[0][0] + buckets[0][1] == n and buckets[-1][0] == 0
    for (o0, c0), (o1, c1) in zip(buckets, buckets[1:]):
        assert o1 + c1 == o0 and c0 >= (25 << 18)

    class Buf:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}
    grad = torch.as_tensor(Buf(), device="cuda:0")
    comm = torch.cuda.Stream()
    for _ in range(2):
        step.upload_batch(im, lb)
        grad.zero_()
        torch.cuda.synchronize()
        step.forward_backward(batch, batch)
        copies = []
        for b, (off, cnt) in enumerate(buckets):
            step.wait_grad_bucket(b, comm.cuda_stream)
            with torch.cuda.stream(comm):
                copies.append(grad[off:off + cnt].clone())
        done = torch.cuda.Event()
        done.record(comm)
        step.wait_event(done.cuda_event)
        step.synchronize()
        torch.cuda.synchronize()
        for (off, cnt), c in zip(buckets, copies):
            assert torch.equal(c, grad[off:off + cnt])
        assert float(grad.abs().sum()) > 0
    step.close()
