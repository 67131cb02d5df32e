"""GPT-2 step on the GPU against PyTorch: single operators against torch fp32 on the same (bf16-rounded)
inputs, the whole step against the CPU oracle (oracle/gpt2_oracle.py: transformers.GPT2LMHeadModel + AdamW).
Tolerances: bf16 kernels with fp32 accumulation, rel 2e-2 on losses and parameter tensors (L2), as stated for
the bf16 mode of the training step."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import gpt2_oracle as O
from sirius_b200 import ops
from sirius_b200._lib import call
from sirius_b200.gpt2_step import GET_GRAD, BgemmDescC, Gpt2Step

pytestmark = pytest.mark.gpu
P = lambda t: C.c_void_p(t.data_ptr())


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bf(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("S,D,H,B", [(128, 64, 3, 2), (256, 32, 2, 1), (72, 64, 1, 1)])
def test_bgemm_heads_in_place_causal_and_trimmed(S, D, H, B):
    Cm = H * D
    qkv = bf((B * S, 3 * Cm), 0.5, 1)
    q = qkv[:, :Cm].float().view(B, S, H, D).permute(0, 2, 1, 3)
    k = qkv[:, Cm:2 * Cm].float().view(B, S, H, D).permute(0, 2, 1, 3)
    ref = torch.tril(q @ k.transpose(-1, -2) * 0.125)
    out = torch.zeros(B * H, S, S, dtype=torch.bfloat16, device="cuda")
    d = BgemmDescC(S, S, D, H, B, 3 * Cm, D, S * 3 * Cm, 3 * Cm, D, S * 3 * Cm, S, S * S, H * S * S, 0.125, 1, 0)
    call("srt_bgemm", C.byref(d), P(qkv), C.c_void_p(qkv.data_ptr() + 2 * Cm), P(out), None)
    torch.cuda.synchronize()
    got = torch.tril(out.float().view(B, H, S, S))      # tiles above the diagonal are not written
    assert rel(got.cpu(), ref.cpu()) < 1e-2
    # P V with the reduction trimmed at the diagonal, output scattered back into [tokens][hidden]
    prob = torch.softmax(ref.masked_fill(torch.triu(torch.ones(S, S, device="cuda"), 1).bool(), -1e30), -1)
    pm = prob.to(torch.bfloat16).contiguous().view(B * H, S, S)
    vt = qkv[:, 2 * Cm:].view(B, S, H, D).permute(0, 2, 3, 1).contiguous()          # [B][H][D][S]
    att = torch.zeros(B * S, Cm, dtype=torch.bfloat16, device="cuda")
    d2 = BgemmDescC(S, D, S, H, B, S, S * S, H * S * S, S, D * S, H * D * S, Cm, D, S * Cm, 1.0, 0, 1)
    call("srt_bgemm", C.byref(d2), P(pm), P(vt), P(att), None)
    torch.cuda.synchronize()
    v = qkv[:, 2 * Cm:].float().view(B, S, H, D).permute(0, 2, 1, 3)
    ref2 = (pm.float().view(B, H, S, S) @ v).permute(0, 2, 1, 3).reshape(B * S, Cm)
    assert rel(att.float().cpu(), ref2.cpu()) < 1e-2
    # A zero below the diagonal (a transposed lower-triangular matrix): reduction starts at the diagonal
    pt = pm.view(B, H, S, S).transpose(-1, -2).contiguous().view(B * H, S, S)
    d3 = BgemmDescC(S, D, S, H, B, S, S * S, H * S * S, S, D * S, H * D * S, Cm, D, S * Cm, 1.0, 0, 2)
    att.zero_()
    call("srt_bgemm", C.byref(d3), P(pt), P(vt), P(att), None)
    torch.cuda.synchronize()
    ref3 = (pt.float().view(B, H, S, S) @ v).permute(0, 2, 1, 3).reshape(B * S, Cm)
    assert rel(att.float().cpu(), ref3.cpu()) < 1e-2
    assert ops.tc_status() == 0


def test_layernorm_forward_backward():
    rows, Cm = 300, 768
    x, dy, add = bf((rows, Cm), 2.0, 1), bf((rows, Cm), 1.0, 2), bf((rows, Cm), 1.0, 3)
    gamma = (torch.randn(Cm) * 0.5 + 1).cuda()
    beta = torch.randn(Cm).cuda()
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    call("srt_layernorm_fwd", P(x), P(gamma), P(beta), P(y), P(mean), P(rstd), rows, Cm, 1e-5, None)
    xr = x.float().requires_grad_(True)
    gr, br = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (Cm,), gr, br, 1e-5)
    assert rel(y.float().cpu(), yr.detach().cpu()) < 5e-3
    yr.backward(dy.float())
    nbytes = ops._lib.lib().srt_layernorm_bwd_scratch_bytes(Cm)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    dx, dgm, dbt = torch.empty_like(x), torch.empty(Cm, device="cuda"), torch.empty(Cm, device="cuda")
    call("srt_layernorm_bwd", P(dy), P(x), P(gamma), P(mean), P(rstd), P(add), P(dx), P(dgm), P(dbt), rows, Cm,
         P(scratch), nbytes, None)
    torch.cuda.synchronize()
    assert rel(dx.float().cpu(), (xr.grad + add.float()).cpu()) < 5e-3
    assert rel(dgm.cpu(), gr.grad.cpu()) < 2e-3 and rel(dbt.cpu(), br.grad.cpu()) < 1e-4


def test_gelu_softmax_transpose_cross_entropy():
    n = 8 * 1000
    x, dy = bf((n,), 2.0, 1), bf((n,), 1.0, 2)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    call("srt_gelu_fwd", P(x), P(y), n, None)
    call("srt_gelu_bwd", P(dy), P(x), P(dx), n, None)
    xr = x.float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr, approximate="tanh")
    yr.backward(dy.float())
    assert rel(y.float().cpu(), yr.detach().cpu()) < 5e-3 and rel(dx.float().cpu(), xr.grad.cpu()) < 5e-3
    # causal softmax, in place, garbage above the diagonal must not matter
    Z, S = 5, 72
    s = bf((Z, S, S), 3.0, 3)
    mask = torch.triu(torch.ones(S, S, device="cuda"), 1).bool()
    sr = s.float().masked_fill(mask, float("-inf")).requires_grad_(True)
    pr = torch.softmax(sr, -1)
    s2 = s.clone().masked_fill(mask, 1e4)
    call("srt_causal_softmax_fwd", P(s2), Z, S, None)
    assert rel(s2.float().cpu(), pr.detach().cpu()) < 5e-3 and float(s2.float().masked_select(mask).abs().max()) == 0.0
    dp = bf((Z, S, S), 1.0, 4)
    pr.backward(dp.float())
    dpm = dp.clone().masked_fill(mask, 1e4)
    call("srt_causal_softmax_bwd", P(s2), P(dpm), Z, S, None)
    assert rel(dpm.float().cpu(), sr.grad.cpu()) < 2e-2 and float(dpm.float().masked_select(mask).abs().max()) == 0.0
    # batched transpose of head slices
    B, Sq, H, D = 2, 40, 3, 16
    qkv = bf((B * Sq, 3 * H * D), 1.0, 5)
    out = torch.empty(B * H, D, Sq, dtype=torch.bfloat16, device="cuda")
    call("srt_batched_transpose", C.c_void_p(qkv.data_ptr() + 2 * (H * D)), P(out), Sq, D, 3 * H * D, D, Sq * 3 * H * D, H, B, None)
    ref = qkv[:, H * D:2 * H * D].view(B, Sq, H, D).permute(0, 2, 3, 1).reshape(B * H, D, Sq)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    # next-token cross entropy over a padded vocabulary
    rows, V, ld = 37, 1000, 1024
    lg = bf((rows, ld), 2.0, 6)
    labels = torch.randint(0, V, (rows,), dtype=torch.int32)
    labels[5] = -1
    lr_ = lg.float()[:, :V].requires_grad_(True)
    valid = labels >= 0
    loss = torch.nn.functional.cross_entropy(lr_[valid.cuda()], labels[valid].long().cuda(), reduction="sum")
    loss.backward()
    row_loss = torch.empty(rows, device="cuda")
    lab = labels.cuda()
    call("srt_lm_cross_entropy", P(lg), P(lab), rows, V, ld, 0.5, P(row_loss), None)
    torch.cuda.synchronize()
    assert abs(float(row_loss.sum()) - float(loss)) < 2e-3 * float(loss)
    assert rel(lg.float()[:, :V].cpu(), (lr_.grad * 0.5).cpu()) < 1e-2
    assert float(lg.float()[:, V:].abs().max()) == 0.0 and float(lg.float()[5].abs().max()) == 0.0


CFG = dict(n_layer=2, n_head=4, d_model=128, vocab=500, ctx=64)


def test_forward_logits_and_first_step_gradients_match_the_oracle():
    B, S = 2, 64
    model = O.build_model(**CFG, seed=0)
    ids = O.make_tokens(B, S, CFG["vocab"], 1)[0]
    step = Gpt2Step(**CFG, max_batch=B, seq=S)
    step.load_state_dict(O.state_arrays(model))
    step.upload_tokens(ids)
    step.forward_only()
    assert rel(step.logits(), O.forward_logits(model, ids).reshape(B * S, -1)) < 2e-2
    loss_ref, grads = O.first_step_gradients(model, ids)
    step.forward_backward()
    assert abs(step.loss() - loss_ref) < 2e-2 * abs(loss_ref)
    worst = max((rel(step.get(n, GET_GRAD), g), n) for n, g in grads.items())
    assert worst[0] < 5e-2, worst
    assert ops.tc_status() == 0
    step.close()


def test_three_adamw_steps_track_the_oracle():
    B, S = 2, 64
    model = O.build_model(**CFG, seed=0)
    batches = O.make_tokens(B, S, CFG["vocab"], 3)
    losses_ref, final = O.train_steps(model, batches)
    step = Gpt2Step(**CFG, max_batch=B, seq=S)
    step.load_state_dict(O.state_arrays(model))
    losses = [step.train_step(ids) for ids in batches]
    for a, b in zip(losses, losses_ref):
        assert abs(a - b) < 2e-2 * abs(b), (losses, losses_ref)
    # AdamW divides by sqrt(v): where the true gradient is zero or nearly so (the key third of c_attn.bias:
    # softmax does not see a constant added to every key; biases that start at zero) the update is the sign of
    # rounding noise times lr, in the oracle as much as here. Such tensors are held to the bound AdamW itself
    # gives, |a - b| <= 2 * lr * steps; every weight matrix and table must meet the relative tolerance.
    lr, steps = 3e-4, len(batches)
    for n, v in final.items():
        got = step.get(n)
        if rel(got, v) < 2e-2:
            continue
        assert n.endswith(".bias"), (n, rel(got, v))
        assert np.abs(got - v).max() <= 2 * lr * steps * 1.01, (n, np.abs(got - v).max())
    # and the step is repeatable bit for bit
    step2 = Gpt2Step(**CFG, max_batch=B, seq=S)
    step2.load_state_dict(O.state_arrays(model))
    assert [step2.train_step(ids) for ids in batches] == losses
    assert np.array_equal(step2.get("transformer.wte.weight"), step.get("transformer.wte.weight"))
    assert ops.tc_status() == 0
    step.close(); step2.close()


@pytest.mark.parametrize("case", ["gpt2_tiny", "gpt2_c4"])
def test_against_the_committed_golden_fixture(case):
    """Seeded weights and token ids, compared with the digests the CPU oracle wrote (tests/golden/*.json):
    the first-step loss (2e-2); every first-step gradient tensor by norm, by sampled entries and by the +-1
    sketch that bounds its relative L2 distance to the oracle's (5e-2: direction, not only size); the loss of
    every step (2e-2); the update the AdamW steps made, by direction and norm, and the final parameters.
    gpt2_c4 is GPT-2 small at batch 8 x 1024 tokens."""
    import json
    import pathlib
    from parity import check_gradient_digests, check_update_digests
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / f"{case}.json").read_text())
    cfg, B, S, steps = doc["config"], doc["batch"], doc["seq"], doc["steps"]
    model = O.build_model(**cfg, seed=doc["seed"])
    batches = O.make_tokens(B, S, cfg["vocab"], steps, seed=doc["seed"])
    step = Gpt2Step(**cfg, max_batch=B, seq=S)
    init = O.state_arrays(model)
    step.load_state_dict(init)
    del model
    ref = doc["fp32"]
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


@pytest.mark.parametrize("B,S,max_batch", [(1, 72, 3), (3, 40, 3)])
def test_ragged_sizes_partial_batches_and_short_sequences(B, S, max_batch):
    """Fewer sequences than the step was created for, sequence lengths that are not a multiple of the 128-row tile
    (so every GEMM has a ragged last tile and attention a partial diagonal block), a vocabulary that is not a
    multiple of 64: same parity as the regular case."""
    cfg = dict(n_layer=2, n_head=2, d_model=64, vocab=333, ctx=80)
    model = O.build_model(**cfg, seed=3)
    ids = O.make_tokens(B, S, cfg["vocab"], 1, seed=5)[0]
    step = Gpt2Step(**cfg, max_batch=max_batch, seq=S)
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


def test_gradient_buckets_tile_the_buffer_and_fire_when_final():
    """As for the ResNet executor: the buckets cover the flat gradient buffer once, last layers first, and a stream
    that waits for a bucket's event copies that bucket's final values while backward is still running."""
    cfg = dict(n_layer=6, n_head=4, d_model=512, vocab=5000, ctx=128)      # ~3 M gradients per layer: several buckets
    B, S = 2, 128
    model = O.build_model(**cfg, seed=0)
    ids = O.make_tokens(B, S, cfg["vocab"], 1)[0]
    step = Gpt2Step(**cfg, max_batch=B, seq=S)
    step.load_state_dict(O.state_arrays(model))
    ptr, n = step.grad_buffer()
    buckets = step.grad_buckets()
    assert len(buckets) >= 2 and buckets[0][0] + buckets[0][1] == n and buckets[-1][0] == 0
    for (o0, c0), (o1, c1) in zip(buckets, buckets[1:]):
        assert o1 + c1 == o0

    class Buf:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}
    grad = torch.as_tensor(Buf(), device="cuda:0")
    comm = torch.cuda.Stream()
    step.upload_tokens(ids)
    for _ in range(2):
        grad.zero_()
        torch.cuda.synchronize()
        step.forward_backward()
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
