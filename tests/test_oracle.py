"""CPU suite: the oracle reproduces the committed golden fixtures (same build container), and the
fixtures carry the fp64 anchor. Small cases only, so the suite stays fast."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import resnet_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", ["resnet14_small", "resnet50_small"])
def test_oracle_reproduces_golden(name):
    with open(os.path.join(GOLD, name + ".json")) as f:
        g = json.load(f)
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(g["arch"], g["seed"])
    batches = O.make_batches(g["batch"], g["steps"], g["image"])
    loss0, grads = O.first_step_gradients(model, batches[0])
    losses = O.train_steps(model, batches)
    assert loss0 == pytest.approx(g["fp32"]["loss0"], rel=1e-6)
    # later steps inherit ReLU-flip noise from thread-count dependent reduction order
    assert losses[0] == pytest.approx(g["fp32"]["losses"][0], rel=1e-6)
    dig = O.summarize(O.state_arrays(model), samples=4)
    for k, d in g["fp32"]["final"].items():
        assert dig[k]["l2"] == pytest.approx(d["l2"], rel=5e-2, abs=1e-6), k
    gd = O.summarize(grads, samples=4)
    rels = [abs(gd[k]["l2"] - d["l2"]) / (d["l2"] + 1e-30) for k, d in g["fp32"]["grad0"].items()]
    assert np.median(rels) < 5e-2


def test_c1_fixture_is_complete():
    with open(os.path.join(GOLD, "resnet152_c1.json")) as f:
        g = json.load(f)
    assert g["arch"] == "resnet152" and g["batch"] == 16 and g["image"] == 224 and g["steps"] == 3
    for prec in ("fp32", "fp64"):
        assert len(g[prec]["losses"]) == 3 and len(g[prec]["final"]) == len(g["fp64"]["final"])
    # 155 conv + fc weights, 155 BN x (weight, bias, mean, var), fc bias
    assert len(g["fp32"]["final"]) == 155 + 1 + 155 * 4 + 1
    # the reference's fp32 path is measurably inexact: the fixture records by how much
    assert abs(g["fp32"]["losses"][2] - g["fp64"]["losses"][2]) > 1e-2


def test_gpt2_oracle_reproduces_the_committed_fixture():
    """The GPT-2 oracle is pinned on its own committed output (the reference holds no vectors for this model):
    same seeds, same losses and parameter digests as tests/golden/gpt2_tiny.json."""
    import json
    import pathlib
    from oracle import gpt2_oracle as G
    from oracle.resnet_oracle import summarize
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / "gpt2_tiny.json").read_text())
    model = G.build_model(**doc["config"], seed=doc["seed"])
    batches = G.make_tokens(doc["batch"], doc["seq"], doc["config"]["vocab"], doc["steps"], seed=doc["seed"])
    losses, final = G.train_steps(model, batches)
    assert np.allclose(losses, doc["fp32"]["losses"], rtol=1e-5)
    dig = summarize(final, samples=4)
    for k, d in doc["fp32"]["final"].items():
        assert abs(dig[k]["l2"] - d["l2"]) <= 1e-5 * d["l2"] + 1e-9, k


def test_swin_oracle_reproduces_the_committed_fixture():
    """Same pin for the Swin oracle: seeds in, committed losses and parameter digests out."""
    import json
    import pathlib
    from oracle import swin_oracle as S
    from oracle.resnet_oracle import summarize
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / "swin_tiny.json").read_text())
    cfg = {k: tuple(v) if isinstance(v, list) else v for k, v in doc["config"].items()}
    model = S.build_model(**cfg, seed=doc["seed"])
    batches = S.make_batches(doc["batch"], doc["steps"], cfg["image"], cfg["num_classes"], seed=doc["seed"])
    losses, final = S.train_steps(model, batches)
    assert np.allclose(losses, doc["fp32"]["losses"], rtol=1e-4)
    dig = summarize(final, samples=4)
    for k, d in doc["fp32"]["final"].items():
        assert abs(dig[k]["l2"] - d["l2"]) <= 1e-4 * d["l2"] + 1e-9, k


def test_distilbert_oracle_reproduces_the_committed_fixture():
    """Same pin for the DistilBERT forward oracle: seeds in, committed digest of the last hidden state out."""
    import json
    import pathlib
    from oracle import distilbert_oracle as D
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / "distilbert_tiny.json").read_text())
    model = D.build_model(**doc["config"], seed=doc["seed"])
    ids = D.make_tokens(doc["batch"], doc["seq"], doc["config"]["vocab"], seed=doc["seed"])
    h = D.last_hidden_state(model, ids)
    d = doc["fp32"]["last_hidden_state"]
    assert list(h.shape) == d["shape"]
    assert abs(float(np.sqrt((h.astype(np.float64) ** 2).sum())) - d["l2"]) <= 1e-5 * d["l2"]
    assert np.allclose(h.reshape(-1)[d["idx"]], d["val"], rtol=1e-4, atol=1e-5)
    assert np.allclose(h[:, 0, :], np.array(d["first_token"]), rtol=1e-4, atol=1e-5)


def test_digest_sketch_measures_distance_and_direction():
    """The +-1 sketch of oracle/digest.py estimates |a - b| / |b| from 16 numbers per tensor: zero for the same
    tensor, the noise level for a perturbed one (within the estimator's 18 % standard error, three sigma here),
    above 1 for an unrelated tensor or a sign error; the sampled entries agree."""
    from oracle import digest as D
    rng = np.random.default_rng(1)
    b = rng.standard_normal(300_000).astype(np.float32)
    d = D.digest({"t": b})["t"]
    assert d["n"] == b.size and len(d["proj"]) == D.NPROJ and len(d["idx"]) == D.NSAMPLES
    assert D.sketch_distance(b, d) == 0.0 and D.sample_distance(b, d) == 0.0
    for eps in (1e-3, 3e-2, 0.3):
        a = b + eps * rng.standard_normal(b.size).astype(np.float32)
        assert 0.45 * eps < D.sketch_distance(a, d) < 1.55 * eps
        assert 0.5 * eps < D.sample_distance(a, d) < 1.5 * eps
    assert D.sketch_distance(-b, d) > 1.0
    assert D.sketch_distance(rng.standard_normal(b.size), d) > 0.7
    # a permutation keeps the norm and the mean, but not the sketch
    assert D.sketch_distance(b[::-1].copy(), d) > 0.7


def test_gpt2_fixture_digests_are_the_oracles():
    """The committed GPT-2 fixture's gradient, final-parameter and update digests are reproduced by the oracle in
    this container (sketch distance and sampled entries at fp32 round-off)."""
    import json
    import pathlib
    from oracle import digest as D
    from oracle import gpt2_oracle as G
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / "gpt2_tiny.json").read_text())
    model = G.build_model(**doc["config"], seed=doc["seed"])
    batches = G.make_tokens(doc["batch"], doc["seq"], doc["config"]["vocab"], doc["steps"], seed=doc["seed"])
    _, grads = G.first_step_gradients(model, batches[0])
    _, final = G.train_steps(model, batches)
    init = G.state_arrays(model)
    for k, d in doc["fp32"]["grad0"].items():
        if d["l2"] > 1e-6:
            assert D.sketch_distance(grads[k], d) < 1e-3 and D.sample_distance(grads[k], d) < 1e-3, k
    for k, d in doc["fp32"]["delta"].items():
        if init[k].ndim >= 2:
            assert D.sketch_distance(final[k] - init[k], d) < 5e-2, k   # AdamW amplifies round-off where g ~ 0


def test_qwen2_oracle_micro_batches_equal_the_whole_batch():
    """The full-size Qwen2 fixture is generated one sequence at a time (host memory); on the tiny configuration
    the accumulated gradient and the losses equal those of the whole batch up to fp32 summation order."""
    import json
    import pathlib
    from oracle import qwen2_oracle as Q
    doc = json.loads((pathlib.Path(__file__).parent / "golden" / "qwen2_tiny.json").read_text())
    model = Q.build_model(**doc["config"], seed=doc["seed"])
    ids = Q.make_tokens(doc["batch"], doc["seq"], doc["config"]["vocab"], 1, seed=doc["seed"])[0]
    l1, g1 = Q.first_step_gradients(model, ids)
    l2, g2 = Q.first_step_gradients(model, ids, micro_batches=doc["batch"])
    assert abs(l1 - l2) < 1e-5 * abs(l1) and abs(l1 - doc["fp32"]["loss0"]) < 1e-5 * abs(l1)
    for k in g1:
        n = np.linalg.norm(g1[k])
        if n > 1e-6:
            assert np.linalg.norm(g1[k] - g2[k]) < 1e-4 * n, k
