"""Shared parity criteria.

Training a deep BatchNorm/ReLU network is discontinuous in its inputs: an activation within
rounding distance of zero flips its ReLU mask (or a max-pool argmax) and changes every upstream
gradient by a finite amount. The reference's own fp32 CPU path therefore differs from exact
arithmetic by far more than 1e-4 once gradients are involved (for ResNet-152, batch 16, the
per-tensor fp32-vs-fp64 gradient difference has a median of 9e-2). The criteria below anchor on
the fp64 run of the same seeded model and require the CUDA result to be as close to it as the
reference's fp32 path is, within `factor`, plus a relative `floor`:

    |ours - exact| <= factor * |ref32 - exact| + floor * |exact|
"""
import numpy as np


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.sqrt(((a - b) ** 2).sum()) / (np.sqrt((b ** 2).sum()) + 1e-30))


def anchored_scalar(ours, ref32, ref64, factor=3.0, floor=1e-4):
    return abs(ours - ref64) <= factor * abs(ref32 - ref64) + floor * max(abs(ref64), 1e-30)


def anchored_tensor(ours, ref32, ref64, factor=3.0, floor=1e-4):
    """Returns (ok, err_ours, err_ref): rel-L2 distances to the fp64 anchor."""
    eo, er = rel_l2(ours, ref64), rel_l2(ref32, ref64)
    return eo <= factor * er + floor, eo, er


def check_tensors(get_ours, ref32: dict, ref64: dict, factor=3.0, floor=1e-4, what=""):
    """Anchored comparison of a set of tensors. Flips are random events, so the criterion is applied
    to the root-mean-square of the per-tensor distances; each single tensor additionally has to stay
    within `factor` times the reference's worst tensor (plus 1e-3, about the weight of one flipped
    activation)."""
    eo = {k: rel_l2(get_ours(k), ref64[k]) for k in ref64}
    er = {k: rel_l2(ref32[k], ref64[k]) for k in ref64}
    rms_o = float(np.sqrt(np.mean(np.square(list(eo.values())))))
    rms_r = float(np.sqrt(np.mean(np.square(list(er.values())))))
    worst = max(eo, key=eo.get)
    print(f"{what}: rel-L2 to the fp64 anchor, rms over tensors: ours {rms_o:.3e}, reference fp32 {rms_r:.3e}; "
          f"worst ours {eo[worst]:.3e} at {worst} (reference there {er[worst]:.3e})")
    assert rms_o <= factor * rms_r + floor, f"{what}: rms {rms_o:.3e} vs reference {rms_r:.3e}"
    cap = factor * max(er.values()) + 1e-3
    bad = [(k, eo[k], er[k]) for k in eo if eo[k] > cap]
    assert not bad, f"{what}: {len(bad)} tensors beyond {cap:.3e}, e.g. {bad[:3]}"


def check_digest(get_ours, dig32: dict, dig64: dict, factor=3.0, floor=1e-4, what=""):
    """Same criterion on the committed per-tensor digests (L2 norm and sampled entries), applied to
    the root-mean-square over all tensors of the relative deviations."""
    n_o, n_r, s_o, s_r = [], [], [], []
    for k, d64 in dig64.items():
        a = np.asarray(get_ours(k), np.float64).ravel()
        l2 = float(np.sqrt((a ** 2).sum()))
        n_o.append(abs(l2 - d64["l2"]) / (d64["l2"] + 1e-30))
        n_r.append(abs(dig32[k]["l2"] - d64["l2"]) / (d64["l2"] + 1e-30))
        scale = d64["l2"] / np.sqrt(a.size) + 1e-30  # typical entry magnitude
        for i, v32, v64 in zip(d64["idx"], dig32[k]["val"], d64["val"]):
            s_o.append(abs(a[i] - v64) / scale)
            s_r.append(abs(v32 - v64) / scale)
    rms = lambda v: float(np.sqrt(np.mean(np.square(v))))
    print(f"{what}: rms relative deviation from the fp64 digest: norms ours {rms(n_o):.3e} / reference "
          f"{rms(n_r):.3e}; sampled entries ours {rms(s_o):.3e} / reference {rms(s_r):.3e}")
    assert rms(n_o) <= factor * rms(n_r) + floor, what
    assert rms(s_o) <= factor * rms(s_r) + floor, what


# ---- committed digests of full-size runs (oracle/digest.py) -------------------------------------------------
def check_gradient_digests(get_grad, dig: dict, tol=5e-2, what=""):
    """First-step gradients against the oracle's digests, per tensor: the relative L2 distance estimated from the
    +-1 sketch, and the root-mean-square deviation of the fixed entries relative to the tensor's rms entry, must
    both stay within `tol` times 1.6 (the sketch estimate of a distance has a relative standard error of 18 %,
    the 32-entry one of 13 %; 1.6 is three of the former). Tensors whose gradient is zero up to rounding (a bias
    softmax cannot see, and the like: norm below 1e-3 of the largest) are skipped. Unlike a norm, both
    quantities are sensitive to direction: a sign error reads 2, an unrelated tensor 1.4."""
    from oracle.digest import sample_distance, sketch_distance
    top = max(d["l2"] for d in dig.values())
    worst = (0.0, None, None)
    for n, d in dig.items():
        if d["l2"] < 1e-3 * top:
            continue
        g = get_grad(n)
        l2 = float(np.sqrt((np.asarray(g, np.float64) ** 2).sum()))
        assert abs(l2 - d["l2"]) < tol * d["l2"], (what, n, "norm", l2, d["l2"])
        ds, de = sketch_distance(g, d), sample_distance(g, d)
        worst = max(worst, (ds, n, "sketch"), (de, n, "entries"))
        assert ds < 1.6 * tol, (what, n, "sketch distance", ds)
        assert de < 1.6 * tol, (what, n, "sampled entries", de)
    print(f"{what}: worst relative distance to the oracle's gradient digests {worst}")


def check_update_digests(get_param, init: dict, dig_delta: dict, dig_final: dict, lr, steps, what=""):
    """The update p_final - p_init after `steps` AdamW steps against the oracle's.

    AdamW's first steps move every entry by about lr * sign(gradient), so where rounding makes a small gradient
    entry change sign the update differs by 2 lr however good the arithmetic is; with gradient errors of a few
    percent that is a few percent of the entries and a relative L2 distance of 0.2-0.35 between two correct
    runs (measured between the oracle's fp32 and bf16-autocast runs of the small configurations), while a wrong
    gradient direction gives 1.4 and a sign error 2. Weight tensors (two or more dimensions in the model, i.e.
    not a bias or a norm scale) therefore must stay below 0.3 in estimated relative L2 distance (measured on a
    B200: 0.06 on the small configurations, 0.09 on GPT-2 small at 8 x 1024) and within 10 %
    in norm; every tensor's final value must match the oracle's in norm (2e-2 plus the drift bound
    2 * lr * steps * sqrt(n) for the vectors) and no sampled entry may be farther than 2 * lr * steps from the
    oracle's beyond 2e-2 of its size."""
    from oracle.digest import sketch_distance
    worst = (0.0, None)
    for n, d in dig_delta.items():
        p = np.asarray(get_param(n), np.float64)
        delta = p - np.asarray(init[n], np.float64)
        is_matrix = np.asarray(init[n]).ndim >= 2
        if is_matrix and d["l2"] > 0:
            dist = sketch_distance(delta, d)
            worst = max(worst, (dist, n))
            assert dist < 0.3, (what, n, "update direction", dist)
            l2 = float(np.sqrt((delta ** 2).sum()))
            assert abs(l2 - d["l2"]) < 0.1 * d["l2"], (what, n, "update norm", l2, d["l2"])
        f = dig_final[n]
        flat = p.ravel()
        l2 = float(np.sqrt((flat ** 2).sum()))
        drift = 0.0 if is_matrix else 2 * lr * steps * np.sqrt(flat.size)
        assert abs(l2 - f["l2"]) <= 2e-2 * f["l2"] + drift, (what, n, "final norm", l2, f["l2"])
        got = flat[np.asarray(f["idx"], dtype=np.int64)]
        lim = 2e-2 * np.abs(np.asarray(f["val"])) + 2 * lr * steps * 1.01
        assert np.all(np.abs(got - np.asarray(f["val"])) <= lim), (what, n, "final entries")
    print(f"{what}: worst estimated relative distance of a weight update to the oracle's {worst}")
