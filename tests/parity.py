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
