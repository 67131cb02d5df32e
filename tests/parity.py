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
    worst = (0.0, "", 0.0)
    bad = []
    for k in ref64:
        ok, eo, er = anchored_tensor(get_ours(k), ref32[k], ref64[k], factor, floor)
        if eo > worst[0]:
            worst = (eo, k, er)
        if not ok:
            bad.append((k, eo, er))
    print(f"{what}: worst rel-L2 to fp64 anchor {worst[0]:.3e} at {worst[1]} (reference fp32 there: {worst[2]:.3e})")
    assert not bad, f"{what}: {len(bad)} tensors farther from exact than the reference allows, e.g. {bad[:3]}"


def check_digest(get_ours, dig32: dict, dig64: dict, factor=3.0, floor=1e-4, what=""):
    """Same criterion on the committed per-tensor digests (L2 norm and sampled entries)."""
    bad, worst = [], 0.0
    for k, d64 in dig64.items():
        a = np.asarray(get_ours(k), np.float64).ravel()
        l2 = float(np.sqrt((a ** 2).sum()))
        if not anchored_scalar(l2, dig32[k]["l2"], d64["l2"], factor, floor):
            bad.append((k, "l2", l2, dig32[k]["l2"], d64["l2"]))
        worst = max(worst, abs(l2 - d64["l2"]) / (d64["l2"] + 1e-30))
        scale = d64["l2"] / np.sqrt(a.size)  # typical entry magnitude
        for i, v32, v64 in zip(d64["idx"], dig32[k]["val"], d64["val"]):
            if abs(a[i] - v64) > factor * abs(v32 - v64) + floor * max(abs(v64), scale) + 1e-12:
                bad.append((k, i, float(a[i]), v32, v64))
    print(f"{what}: worst relative L2-norm deviation from the fp64 digest {worst:.3e}")
    assert not bad, f"{what}: {len(bad)} digest entries off, e.g. {bad[:3]}"
