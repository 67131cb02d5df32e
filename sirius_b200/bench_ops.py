"""Per-layer micro-benchmark of the convolution kernels on the ResNet-152 layer shapes.


    python -m sirius_b200.bench_ops [--batch 64] [--case NAME] [--pass fprop|dgrad|wgrad|all] [--iters 20]

Each case is timed with CUDA events on the launching stream after warm-up; between timed launches a
buffer larger than L2 is rewritten so every launch starts cold. Prints one JSON line per case/pass.
Used for the per-shape roofline table and as the small, self-terminating command for ncu captures.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops
from ._lib import IMPL_AUTO

# name: (H, W, C, K, R, stride, pad)  -- activations are batch x H x W x C
CASES = {
    "stem_7x7": (224, 224, 8, 64, 7, 2, 3),
    "l1_1x1_reduce": (56, 56, 256, 64, 1, 1, 0),
    "l1_3x3": (56, 56, 64, 64, 3, 1, 1),
    "l1_1x1_expand": (56, 56, 64, 256, 1, 1, 0),
    "l2_1x1_reduce": (28, 28, 512, 128, 1, 1, 0),
    "l2_3x3": (28, 28, 128, 128, 3, 1, 1),
    "l2_1x1_expand": (28, 28, 128, 512, 1, 1, 0),
    "l3_1x1_reduce": (14, 14, 1024, 256, 1, 1, 0),
    "l3_3x3": (14, 14, 256, 256, 3, 1, 1),
    "l3_1x1_expand": (14, 14, 256, 1024, 1, 1, 0),
    "l4_1x1_reduce": (7, 7, 2048, 512, 1, 1, 0),
    "l4_3x3": (7, 7, 512, 512, 3, 1, 1),
    "l4_1x1_expand": (7, 7, 512, 2048, 1, 1, 0),
    "l3_3x3_s2": (28, 28, 256, 256, 3, 2, 1),
    "l3_ds_1x1_s2": (28, 28, 512, 1024, 1, 2, 0),
    # synthetic shapes for pipeline studies: long reductions, one wave of tiles
    "syn_1x1_k4096_n256": (14, 14, 4096, 256, 1, 1, 0),
    "syn_1x1_k4096_n128": (14, 14, 4096, 128, 1, 1, 0),
    "syn_1x1_k4096_n64": (14, 14, 4096, 64, 1, 1, 0),
}


def run_case(name, batch, which, iters, flush):
    H, W, C, K, R, stride, pad = CASES[name]
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(batch, H, W, C, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(K, R, R, C, device=dev, generator=g) * (R * R * C) ** -0.5).to(torch.bfloat16)
    P = (H + 2 * pad - R) // stride + 1
    dy = torch.randn(batch, P, P, K, device=dev, generator=g).to(torch.bfloat16)
    wt = ops.filter_transpose(w)
    flops = 2.0 * batch * P * P * K * R * R * C
    fns = {
        "fprop": lambda: ops.conv_fprop(x, w, stride, pad, impl=IMPL_AUTO),
        "dgrad": lambda: ops.conv_dgrad(dy, wt, x.shape, stride, pad, impl=IMPL_AUTO),
        "wgrad": lambda: ops.conv_wgrad(dy, x, R, R, stride, pad, impl=IMPL_AUTO),
    }
    # bytes every launch must move at least once: both operands read, result written
    io = {
        "fprop": (x.numel() + w.numel() + dy.numel()) * 2,
        "dgrad": (x.numel() + w.numel() + dy.numel()) * 2,
        "wgrad": (x.numel() + dy.numel()) * 2 + w.numel() * 4,
    }
    scrub = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev) if flush else None
    out = []
    for p in (["fprop", "dgrad", "wgrad"] if which == "all" else [which]):
        fn = fns[p]
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        # enqueue every (flush, launch) pair before synchronising, so the host runs ahead of the GPU
        # and the events bracket device time only
        evs = []
        for _ in range(iters):
            if scrub is not None:
                scrub.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        total = sum(a.elapsed_time(b) for a, b in evs)
        us = total / iters * 1e3
        rec = {"case": name, "pass": p, "batch": batch, "us": round(us, 2),
               "tflops": round(flops / us / 1e6, 1), "min_gbytes_per_s": round(io[p] / us / 1e3, 1),
               "gflop": round(flops / 1e9, 2), "mbytes": round(io[p] / 1e6, 1), "tc_status": ops.tc_status()}
        print(json.dumps(rec), flush=True)
        out.append(rec)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--case", default="all")
    ap.add_argument("--pass", dest="which", default="all", choices=["fprop", "dgrad", "wgrad", "all"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    for name in (CASES if a.case == "all" else [a.case]):
        run_case(name, a.batch, a.which, a.iters, not a.no_flush)


if __name__ == "__main__":
    main()
