"""Per-layer micro-benchmark of the convolution and BatchNorm kernels on the ResNet-152 layer shapes
(a measurement tool beside bench.py; nothing in the library imports it).

    python bench_layers.py [--batch 64] [--case NAME] [--pass fprop|fprop_stats|dgrad|wgrad|all|bn] [--iters 20]
                           [--plan gather,tile_n,pair]

Each case is timed with CUDA events on the launching stream after warm-up; between timed launches a
buffer larger than L2 is rewritten so every launch starts cold. Prints one JSON line per case/pass.
Used for the per-shape roofline table and as the small, self-terminating command for ncu captures.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import torch

from sirius_b200 import _lib, ops
from sirius_b200._lib import IMPL_AUTO, SRT_BF16, ConvDesc

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


PLAN = ""


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
    # fprop whose epilogue also takes the BatchNorm column sums (the convolution launch alone, no finalize)
    d = ConvDesc.make(batch, H, W, C, K, R, R, stride, pad)
    y_st = torch.empty_like(dy)
    nb = _lib.lib().srt_conv_fprop_bn_stats_bytes(ctypes.byref(d))
    partial = torch.empty(nb, dtype=torch.uint8, device=dev)
    slabs = ctypes.c_int(0)

    def fprop_stats():
        _lib.call("srt_conv_fprop_bn_stats", ctypes.byref(d), SRT_BF16, IMPL_AUTO, x.data_ptr(), w.data_ptr(), y_st.data_ptr(),
                  None, partial.data_ptr(), nb, ctypes.byref(slabs), torch.cuda.current_stream().cuda_stream)

    fns = {
        "fprop_stats": fprop_stats,
        "fprop": lambda: ops.conv_fprop(x, w, stride, pad, impl=IMPL_AUTO),
        "dgrad": lambda: ops.conv_dgrad(dy, wt, x.shape, stride, pad, impl=IMPL_AUTO),
        "wgrad": lambda: ops.conv_wgrad(dy, x, R, R, stride, pad, impl=IMPL_AUTO),
    }
    # bytes every launch must move at least once: both operands read, result written
    io = {
        "fprop_stats": (x.numel() + w.numel() + dy.numel()) * 2 + nb,
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
        rec = {"case": name, "pass": p, "batch": batch, "plan": PLAN, "us": round(us, 2),
               "tflops": round(flops / us / 1e6, 1), "min_gbytes_per_s": round(io[p] / us / 1e3, 1),
               "gflop": round(flops / 1e9, 2), "mbytes": round(io[p] / 1e6, 1), "tc_status": ops.tc_status()}
        print(json.dumps(rec), flush=True)
        out.append(rec)
    return out


# BatchNorm shapes of ResNet-152: name -> (H, W, C, residual unit)
BN_CASES = {
    "bn_stem_c64": (112, 112, 64, False),
    "bn_l1_c64": (56, 56, 64, False),
    "bn_l1_c256_res": (56, 56, 256, True),
    "bn_l2_c128": (28, 28, 128, False),
    "bn_l2_c512_res": (28, 28, 512, True),
    "bn_l3_c256": (14, 14, 256, False),
    "bn_l3_c1024_res": (14, 14, 1024, True),
    "bn_l4_c512": (7, 7, 512, False),
    "bn_l4_c2048_res": (7, 7, 2048, True),
    # next to no data: the fixed cost of the launches (and of the grid barriers of the one-launch kernels)
    "bn_fixed_cost_c64": (2, 2, 64, False),
}


def run_bn_case(name, batch, iters, flush, one_launch=False, bits=False):
    """Forward (statistics + apply) and backward of one BatchNorm(+residual)+ReLU layer. The byte
    counts are the tensors each pass has to move once: forward reads z twice (statistics, apply),
    reads the residual and writes y; backward reads dy and z twice (sums, apply), the stored y twice
    in a residual unit (ReLU mask), and writes dz (and the gradient of the residual branch)."""
    from sirius_b200._lib import call
    H, W, C, res = BN_CASES[name]
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rows = batch * H * W
    z = torch.randn(rows, C, device=dev, generator=g).to(torch.bfloat16)
    r = torch.randn(rows, C, device=dev, generator=g).to(torch.bfloat16) if res else None
    dy = torch.randn(rows, C, device=dev, generator=g).to(torch.bfloat16)
    y = torch.empty_like(z)
    dz = torch.empty_like(z)
    dres = torch.empty_like(z) if res else None
    f32 = lambda v: torch.full((C,), v, dtype=torch.float32, device=dev)
    gamma, beta, rm, rv = f32(1.0), f32(0.0), f32(0.0), f32(1.0)
    mean, invstd, scale, shift, dgamma, dbeta = (f32(0.0) for _ in range(6))
    scratch, nscr = ops.bn_scratch(rows, C, dev)
    P, st, dt = ops._p, ops._stream, ops._dt(z)

    def fwd():
        call("srt_bn_stats", dt, P(z), rows, C, P(gamma), P(beta), 1e-5, 0.1, P(rm), P(rv), P(mean), P(invstd),
             P(scale), P(shift), P(scratch), nscr, st())
        call("srt_bn_apply", dt, P(z), P(r), P(y), rows, C, P(scale), P(shift), 1, st())

    def bwd():
        call("srt_bn_backward", dt, P(dy), P(y if res else None), P(z), rows, C, P(gamma), P(mean), P(invstd),
             P(scale), P(shift), 1, P(dz), P(dres), P(dgamma), P(dbeta), P(scratch), nscr, st())

    if one_launch:
        def fwd():
            call("srt_bn_forward_fused", dt, P(z), P(r), P(y), rows, C, P(gamma), P(beta), 1e-5, 0.1, P(rm), P(rv), P(mean),
                 P(invstd), P(scale), P(shift), 1, st())

        def bwd():
            call("srt_bn_backward_fused", dt, P(dy), P(y if res else None), P(z), rows, C, P(gamma), P(mean), P(invstd),
                 P(scale), P(shift), 1, P(dz), P(dres), P(dgamma), P(dbeta), st())

    if bits and res:
        # residual unit as the training step runs it: the forward apply leaves the ReLU mask as one bit per element,
        # the backward reads the bits instead of y and writes no masked copy of dy
        mask = torch.empty(z.numel() // 8, dtype=torch.uint8, device=dev)

        def fwd():
            call("srt_bn_stats", dt, P(z), rows, C, P(gamma), P(beta), 1e-5, 0.1, P(rm), P(rv), P(mean), P(invstd),
                 P(scale), P(shift), P(scratch), nscr, st())
            call("srt_bn_apply_bits", dt, P(z), P(r), P(y), rows, C, P(scale), P(shift), P(mask), st())

        def bwd():
            call("srt_bn_backward_bits", dt, P(dy), P(mask), P(z), rows, C, P(gamma), P(mean), P(invstd), P(dz), None,
                 P(dgamma), P(dbeta), P(scratch), nscr, int(one_launch), st())

    t = z.numel() * 2
    io = {"bn_fwd": t * (4 if res else 3), "bn_bwd": t * (8 if res else 5)}
    if bits and res:
        io = {"bn_fwd": t * (4 + 1 / 16), "bn_bwd": t * (5 + 2 / 16)}
    scrub = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev) if flush else None
    fwd()
    for p, fn in (("bn_fwd", fwd), ("bn_bwd", bwd)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
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
        us = sum(a.elapsed_time(b) for a, b in evs) / iters * 1e3
        print(json.dumps({"case": name, "pass": p, "one_launch": one_launch, "relu_bits": bool(bits and res), "batch": batch, "us": round(us, 2),
                          "gbytes_per_s": round(io[p] / us / 1e3, 1), "mbytes": round(io[p] / 1e6, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--case", default="all")
    ap.add_argument("--pass", dest="which", default="all", choices=["fprop", "fprop_stats", "dgrad", "wgrad", "all", "bn"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--one-launch", action="store_true", help="BatchNorm cases: the one-launch kernels")
    ap.add_argument("--relu-bits", action="store_true", help="BatchNorm residual cases: mask bits instead of the stored output")
    ap.add_argument("--plan", default="", help="fprop/dgrad plan override 'gather,tile_n,pair' (srt_conv_plan_override)")
    a = ap.parse_args()
    global PLAN
    PLAN = a.plan
    if a.plan:
        _lib.lib().srt_conv_plan_override(*[int(v) for v in a.plan.split(",")])
    if a.which == "bn":
        for name in (BN_CASES if a.case == "all" else [a.case]):
            run_bn_case(name, a.batch, a.iters, not a.no_flush, a.one_launch, a.relu_bits)
        return
    for name in (CASES if a.case == "all" else [a.case]):
        run_case(name, a.batch, a.which, a.iters, not a.no_flush)


if __name__ == "__main__":
    main()
