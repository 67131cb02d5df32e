"""Linear memory model of the training executors, mem_MB = base + slope * batch, measured on the device.

The TrainAdjuster turns megabytes into batch sizes with one (base, slope) pair per model
(server/train_adjuster.cc:642-698 of the reference: constants fit by hand on V100/A100 for its PyTorch models).
This module measures the pairs for this library's executors: it builds each executor at two batch sizes, reads
the device memory the construction took (cudaMemGetInfo before/after, which is what the inference side can or
cannot get) and the executor's own accounting (memory_bytes), and fits the line through the two points.

    python -m sirius_b200.mem_model            # prints one JSON object: {model: {base_mb, slope_mb, ...}}

The values it printed on a B200 are the "measured" table of srt_adjuster_model_mem_param_measured."""
from __future__ import annotations

import json


def _device_used(fn):
    import torch
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    obj = fn()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    mb = obj.memory_bytes()
    own = sum(mb) if isinstance(mb, (tuple, list)) else int(mb)
    obj.close()
    torch.cuda.synchronize()
    return (free0 - free1) / 2 ** 20, own / 2 ** 20


def _fit(make, b_lo, b_hi):
    lo_dev, lo_own = _device_used(lambda: make(b_lo))
    hi_dev, hi_own = _device_used(lambda: make(b_hi))
    slope = (hi_dev - lo_dev) / (b_hi - b_lo)
    slope_own = (hi_own - lo_own) / (b_hi - b_lo)
    return {"base_mb": round(lo_dev - slope * b_lo, 1), "slope_mb": round(slope, 2),
            "base_mb_accounted": round(lo_own - slope_own * b_lo, 1), "slope_mb_accounted": round(slope_own, 2),
            "batches": [b_lo, b_hi], "device_mb": [round(lo_dev, 1), round(hi_dev, 1)]}


def measure(models=("resnet152", "swin_b", "gpt2", "qwen")) -> dict:
    import torch
    from .gpt2_step import Gpt2Step
    from .qwen2_step import Qwen2Step
    from .step import ResNetStep
    from .swin_step import SwinStep
    torch.cuda.init()
    torch.zeros(1, device="cuda")          # the context itself is not the executor's memory
    makers = {
        "resnet152": (lambda b: ResNetStep(arch="resnet152", max_batch=b, image=224, dtype="bf16"), 16, 64),
        "swin_b": (lambda b: SwinStep(max_batch=b), 8, 32),
        "gpt2": (lambda b: Gpt2Step(max_batch=b, seq=1024), 2, 8),
        "qwen": (lambda b: Qwen2Step(max_batch=b, seq=2048), 1, 4),
    }
    out = {}
    for m in models:
        make, lo, hi = makers[m]
        make(lo).close()                   # first construction also loads kernels and library workspaces: not counted
        out[m] = _fit(make, lo, hi)
    return out


if __name__ == "__main__":
    print(json.dumps(measure()), flush=True)
