"""Generates the committed golden fixtures of the ResNet training step by running the CPU oracle
(stock torchvision + PyTorch CPU, the calls of the reference's train/resnet152.py:22-28,84-91)
in the build container.  Usage:  python tests/golden/make_resnet_golden.py [case ...]

Each fixture holds the fp32 result (what the reference's CPU path computes) and the fp64 result
from the same seeded weights and inputs (the exact-arithmetic anchor), so a test can state how far
the reference's own fp32 arithmetic is from exact and require the CUDA path to be as close.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import resnet_oracle as O  # noqa: E402

CASES = {
    # name: (arch, batch, image, steps)
    "resnet14_small": ("resnet14", 8, 64, 2),
    "resnet50_small": ("resnet50", 4, 64, 2),
    "resnet152_c1": ("resnet152", 16, 224, 3),
}


def run_precision(arch, batch, image, steps, double, autocast=False):
    model = O.build_model(arch, 0, double=double)
    batches = O.make_batches(batch, steps, image, double=double)
    loss0, grads = O.first_step_gradients(model, batches[0], autocast_bf16=autocast)
    losses = O.train_steps(model, batches, autocast_bf16=autocast)
    return {"loss0": loss0, "losses": losses, "grad0": O.summarize(grads, samples=4),
            "final": O.summarize(O.state_arrays(model), samples=4)}


def run(name):
    arch, batch, image, steps = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    doc = {"case": name, "arch": arch, "batch": batch, "image": image, "steps": steps, "seed": 0,
           "torch": torch.__version__, "optimizer": {"lr": 0.1, "momentum": 0.9, "weight_decay": 1e-4},
           "fp32": run_precision(arch, batch, image, steps, False),
           "fp64": run_precision(arch, batch, image, steps, True),
           # PyTorch's own reduced-precision path on the CPU: how far bf16 training drifts from exact
           "bf16_autocast": run_precision(arch, batch, image, steps, False, autocast=True)}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "fp32 losses", doc["fp32"]["losses"], "fp64 losses", doc["fp64"]["losses"],
          "bf16 autocast losses", doc["bf16_autocast"]["losses"])


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
