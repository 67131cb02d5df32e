"""Generates the committed golden fixtures of the Swin training step by running the CPU oracle (torchvision
SwinTransformer + torch.optim.AdamW on the host, the calls of the reference's train/swin_b.py:38,83-95) in the build
container.  Usage:  python tests/golden/make_swin_golden.py [case ...]

A fixture holds the seeds, the per-step losses, and per-tensor digests (L2 norm, mean, a few fixed entries) of the
first-step gradients and of the parameters after the last step."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import swin_oracle as O  # noqa: E402
from oracle.digest import digest  # noqa: E402

CASES = {
    # name: (config, batch, steps)
    "swin_tiny": (dict(image=224, patch=4, embed=32, depths=(2, 2, 2, 2), heads=(2, 4, 8, 16), window=7, num_classes=40), 2, 3),
    "swin_b_c3": (dict(image=224, patch=4, embed=128, depths=(2, 2, 18, 2), heads=(4, 8, 16, 32), window=7, num_classes=1000),
                  32, 2),
}


def run(name):
    cfg, batch, steps = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(**cfg, seed=0)
    batches = O.make_batches(batch, steps, cfg["image"], cfg["num_classes"], seed=0)
    loss0, grads = O.first_step_gradients(model, batches[0])
    losses, final = O.train_steps(model, batches)
    init = O.state_arrays(model)
    doc = {"case": name, "config": {k: list(v) if isinstance(v, tuple) else v for k, v in cfg.items()}, "batch": batch,
           "steps": steps, "seed": 0, "torch": torch.__version__,
           "optimizer": {"kind": "AdamW", "lr": 1e-3, "betas": [0.9, 0.999], "eps": 1e-8, "weight_decay": 0.01},
           "fp32": {"loss0": loss0, "losses": losses, "grad0": digest(grads), "final": digest(final),
                    "delta": digest({k: final[k] - init[k] for k in final})}}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "losses", losses)


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
