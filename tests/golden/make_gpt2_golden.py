"""Generates the committed golden fixtures of the GPT-2 training step by running the CPU oracle
(transformers.GPT2LMHeadModel + torch.optim.AdamW on the host, the calls of the reference's train/gpt2.py:26,90-97)
in the build container.  Usage:  python tests/golden/make_gpt2_golden.py [case ...]

A fixture holds the seeds, the per-step losses, and per-tensor digests (oracle/digest.py: L2 norm, mean, fixed entries
and a +-1 sketch that lets a test bound the relative L2 distance) of the first-step gradients, of the parameters
after the last step and of the update (final - initial) those steps made."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import gpt2_oracle as O  # noqa: E402
from oracle.digest import digest  # noqa: E402

CASES = {
    # name: (config, batch, seq, steps)
    "gpt2_tiny": (dict(n_layer=2, n_head=4, d_model=128, vocab=500, ctx=64), 2, 64, 3),
    "gpt2_c4": (dict(n_layer=12, n_head=12, d_model=768, vocab=50257, ctx=1024), 8, 1024, 3),
}


def run(name):
    cfg, batch, seq, steps = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(**cfg, seed=0)
    batches = O.make_tokens(batch, seq, cfg["vocab"], steps, seed=0)
    loss0, grads = O.first_step_gradients(model, batches[0])
    losses, final = O.train_steps(model, batches)
    init = O.state_arrays(model)
    doc = {"case": name, "config": cfg, "batch": batch, "seq": seq, "steps": steps, "seed": 0, "torch": torch.__version__,
           "optimizer": {"kind": "AdamW", "lr": 3e-4, "betas": [0.9, 0.999], "eps": 1e-8, "weight_decay": 0.01},
           "fp32": {"loss0": loss0, "losses": losses, "grad0": digest(grads), "final": digest(final),
                    "delta": digest({k: final[k] - init[k] for k in final})}}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "losses", losses)


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
