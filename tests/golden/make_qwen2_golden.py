"""Generates the committed golden fixtures of the Qwen2 training step by running the CPU oracle (transformers
Qwen2ForCausalLM + torch.optim.AdamW on the host, the calls of the reference's train/qwen.py:35-37,80-91) in the build
container.  Usage:  python tests/golden/make_qwen2_golden.py [case ...]

A fixture holds the seeds, the per-step losses, and per-tensor digests (L2 norm, mean, a few fixed entries) of the
first-step gradients and of the parameters after the last step. qwen2_05b_s2048 is the 0.5B shape at one sequence of
2048 tokens (the benchmark configuration runs four per GPU; one keeps the CPU run to minutes)."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import qwen2_oracle as O  # noqa: E402
from oracle.resnet_oracle import summarize  # noqa: E402

CASES = {
    # name: (config, batch, seq, steps)
    "qwen2_tiny": (dict(n_layer=2, n_head=4, n_kv_head=2, hidden=128, intermediate=256, vocab=500), 2, 128, 3),
    "qwen2_05b_s2048": (dict(n_layer=24, n_head=14, n_kv_head=2, hidden=896, intermediate=4864, vocab=151936), 1, 2048, 2),
}


def run(name):
    cfg, batch, seq, steps = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(**cfg, seed=0)
    batches = O.make_tokens(batch, seq, cfg["vocab"], steps, seed=0)
    loss0, grads = O.first_step_gradients(model, batches[0])
    losses, final = O.train_steps(model, batches)
    doc = {"case": name, "config": cfg, "batch": batch, "seq": seq, "steps": steps, "seed": 0, "torch": torch.__version__,
           "optimizer": {"kind": "AdamW", "lr": 3e-4, "betas": [0.9, 0.999], "eps": 1e-8, "weight_decay": 0.01},
           "fp32": {"loss0": loss0, "losses": losses, "grad0": summarize(grads, samples=4), "final": summarize(final, samples=4)}}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "losses", losses)


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
