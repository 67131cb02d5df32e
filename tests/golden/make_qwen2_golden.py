"""Generates the committed golden fixtures of the Qwen2 training step by running the CPU oracle (transformers
Qwen2ForCausalLM + torch.optim.AdamW on the host, the calls of the reference's train/qwen.py:35-37,80-91) in the build
container.  Usage:  python tests/golden/make_qwen2_golden.py [case ...]

A fixture holds the seeds, the per-step losses, and per-tensor digests (oracle/digest.py: L2 norm, mean, fixed entries
and a +-1 sketch) of the first-step gradients, of the parameters after the last step and of the update those steps
made. qwen2_05b_b4_s2048 is the 0.5B shape at four sequences of 2048 tokens, the per-GPU batch of the benchmark
configuration; the oracle runs the four sequences one at a time and accumulates (see qwen2_oracle._loss_backward), which
keeps eager attention's saved probabilities of one sequence in host memory at a time."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import qwen2_oracle as O  # noqa: E402
from oracle.digest import digest  # noqa: E402

CASES = {
    # name: (config, batch, seq, steps, oracle micro-batches)
    "qwen2_tiny": (dict(n_layer=2, n_head=4, n_kv_head=2, hidden=128, intermediate=256, vocab=500), 2, 128, 3, 1),
    "qwen2_05b_b4_s2048": (dict(n_layer=24, n_head=14, n_kv_head=2, hidden=896, intermediate=4864, vocab=151936),
                           4, 2048, 2, 4),
}


def run(name):
    cfg, batch, seq, steps, micro = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(**cfg, seed=0)
    batches = O.make_tokens(batch, seq, cfg["vocab"], steps, seed=0)
    loss0, grads = O.first_step_gradients(model, batches[0], micro_batches=micro)
    losses, final = O.train_steps(model, batches, micro_batches=micro)
    init = O.state_arrays(model)
    doc = {"case": name, "config": cfg, "batch": batch, "seq": seq, "steps": steps, "oracle_micro_batches": micro, "seed": 0, "torch": torch.__version__,
           "optimizer": {"kind": "AdamW", "lr": 3e-4, "betas": [0.9, 0.999], "eps": 1e-8, "weight_decay": 0.01},
           "fp32": {"loss0": loss0, "losses": losses, "grad0": digest(grads), "final": digest(final),
                    "delta": digest({k: final[k] - init[k] for k in final})}}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "losses", losses)


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
