"""Generates the committed golden fixtures of the DistilBERT forward pass by running the CPU oracle
(transformers.DistilBertModel on the host) in the build container.
Usage:  python tests/golden/make_distilbert_golden.py [case ...]

A fixture holds the seeds and a digest of the last hidden state (L2 norm, mean, fixed entries, and the full first and
last token vectors of every sequence). distilbert_base_s128 is the benchmark configuration: batch 1, 128 tokens."""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import distilbert_oracle as O  # noqa: E402

CASES = {
    # name: (config, batch, seq)
    "distilbert_tiny": (dict(n_layer=2, n_head=4, dim=128, hidden_dim=256, vocab=500, max_pos=64), 3, 32),
    "distilbert_base_s128": (dict(n_layer=6, n_head=12, dim=768, hidden_dim=3072, vocab=30522, max_pos=512), 1, 128),
}


def digest(h):
    flat = h.reshape(-1)
    idx = np.linspace(0, flat.size - 1, 16).astype(np.int64)
    return {"shape": list(h.shape), "l2": float(np.sqrt((flat.astype(np.float64) ** 2).sum())), "mean": float(flat.mean()),
            "abs_max": float(np.abs(flat).max()), "idx": idx.tolist(), "val": [float(flat[i]) for i in idx],
            "first_token": h[:, 0, :].astype(np.float64).round(6).tolist(),
            "last_token": h[:, -1, :].astype(np.float64).round(6).tolist()}


def run(name):
    cfg, batch, seq = CASES[name]
    torch.set_num_threads(os.cpu_count() or 1)
    model = O.build_model(**cfg, seed=0)
    ids = O.make_tokens(batch, seq, cfg["vocab"], seed=0)
    h = O.last_hidden_state(model, ids)
    doc = {"case": name, "config": cfg, "batch": batch, "seq": seq, "seed": 0, "torch": torch.__version__,
           "fp32": {"last_hidden_state": digest(h)}}
    with open(os.path.join(HERE, name + ".json"), "w") as f:
        json.dump(doc, f)
    print(name, "l2", doc["fp32"]["last_hidden_state"]["l2"])


if __name__ == "__main__":
    for n in (sys.argv[1:] or list(CASES)):
        run(n)
