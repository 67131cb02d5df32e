"""CPU oracle of the GPT-2 training step: the model class and calls of the reference's training script
(train/gpt2.py:26,90-97: transformers.GPT2LMHeadModel, loss = model(ids, labels=ids).loss, AdamW) run by stock
PyTorch on the host. TEST INFRASTRUCTURE ONLY: never imported by the product.

The arithmetic lives in PyTorch and transformers, which are not part of the reference tree; the reference has no
golden vectors for this model, so the pin is this oracle's own output on seeded weights and token ids
(tests/golden/gpt2_*.json, written by tests/golden/make_gpt2_golden.py)."""
from __future__ import annotations

import copy

import numpy as np
import torch


def build_model(n_layer, n_head, d_model, vocab, ctx, seed=0, double=False):
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(seed)
    cfg = GPT2Config(vocab_size=vocab, n_positions=ctx, n_embd=d_model, n_layer=n_layer, n_head=n_head,
                     resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, attn_implementation="eager")
    m = GPT2LMHeadModel(cfg)
    m.train()
    return m.double() if double else m


def make_tokens(batch, seq, vocab, steps, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=g) for _ in range(steps)]


def state_arrays(model):
    """Parameters under the names the step object uses (lm_head.weight is the tied token table)."""
    return {k: v.detach().cpu().float().numpy().copy() for k, v in model.state_dict().items()
            if k.startswith("transformer.") and not k.endswith(".attn.bias") and not k.endswith(".masked_bias")}


def first_step_gradients(model, ids, autocast_bf16=False):
    m = copy.deepcopy(model)
    with torch.autocast("cpu", dtype=torch.bfloat16, enabled=autocast_bf16):
        loss = m(ids, labels=ids).loss
    loss.backward()
    grads = {k: p.grad.detach().float().numpy().copy() for k, p in m.named_parameters() if k.startswith("transformer.")}
    return float(loss.detach()), grads


def train_steps(model, batches, lr=3e-4, weight_decay=0.01, autocast_bf16=False):
    m = copy.deepcopy(model)
    opt = torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=weight_decay)
    losses = []
    for ids in batches:
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cpu", dtype=torch.bfloat16, enabled=autocast_bf16):
            loss = m(ids, labels=ids).loss
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses, state_arrays(m)


def forward_logits(model, ids):
    with torch.no_grad():
        return model(ids).logits.float().numpy()
