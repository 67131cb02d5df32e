"""CPU oracle of the DistilBERT forward pass served by the stand-in inference worker: transformers.DistilBertModel
(the architecture behind the reference's `distilbert_base` inference model, server/model_store/infer_model.cc:46-58)
run by stock PyTorch on the host. TEST INFRASTRUCTURE ONLY: never imported by the product.

The arithmetic lives in PyTorch and transformers, which are not part of the reference tree, and the reference holds
no golden vectors for this model (it loads a compiled TVM module): the pin is this oracle's own output on seeded
weights and token ids (tests/golden/distilbert_*.json, written by tests/golden/make_distilbert_golden.py)."""
from __future__ import annotations

import torch


def build_model(n_layer, n_head, dim, hidden_dim, vocab, max_pos=512, seed=0):
    from transformers import DistilBertConfig, DistilBertModel
    torch.manual_seed(seed)
    cfg = DistilBertConfig(vocab_size=vocab, max_position_embeddings=max_pos, n_layers=n_layer, n_heads=n_head, dim=dim,
                           hidden_dim=hidden_dim, dropout=0.0, attention_dropout=0.0, activation="gelu",
                           sinusoidal_pos_embds=False, attn_implementation="eager")
    m = DistilBertModel(cfg)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():   # biases and norm offsets start at zero and norm scales at one: give them seeded values
        for n, p in m.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
            elif "LayerNorm.weight" in n or "layer_norm.weight" in n:
                p.copy_(1.0 + torch.randn(p.shape, generator=g) * 0.1)
    m.eval()
    return m


def make_tokens(batch, seq, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, seq), generator=g)


def state_arrays(model):
    return {k: v.detach().cpu().float().numpy().copy() for k, v in model.state_dict().items()}


def last_hidden_state(model, ids):
    with torch.no_grad():
        return model(input_ids=ids).last_hidden_state.float().numpy()
