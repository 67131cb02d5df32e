"""CPU oracle of the Qwen2 training step: the model class and calls of the reference's training script
(train/qwen.py:35-37,80-91: a transformers Qwen2 causal LM, loss = model(ids, labels=ids).loss, AdamW) run by stock
PyTorch on the host. TEST INFRASTRUCTURE ONLY: never imported by the product.

The arithmetic lives in PyTorch and transformers, which are not part of the reference tree; the reference has no
golden vectors for this model, so the pin is this oracle's own output on seeded weights and token ids
(tests/golden/qwen2_*.json, written by tests/golden/make_qwen2_golden.py)."""
from __future__ import annotations

import copy

import torch


def build_model(n_layer, n_head, n_kv_head, hidden, intermediate, vocab, max_pos=4096, seed=0):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(seed)
    cfg = Qwen2Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=intermediate, num_hidden_layers=n_layer,
                      num_attention_heads=n_head, num_key_value_heads=n_kv_head, max_position_embeddings=max_pos,
                      rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_dropout=0.0,
                      use_sliding_window=False, attn_implementation="eager")
    m = Qwen2ForCausalLM(cfg)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():   # the projection biases start at zero; give them seeded values of a visible size
        for n, p in m.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    m.train()
    return m


def make_tokens(batch, seq, vocab, steps, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=g) for _ in range(steps)]


def state_arrays(model):
    return {k: v.detach().cpu().float().numpy().copy() for k, v in model.state_dict().items() if k.startswith("model.")}


def forward_logits(model, ids):
    with torch.no_grad():
        return model(ids).logits.float().numpy()


def _loss_backward(m, ids, micro_batches):
    """Mean next-token loss over the batch, back-propagated. micro_batches > 1 runs the sequences in equal groups
    and scales each group's mean loss by 1 / micro_batches before backward: every sequence holds the same number
    of predicted tokens, so the accumulated gradient is that of the whole batch (up to fp32 summation order)
    while the activations of one group at a time fit the host's memory."""
    total = 0.0
    for chunk in ids.chunk(micro_batches):
        loss = m(chunk, labels=chunk).loss / micro_batches
        loss.backward()
        total += float(loss.detach())
    return total


def first_step_gradients(model, ids, micro_batches=1):
    m = copy.deepcopy(model)
    loss = _loss_backward(m, ids, micro_batches)
    return loss, {k: p.grad.detach().float().numpy().copy() for k, p in m.named_parameters() if k.startswith("model.")}


def train_steps(model, batches, lr=3e-4, weight_decay=0.01, micro_batches=1):
    m = copy.deepcopy(model)
    opt = torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=weight_decay)
    losses = []
    for ids in batches:
        opt.zero_grad(set_to_none=True)
        losses.append(_loss_backward(m, ids, micro_batches))
        opt.step()
    return losses, state_arrays(m)
