"""CPU oracle of the Swin training step: the model class and calls of the reference's training script
(train/swin_b.py:38,83-95: torchvision swin_b, CrossEntropyLoss; AdamW as in the DDP configuration) run by stock
PyTorch on the host, stochastic depth off. TEST INFRASTRUCTURE ONLY: never imported by the product.

The arithmetic lives in PyTorch and torchvision, which are not part of the reference tree; the reference has no
golden vectors for this model, so the pin is this oracle's own output on seeded weights and inputs
(tests/golden/swin_*.json, written by tests/golden/make_swin_golden.py)."""
from __future__ import annotations

import copy

import torch


def build_model(image=224, patch=4, embed=128, depths=(2, 2, 18, 2), heads=(4, 8, 16, 32), window=7, num_classes=1000, seed=0):
    from torchvision.models.swin_transformer import SwinTransformer
    torch.manual_seed(seed)
    m = SwinTransformer(patch_size=[patch, patch], embed_dim=embed, depths=list(depths), num_heads=list(heads),
                        window_size=[window, window], stochastic_depth_prob=0.0, num_classes=num_classes)
    # the bias tables and the zero biases start too small to show up in a loss; give them seeded values of a visible size
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("relative_position_bias_table"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.5)
            elif n.endswith(".bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    m.train()
    return m


def make_batches(batch, steps, image=224, num_classes=1000, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(batch, 3, image, image, generator=g), torch.randint(0, num_classes, (batch,), generator=g))
            for _ in range(steps)]


def state_arrays(model):
    return {k: v.detach().cpu().float().numpy().copy() for k, v in model.state_dict().items()
            if not k.endswith("relative_position_index")}


def forward_logits(model, images):
    with torch.no_grad():
        return model(images).float().numpy()


def first_step_gradients(model, batch):
    m = copy.deepcopy(model)
    loss = torch.nn.functional.cross_entropy(m(batch[0]), batch[1])
    loss.backward()
    return float(loss.detach()), {k: p.grad.detach().float().numpy().copy() for k, p in m.named_parameters()}


def train_steps(model, batches, lr=1e-3, weight_decay=0.01):
    m = copy.deepcopy(model)
    opt = torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=weight_decay)
    losses = []
    for images, labels in batches:
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(m(images), labels)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses, state_arrays(m)
