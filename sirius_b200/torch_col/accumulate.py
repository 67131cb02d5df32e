"""GradAccumulator (pytorch/torch_col/accumulate.py:7-49): keeps the gradient of the global batch while
micro-batches come and go, so a killed micro-batch only loses its own work.

Two back ends with the same three methods: a sirius_b200 step object (the accumulation and the
optimizer run as fused kernels over its flat buffers) or a torch.nn.Module (the reference's code path,
used on CPU ranks in the tests)."""
from __future__ import annotations

from collections import defaultdict


class GradAccumulator:
    def __init__(self, model, exchange=None):
        """exchange: a sirius_b200.ddp.GradExchange for data-parallel training with a step object. The ranks of a
        job may run different numbers of micro-batches per global batch, so what they exchange is the accumulated
        gradient, once, right before the update (DDP's no_sync on every micro-batch but the last,
        pytorch/torch_col/dynamic_batch.py:155-167)."""
        self._step = model if hasattr(model, 'optimizer_step') and hasattr(model, 'accumulate') else None
        self._exchange = exchange
        if exchange is not None and self._step is None:
            raise ValueError("a GradExchange works on a step object; torch modules bring their own all-reduce")
        if self._step is None:
            import torch
            self.param_list = [p for p in model.parameters() if p.requires_grad]
            self.param_grads = defaultdict(dict)
            for p in self.param_list:
                self.param_grads[p]['global'] = torch.zeros_like(p)
                self.param_grads[p]['local'] = None

    def accumulate(self):
        if self._step is not None:
            return self._step.accumulate()
        for p in self.param_list:
            self.param_grads[p]['global'] += p.grad
            p.grad.zero_()

    def step(self, optimizer=None, scaler=None, do_zero_grad=True):
        if self._step is not None:
            if self._exchange is not None:
                self._exchange.allreduce(self._step, accumulated=True)   # sum over ranks, on the library's NCCL stream
            return self._step.optimizer_step()  # uses and then clears the accumulated gradient
        for p in self.param_list:
            self.param_grads[p]['local'] = p.grad
            p.grad = self.param_grads[p]['global']
        if scaler is not None:
            scaler.step(optimizer)
            scaler.update()
        else:
            optimizer.step()
        for p in self.param_list:
            p.grad = self.param_grads[p]['local']
        if do_zero_grad:
            self.zero_grad()

    def zero_grad(self):
        if self._step is None:
            for p in self.param_list:
                self.param_grads[p]['global'].zero_()
