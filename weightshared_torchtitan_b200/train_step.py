"""One optimisation step of the weight-shared decoder under token data parallelism.

Mirrors the order of Trainer.train_step / forward_backward_step in the reference
(torchtitan/train.py:404-527): zero grads -> forward + loss -> backward -> gradient
averaging over the data-parallel ranks -> clip -> optimizer step. The averaging is one
all-reduce of the flat arena (dp.GradArena) instead of DDP's bucketed hooks.
"""
from __future__ import annotations

from typing import Optional

import torch

from .decoder import WeightSharedDecoder
from .dp import GradArena


class TrainStep:
    """All parameters live in one flat fp32 buffer with the layout of the gradient arena
    (``flat=True``), so AdamW and the clip are single passes over one tensor and the
    compute-dtype copies of the weights are re-cast by ONE kernel after the optimizer step.
    ``flat=False`` keeps per-parameter storage and lets the model re-cast its copies one by
    one (the reference's post_optimizer_hook slot)."""

    def __init__(self, model: WeightSharedDecoder, lr: float = 3e-4, weight_decay: float = 0.1,
                 max_norm: Optional[float] = 1.0, process_group=None, flat: bool = True):
        self.model = model
        self.arena = GradArena(model, process_group)
        self.flat = bool(flat)
        if self.flat:
            master = self.arena.flatten_parameters()
            model._cache.bind(self.arena)
            self._flat_param = torch.nn.Parameter(master, requires_grad=True)
            self._flat_param.grad = self.arena.buffer
            opt_params = [self._flat_param]
        else:
            opt_params = self.arena.params
        # AdamW as in the reference's default optimizer (torchtitan/components/optimizer.py:243-326).
        self.optimizer = torch.optim.AdamW(opt_params, lr=lr, betas=(0.9, 0.95), eps=1e-8,
                                           weight_decay=weight_decay, fused=self.arena.buffer.is_cuda)
        self.max_norm = max_norm

    def __call__(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self.arena.zero()
        loss = self.model.loss(tokens, labels)
        loss.backward()
        self.arena.all_reduce_mean()
        if self.max_norm is not None:
            self.arena.clip_(self.max_norm)
        self.optimizer.step()
        # the master weights changed: the compute-dtype copies follow (fused optimizers leave
        # the version counters alone, so this must be explicit)
        if self.flat:
            self.arena.refresh_compute_copies()
        else:
            self.model.post_optimizer_hook()
        return loss.detach()
