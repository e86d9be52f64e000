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
    def __init__(self, model: WeightSharedDecoder, lr: float = 3e-4, weight_decay: float = 0.1,
                 max_norm: Optional[float] = 1.0, process_group=None):
        self.model = model
        self.arena = GradArena(model, process_group)
        # AdamW as in the reference's default optimizer (torchtitan/components/optimizer.py:243-326).
        self.optimizer = torch.optim.AdamW(self.arena.params, lr=lr, betas=(0.9, 0.95), eps=1e-8,
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
        return loss.detach()
