"""One optimisation step of the weight-shared decoder under token data parallelism.

Mirrors the order of Trainer.train_step / forward_backward_step in the reference
(torchtitan/train.py:404-527): zero grads -> forward + loss -> backward -> gradient
averaging over the data-parallel ranks -> clip -> optimizer step. The averaging is one
all-reduce of the flat arena (dp.GradArena) instead of DDP's bucketed hooks.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .decoder import WeightSharedDecoder
from .dp import GradArena


class TrainStep:
    """All parameters live in one flat fp32 buffer with the layout of the gradient arena
    (``flat=True``). On a GPU the clip, AdamW and the refresh of the bf16 compute copies of
    the weights are then ONE pass over the arenas after one pass over the gradients for the
    norm (``fused_update=True``: wsl_grad_sumsq_partials + wsl_adamw_flat_step); with
    ``fused_update=False`` torch.optim.AdamW steps the flat tensor and one cast kernel
    refreshes the copies. ``flat=False`` keeps per-parameter storage and lets the model re-cast
    its copies one by one (the reference's post_optimizer_hook slot)."""

    def __init__(self, model: WeightSharedDecoder, lr: float = 3e-4, weight_decay: float = 0.1,
                 max_norm: Optional[float] = 1.0, process_group=None, flat: bool = True,
                 fused_update: bool = True):
        self.model = model
        self.arena = GradArena(model, process_group)
        self.flat = bool(flat)
        self.lr, self.weight_decay, self.betas, self.eps = lr, weight_decay, (0.9, 0.95), 1e-8
        self.max_norm = max_norm
        self.fused_update = bool(fused_update) and self.flat and self.arena.buffer.is_cuda
        self.optimizer = None
        self.steps = 0
        if self.flat:
            master = self.arena.flatten_parameters()
            model._cache.bind(self.arena)
        if self.fused_update:
            self.exp_avg = torch.zeros_like(master)
            self.exp_avg_sq = torch.zeros_like(master)
            self._partials = torch.zeros(ops.SUMSQ_PARTIALS, device=master.device, dtype=torch.float32)
            return
        if self.flat:
            self._flat_param = torch.nn.Parameter(master, requires_grad=True)
            self._flat_param.grad = self.arena.buffer
            opt_params = [self._flat_param]
        else:
            opt_params = self.arena.params
        # AdamW as in the reference's default optimizer (torchtitan/components/optimizer.py:243-326).
        self.optimizer = torch.optim.AdamW(opt_params, lr=lr, betas=self.betas, eps=self.eps,
                                           weight_decay=weight_decay, fused=self.arena.buffer.is_cuda)

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step, before clipping."""
        if self.fused_update:
            return self._partials.sum().sqrt()
        return self._last_norm

    def __call__(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self.arena.zero()
        loss = self.model.loss(tokens, labels)
        loss.backward()
        self.arena.all_reduce_mean()
        self.steps += 1
        if self.fused_update:
            clip = self.max_norm is not None
            if clip:
                ops.grad_sumsq_partials(self.arena.buffer, self._partials)
            copy = self.arena.compute_buffer(self.model.compute_dtype) \
                if self.model.compute_dtype == torch.bfloat16 else None
            ops.adamw_flat_step(self.arena.master, self.arena.buffer, self.exp_avg, self.exp_avg_sq, copy,
                                self.lr, self.betas[0], self.betas[1], self.eps, self.weight_decay,
                                self.steps, self._partials if clip else None, self.max_norm)
            self.arena.refresh_compute_copies(skip=copy)
            return loss.detach()
        if self.max_norm is not None:
            self._last_norm = self.arena.clip_(self.max_norm)
        self.optimizer.step()
        # the master weights changed: the compute-dtype copies follow (fused optimizers leave
        # the version counters alone, so this must be explicit)
        if self.flat:
            self.arena.refresh_compute_copies()
        else:
            self.model.post_optimizer_hook()
        return loss.detach()
