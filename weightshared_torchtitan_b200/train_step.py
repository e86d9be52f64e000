"""One optimisation step of the weight-shared decoder under token data parallelism.

Mirrors the order of Trainer.train_step / forward_backward_step in the reference
(torchtitan/train.py:404-527): zero grads -> forward + loss -> backward -> gradient
averaging over the data-parallel ranks -> clip -> optimizer step. The averaging is an
all-reduce of the flat arena (dp.GradArena) instead of DDP's bucketed hooks: either one call
after backward, or buckets launched from inside backward as their gradients become final
(``overlap=True``, what DDP's buckets do, torchtitan/models/llama3/infra/parallelize.py:428-444).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from . import _lib, ops
from .decoder import WeightSharedDecoder
from .dp import GradArena


class TrainStep:
    """All parameters live in one flat fp32 buffer with the layout of the gradient arena
    (``flat=True``). On a GPU the clip, AdamW and the refresh of the bf16 compute copies of
    the weights are then ONE pass over the arenas after one pass over the gradients for the
    norm (``fused_update=True``: wsl_grad_sumsq_partials + wsl_adamw_flat_step); with
    ``fused_update=False`` torch.optim.AdamW steps the flat tensor and one cast kernel
    refreshes the copies. ``flat=False`` keeps per-parameter storage and lets the model re-cast
    its copies one by one (the reference's post_optimizer_hook slot).

    ``lr`` may be a float or a callable ``step -> float`` (the slot of the reference's
    LR scheduler, torchtitan/components/lr_scheduler.py); a per-call ``lr=`` overrides both.

    ``overlap=True`` exchanges gradients in buckets of ``bucket_bytes`` while backward runs.
    The collective's kernel shares the SMs with the library's GEMMs. With ``reserved_sms`` > 0
    the GEMMs leave that many SMs free while a bucket is estimated to be in flight (option
    RESERVED_SMS of the library; ``link_gbs`` is the all-reduce rate used for that estimate).
    Measured at 2 GPUs this gave nothing over plain overlap (the GEMM grids of two waves
    already yield SMs gracefully), so the default is 0.

    ``status_every`` > 0: every that many steps the device status words are read (this waits
    for the device) and a bounded wait that ran out in any kernel since raises WslError.
    """

    def __init__(self, model: WeightSharedDecoder, lr=3e-4, weight_decay: float = 0.1,
                 max_norm: Optional[float] = 1.0, process_group=None, flat: bool = True,
                 fused_update: bool = True, overlap: bool = False, bucket_bytes: int = 256 << 20,
                 reserved_sms: int = 0, link_gbs: float = 300.0, status_every: int = 64):
        self.model = model
        self.arena = GradArena(model, process_group)
        self.flat = bool(flat)
        self.lr = lr
        self.weight_decay, self.betas, self.eps = weight_decay, (0.9, 0.95), 1e-8
        self.max_norm = max_norm
        self.fused_update = bool(fused_update) and self.flat and self.arena.buffer.is_cuda
        self.optimizer = None
        self.steps = 0
        self.status_every = int(status_every)
        self.overlap = bool(overlap) and self.arena.has_ready_order
        self.bucket_bytes = int(bucket_bytes)
        self.reserved_sms = int(reserved_sms)
        self.link_gbs = float(link_gbs)
        self.timing: Optional[Dict[str, list]] = None    # set to {} to collect all-reduce events
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
        self.optimizer = torch.optim.AdamW(opt_params, lr=self._lr_at(1), betas=self.betas, eps=self.eps,
                                           weight_decay=weight_decay, fused=self.arena.buffer.is_cuda)

    # ------------------------------------------------------------------------- helpers
    def _lr_at(self, step: int) -> float:
        return float(self.lr(step)) if callable(self.lr) else float(self.lr)

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step, before clipping."""
        if self.fused_update:
            return self._partials.sum().sqrt()
        return self._last_norm

    def check_status(self) -> None:
        """Raise WslError if a bounded device-side wait ran out in any kernel so far (the words
        name the role, block and work unit). Waits for the device."""
        if not self.arena.buffer.is_cuda:
            return
        torch.cuda.synchronize()
        st, words = _lib.poll_status()
        if st != 0:
            raise _lib.WslError(st, f"device status words {words} (role, block, unit)")

    # ------------------------------------------------------------------ checkpoint state
    def _torch_moments(self, p: torch.Tensor):
        """(exp_avg, exp_avg_sq) of torch.optim.AdamW for parameter `p`, created as zeros when the
        optimizer has not stepped yet."""
        st = self.optimizer.state[p]
        if "exp_avg" not in st:
            fused = self.arena.buffer.is_cuda
            st["step"] = (torch.zeros((), dtype=torch.float32, device=p.device) if fused
                          else torch.tensor(0.0, dtype=torch.float32))
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st["exp_avg"], st["exp_avg_sq"]

    def _moment_views(self):
        """name -> (exp_avg, exp_avg_sq) views per parameter, whatever the optimizer's layout."""
        out = {}
        if self.fused_update or self.flat:
            if self.fused_update:
                m, v = self.exp_avg, self.exp_avg_sq
            else:
                m, v = self._torch_moments(self._flat_param)
            for n, p, off in zip(self.arena.names, self.arena.params, self.arena.offsets):
                k = p.numel()
                out[n] = (m[off:off + k].view(p.shape), v[off:off + k].view(p.shape))
        else:
            for n, p in zip(self.arena.names, self.arena.params):
                out[n] = self._torch_moments(p)
        return out

    def state_dict(self) -> Dict[str, object]:
        """Optimizer state of the step in one layout for all three optimizer paths: the step
        count (bias correction), the learning rate when it is a constant and, per parameter
        under its arena name, the two AdamW moments -- the content of torch.optim.AdamW's state
        ('step', 'exp_avg', 'exp_avg_sq'), so a run resumes with warm moments as the reference
        does through OptimizersContainer (torchtitan/components/optimizer.py) and its
        checkpointer. The tensors are views of the live state."""
        out: Dict[str, object] = {"steps": self.steps, "lr": None if callable(self.lr) else float(self.lr)}
        for n, (m, v) in self._moment_views().items():
            out[f"exp_avg.{n}"] = m
            out[f"exp_avg_sq.{n}"] = v
        return out

    @torch.no_grad()
    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.steps = int(sd["steps"])
        if sd.get("lr") is not None and not callable(self.lr):
            self.lr = float(sd["lr"])
        for n, (m, v) in self._moment_views().items():
            m.copy_(sd[f"exp_avg.{n}"])
            v.copy_(sd[f"exp_avg_sq.{n}"])
        if self.optimizer is not None:
            for st in self.optimizer.state.values():
                if "step" in st:
                    st["step"].fill_(float(self.steps))

    # ------------------------------------------------------------------------ the step
    def _bucket_launched(self, nbytes: int) -> None:
        """A bucket went to the collective's stream: the GEMMs enqueued from now on share the
        GPU with it for about nbytes / link rate; they leave SMs free for that long."""
        if self.reserved_sms > 0 and self.arena.buffer.is_cuda:
            ops.reserve_sms(self.reserved_sms, 1.5 * nbytes / (self.link_gbs * 1e6))

    def gradients(self, tokens: torch.Tensor, labels: torch.Tensor, exchange: bool = True) -> torch.Tensor:
        """Zero the arena, forward + loss + backward and (``exchange``) the gradient average over
        the data-parallel ranks, without the optimizer step: afterwards ``arena.buffer`` holds the
        gradients the optimizer would see. Returns the detached loss of this rank's batch."""
        arena = self.arena
        overlap = exchange and self.overlap and arena.world_size() > 1
        arena.zero()
        if overlap:
            arena.on_bucket = self._bucket_launched
            arena.begin_overlap(self.bucket_bytes)
            self.model.grad_ready_hook = arena.notify_ready
        try:
            loss = self.model.loss(tokens, labels)
            if overlap:
                arena.notify_ready(0)        # the head's gradient is final before backward starts
            loss.backward()
        finally:
            self.model.grad_ready_hook = None
        ev = None
        if self.timing is not None and arena.buffer.is_cuda:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if overlap:
            arena.finish_overlap()
            ops.reserve_sms(0, 0.0)
        elif exchange:
            arena.all_reduce_mean()
        if ev is not None:
            ev[1].record()
            self.timing.setdefault("allreduce_wait", []).append(ev)
        return loss.detach()

    def __call__(self, tokens: torch.Tensor, labels: torch.Tensor, lr: Optional[float] = None) -> torch.Tensor:
        arena = self.arena
        loss = self.gradients(tokens, labels, exchange=True)
        self.steps += 1
        step_lr = float(lr) if lr is not None else self._lr_at(self.steps)
        if self.fused_update:
            clip = self.max_norm is not None
            if clip:
                ops.grad_sumsq_partials(arena.buffer, self._partials)
            copy = arena.compute_buffer(self.model.compute_dtype) \
                if self.model.compute_dtype == torch.bfloat16 else None
            ops.adamw_flat_step(arena.master, arena.buffer, self.exp_avg, self.exp_avg_sq, copy,
                                step_lr, self.betas[0], self.betas[1], self.eps, self.weight_decay,
                                self.steps, self._partials if clip else None, self.max_norm)
            arena.refresh_compute_copies(skip=copy)
        else:
            if self.max_norm is not None:
                self._last_norm = arena.clip_(self.max_norm)
            for grp in self.optimizer.param_groups:
                grp["lr"] = step_lr
            self.optimizer.step()
            # the master weights changed: the compute-dtype copies follow (fused optimizers leave
            # the version counters alone, so this must be explicit)
            if self.flat:
                arena.refresh_compute_copies()
            else:
                self.model.post_optimizer_hook()
        if self.status_every > 0 and self.steps % self.status_every == 0:
            self.check_status()
        return loss
