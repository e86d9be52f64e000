"""Token data-parallel gradient exchange: one flat fp32 arena, all-reduced once per step.

Replaces the reference's DDP wrapper for this path: apply_ddp ->
replicate(model, device_mesh, bucket_cap_mb=100), torchtitan/models/llama3/infra/
parallelize.py:428-444, which averages every gradient across ranks through bucketed
all-reduces fired by autograd hooks and overlapped with the backward pass. Here the fused
kernels accumulate weight gradients in place (no autograd hook ever fires for them), so all
`param.grad` tensors are made views of ONE contiguous fp32 buffer, laid out in the order in
which the gradients become final during a step:

    [ output head | final norm, last layer | ... | layer l adapters + norms, and the shared
      block whose first user is layer l | ... | layer 0 | embedding ]

The buffer is averaged either with a single all-reduce after backward (all_reduce_mean), or
in buckets of contiguous ranges launched from the backward pass as soon as everything in
them is final (begin_overlap / notify_ready / finish_overlap), which hides the exchange
behind the remaining backward kernels as DDP's buckets do. Weights are replicated; forward
and dX need no communication. With NCCL these are ncclAllReduce calls over NVLink/NVSwitch;
the same code runs on gloo for CPU tests.
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def _order_key(name: str) -> int:
    """Layout class of a parameter when the model does not say when its gradients are final."""
    if name.startswith("blocks."):
        return 0
    if "_offset." in name:
        return 1
    if name.startswith("tok_embeddings."):
        return 2
    return 3


class GradArena:
    """Owns the flat gradient buffer of a model and points every param.grad into it.

    If the model has ``grad_ready_rank(name) -> int`` (WeightSharedDecoder does), parameters
    are laid out by that rank: rank k holds everything whose gradient is final once the model
    has reported ``grad_ready_hook(k)`` during backward. Otherwise the four layout classes
    (shared, adapters, embedding, other) are used and every range counts as final only at the
    end of backward.
    """

    def __init__(self, model: nn.Module, process_group: Optional[dist.ProcessGroup] = None):
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        rank_of: Callable[[str], int] = getattr(model, "grad_ready_rank", None) or _order_key
        self.has_ready_order = hasattr(model, "grad_ready_rank")
        named.sort(key=lambda np_: rank_of(np_[0]))   # stable: keeps registration order inside a rank
        for n, p in named:
            if p.dtype != torch.float32:
                raise TypeError(f"GradArena needs fp32 master parameters; {n} is {p.dtype}")
        self.names: List[str] = [n for n, _ in named]
        self.params: List[nn.Parameter] = [p for _, p in named]
        # 64-element (256-byte) alignment of every slice keeps the kernels' 16-byte rule.
        self.offsets: List[int] = []
        total = 0
        for p in self.params:
            self.offsets.append(total)
            total += (p.numel() + 63) // 64 * 64
        dev = self.params[0].device
        self.buffer = torch.zeros(total, device=dev, dtype=torch.float32)
        for p, off in zip(self.params, self.offsets):
            p.grad = self.buffer[off:off + p.numel()].view(p.shape)
        self.group = process_group
        # (rank, begin, end) element ranges, ascending in rank and contiguous
        self.ready_bounds: List[Tuple[int, int, int]] = []
        for n, p, off in zip(self.names, self.params, self.offsets):
            r = rank_of(n)
            end = off + (p.numel() + 63) // 64 * 64
            if self.ready_bounds and self.ready_bounds[-1][0] == r:
                self.ready_bounds[-1] = (r, self.ready_bounds[-1][1], end)
            else:
                self.ready_bounds.append((r, off, end))
        self.master: Optional[torch.Tensor] = None      # flat fp32 parameters (flatten_parameters)
        self._copies = {}                                # dtype -> flat compute copy of `master`
        self._slot = {id(p): (off, p.numel()) for p, off in zip(self.params, self.offsets)}
        # state of an overlapped exchange (begin_overlap .. finish_overlap)
        self._ov_active = False
        self._ov_sent = 0
        self._ov_ready = 0
        self._ov_bucket = 0
        self._ov_works: list = []
        self.on_bucket: Optional[Callable[[int], None]] = None   # called with the bytes of each bucket launched

    # ------------------------------------------------------------- flat master parameters
    def flatten_parameters(self) -> torch.Tensor:
        """Moves every parameter into ONE flat fp32 buffer with the arena's layout (param.data
        becomes a view of it), so that the optimizer, the clip and the refresh of the
        compute-dtype copies each run as one pass over one tensor. Call it before the optimizer
        is built. Returns the flat buffer."""
        if self.master is None:
            self.master = torch.zeros_like(self.buffer)
            with torch.no_grad():
                for p, off in zip(self.params, self.offsets):
                    v = self.master[off:off + p.numel()].view(p.shape)
                    v.copy_(p.data)
                    p.data = v
        return self.master

    def compute_view(self, p: torch.Tensor, dtype: torch.dtype) -> Optional[torch.Tensor]:
        """The compute-dtype copy of parameter `p` as a view of one flat buffer that
        refresh_compute_copies() re-casts from the master in a single pass; None when `p` is
        not in the arena or the parameters have not been flattened."""
        slot = self._slot.get(id(p))
        if slot is None or self.master is None:
            return None
        off, n = slot
        return self.compute_buffer(dtype)[off:off + n].view(p.shape)

    def compute_buffer(self, dtype: torch.dtype) -> torch.Tensor:
        """The flat compute copy in `dtype` (created on first use)."""
        buf = self._copies.get(dtype)
        if buf is None:
            buf = self.master.to(dtype)
            self._copies[dtype] = buf
        return buf

    def refresh_compute_copies(self, skip: Optional[torch.Tensor] = None) -> None:
        """After the optimizer changed the master parameters: one cast kernel per compute dtype
        (fused optimizers do not bump the tensors' version counters, so nothing else would
        notice the change). `skip`: a copy the optimizer kernel has already rewritten."""
        for buf in self._copies.values():
            if buf is not skip:
                buf.copy_(self.master)

    @property
    def nbytes(self) -> int:
        return self.buffer.numel() * 4

    def zero(self) -> None:
        """Replaces optimizer.zero_grad(): grads must stay attached to the arena."""
        self.buffer.zero_()

    def check_attached(self) -> None:
        for n, p, off in zip(self.names, self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.buffer.data_ptr() + 4 * off:
                raise RuntimeError(f"gradient of {n} was detached from the arena "
                                   "(zero_grad(set_to_none=True)?); call GradArena.zero() instead")

    def world_size(self) -> int:
        if not dist.is_available() or not dist.is_initialized():
            return 1
        return dist.get_world_size(self.group)

    def _reduce_range(self, begin: int, end: int, async_op: bool):
        """Average buffer[begin:end] over the ranks; returns the work handle when async."""
        view = self.buffer[begin:end]
        if dist.get_backend(self.group) == "nccl":
            return dist.all_reduce(view, op=dist.ReduceOp.AVG, group=self.group, async_op=async_op)
        # gloo has no AVG: sum, then divide once the sum is there
        work = dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        if not async_op:
            view.div_(self.world_size())
            return None
        return _DivideAfter(work, view, self.world_size())

    def all_reduce_mean(self) -> None:
        """Average the arena over the data-parallel ranks (no-op for a single process)."""
        if self.world_size() == 1:
            return
        self._reduce_range(0, self.buffer.numel(), async_op=False)

    # ---------------------------------------------- exchange overlapped with the backward pass
    def begin_overlap(self, bucket_bytes: int = 256 << 20) -> None:
        """Start of a step whose gradients are exchanged in buckets while backward still runs.
        Ranges are launched (asynchronously, on the backend's own stream, ordered after the
        kernels already enqueued on the current stream) once at least `bucket_bytes` of
        contiguous final gradients are pending."""
        self._ov_active = self.world_size() > 1
        self._ov_sent = 0
        self._ov_ready = 0
        self._ov_bucket = max(int(bucket_bytes) // 4, 1)
        self._ov_works = []

    def notify_ready(self, rank: int) -> None:
        """Everything of ready-rank <= `rank` is final (the model's grad_ready_hook)."""
        if not self._ov_active:
            return
        for r, b, e in self.ready_bounds:
            if r <= rank and e > self._ov_ready:
                self._ov_ready = e
        self._launch_pending(force=False)

    def _launch_pending(self, force: bool) -> None:
        n = self._ov_ready - self._ov_sent
        if n <= 0 or (not force and n < self._ov_bucket):
            return
        work = self._reduce_range(self._ov_sent, self._ov_ready, async_op=True)
        self._ov_works.append(work)
        if self.on_bucket is not None:
            self.on_bucket(4 * n)
        self._ov_sent = self._ov_ready

    def finish_overlap(self) -> None:
        """End of backward: launch what is left and make the current stream wait for every
        bucket. Afterwards the whole arena holds the averaged gradients."""
        if not self._ov_active:
            return
        self._ov_ready = self.buffer.numel()
        self._launch_pending(force=True)
        for w in self._ov_works:
            w.wait()
        self._ov_works = []
        self._ov_active = False

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of all gradients (identical on every rank after all_reduce_mean, so
        clipping needs no further collective: torchtitan/distributed/utils.py:369-372)."""
        return torch.linalg.vector_norm(self.buffer)

    def clip_(self, max_norm: float) -> torch.Tensor:
        norm = self.grad_norm()
        scale = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        self.buffer.mul_(scale)
        return norm


class _DivideAfter:
    """Work handle of a summing all-reduce whose result still has to be divided (gloo)."""

    def __init__(self, work, view: torch.Tensor, world: int):
        self.work, self.view, self.world = work, view, world

    def wait(self) -> None:
        self.work.wait()
        self.view.div_(self.world)


def broadcast_parameters(model: nn.Module, src: int = 0, group=None) -> None:
    """Make every rank's replica identical to rank `src` (weights are replicated in token DP)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    with torch.no_grad():
        for p in model.parameters():
            dist.broadcast(p.data, src=src, group=group)
    # compute-dtype copies of the old values (also a flat copy bound to an arena) must follow
    hook = getattr(model, "post_optimizer_hook", None)
    if callable(hook):
        hook()


def shard_tokens(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) sequence indices of a global batch owned by `rank` (contiguous split)."""
    if global_batch % world != 0:
        raise ValueError("global batch must divide evenly over the data-parallel ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per
