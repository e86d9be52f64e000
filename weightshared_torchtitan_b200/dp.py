"""Token data-parallel gradient exchange: one flat fp32 arena, one all-reduce per step.

Replaces the reference's DDP wrapper for this path: apply_ddp ->
replicate(model, device_mesh, bucket_cap_mb=100), torchtitan/models/llama3/infra/
parallelize.py:428-444, which averages every gradient across ranks through bucketed
all-reduces fired by autograd hooks. Here the fused kernels accumulate weight gradients in
place (no autograd hook ever fires for them), so all `param.grad` tensors are made views of
ONE contiguous fp32 buffer laid out

    [ shared base weights (unique blocks) | adapters of all layers | embedding | norms, head ]

and the whole buffer is averaged with a single all-reduce after backward. Weights are
replicated; forward and dX need no communication. With NCCL this is one ncclAllReduce over
NVLink/NVSwitch; the same code runs on gloo for CPU tests.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def _order_key(name: str) -> int:
    if name.startswith("blocks."):
        return 0
    if "_offset." in name:
        return 1
    if name.startswith("tok_embeddings."):
        return 2
    return 3


class GradArena:
    """Owns the flat gradient buffer of a model and points every param.grad into it."""

    def __init__(self, model: nn.Module, process_group: Optional[dist.ProcessGroup] = None):
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        named.sort(key=lambda np_: _order_key(np_[0]))   # stable: keeps registration order inside a class
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
        self.section_bounds = self._sections()
        self.master: Optional[torch.Tensor] = None      # flat fp32 parameters (flatten_parameters)
        self._copies = {}                                # dtype -> flat compute copy of `master`
        self._slot = {id(p): (off, p.numel()) for p, off in zip(self.params, self.offsets)}

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

    def _sections(self) -> List[Tuple[str, int, int]]:
        """(label, begin, end) element ranges of the four layout classes."""
        labels = ("shared", "adapters", "embedding", "other")
        out = []
        for cls, label in enumerate(labels):
            idx = [i for i, n in enumerate(self.names) if _order_key(n) == cls]
            if not idx:
                continue
            b = self.offsets[idx[0]]
            last = idx[-1]
            e = self.offsets[last] + (self.params[last].numel() + 63) // 64 * 64
            out.append((label, b, e))
        return out

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

    def all_reduce_mean(self) -> None:
        """Average the arena over the data-parallel ranks (no-op for a single process)."""
        if not dist.is_available() or not dist.is_initialized():
            return
        world = dist.get_world_size(self.group)
        if world == 1:
            return
        backend = dist.get_backend(self.group)
        if backend == "nccl":
            dist.all_reduce(self.buffer, op=dist.ReduceOp.AVG, group=self.group)
        else:   # gloo has no AVG
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM, group=self.group)
            self.buffer.div_(world)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of all gradients (identical on every rank after all_reduce_mean, so
        clipping needs no further collective: torchtitan/distributed/utils.py:369-372)."""
        return torch.linalg.vector_norm(self.buffer)

    def clip_(self, max_norm: float) -> torch.Tensor:
        norm = self.grad_norm()
        scale = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        self.buffer.mul_(scale)
        return norm


def broadcast_parameters(model: nn.Module, src: int = 0, group=None) -> None:
    """Make every rank's replica identical to rank `src` (weights are replicated in token DP)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    with torch.no_grad():
        for p in model.parameters():
            dist.broadcast(p.data, src=src, group=group)


def shard_tokens(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) sequence indices of a global batch owned by `rank` (contiguous split)."""
    if global_batch % world != 0:
        raise ValueError("global batch must divide evenly over the data-parallel ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per
