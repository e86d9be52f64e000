"""nn.Module surface of the path, mirroring the reference's names and argument meaning.

  LoRAModule        same constructor, attributes and forward as
                    torchtitan/models/llama3/model/model.py:148-192 (alpha = 2*rank, so the
                    scale alpha/rank is 2; w_a / w_b are nn.Linear(bias=False); *_override share
                    a Linear object between adapters). reset_parameters is the reference's
                    intent (kaiming-uniform A, zero B); the reference's own method raises
                    NameError because `math` is never imported there.
  broadcast_add     torchtitan/models/llama3/model/model.py:111-145.
  SharedLoRALinear  the fused drop-in for  broadcast_add(base(x), offset(x))  with equal
                    widths: holds REFERENCES to an existing nn.Linear (possibly shared by many
                    layers) and an existing LoRAModule, so parameter names, state_dict and
                    optimizers are unchanged.
  FactorizedEmbedding  nn.Embedding(V, r_e) -> nn.Linear(r_e, d, bias=False); not in the
                    reference (torchtitan/experiments/qwen3/model/model.py:350 is a full
                    nn.Embedding), named after its parts.

All compute goes through libwsl.so; CPU tensors raise.
"""
from __future__ import annotations

import math
import weakref
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
from torch.optim.optimizer import register_optimizer_step_post_hook

from . import functional as WF
from . import ops


def broadcast_add(base: torch.Tensor, delta: torch.Tensor, *, dim: int = -1, g: int = 1) -> torch.Tensor:
    """broadcast(base) + delta: `base` has g*D features, `delta` H*D; each group of H/g heads
    reuses one template. Same signature and result as the reference function."""
    if dim < 0:
        dim += base.dim()
    big, small = delta.shape[dim], base.shape[dim]
    assert big % small == 0, "delta and base feature dims incompatible"
    if big == small:
        return base + delta
    reps = big // small
    d_head = small // g
    lead, tail = list(base.shape[:dim]), list(base.shape[dim + 1:])
    b = base.reshape(*lead, g, 1, d_head, *tail)
    dl = delta.reshape(*lead, g, reps, d_head, *tail)
    return (b + dl).reshape(delta.shape)


class CopyCache:
    """Compute-dtype copies of master parameters, refreshed when the parameter changes.

    The reference runs fp32 master weights under torch.autocast(bfloat16)
    (torchtitan/distributed/utils.py:219-239), which re-casts every weight on every use. A
    base weight shared by L layers would be cast L times per pass; this cache casts once per
    optimizer step and hands every user the same bf16 tensor.

    A copy is re-cast when the parameter's version counter or address changed. Fused and
    foreach optimizers update parameters WITHOUT bumping the version counter, so the copies of
    every cache that is not bound to a source are also dropped after EVERY optimizer step of
    the process (a global post-step hook, registered below); the reference's
    post_optimizer_hook slot does the same explicitly. A cache bound with bind() is refreshed
    by the owner of its source in one pass instead.
    """

    _live: "weakref.WeakSet[CopyCache]" = weakref.WeakSet()

    def __init__(self):
        self._store: Dict[Tuple[int, ...], Tuple[Tuple[int, ...], torch.Tensor]] = {}
        self._source = None
        CopyCache._live.add(self)

    def bind(self, source) -> None:
        """`source.compute_view(param, dtype)` (dp.GradArena with flattened parameters) then
        supplies the copies: views of one flat buffer that the owner of the optimizer step
        re-casts in a single pass, instead of one cast per parameter keyed on its version."""
        self._source = source
        self._store.clear()

    def get(self, dtype: torch.dtype, *params: torch.Tensor) -> torch.Tensor:
        """Copy of `params` (concatenated along dim 0 if several) in `dtype`."""
        if len(params) == 1 and params[0].dtype == dtype:
            return params[0].detach()
        if self._source is not None and len(params) == 1:
            v = self._source.compute_view(params[0], dtype)
            if v is not None:
                return v
        key = tuple(id(p) for p in params) + (hash(dtype),)
        ver = tuple(p._version for p in params) + tuple(p.data_ptr() for p in params)
        hit = self._store.get(key)
        if hit is not None and hit[0] == ver:
            return hit[1]
        with torch.no_grad():
            src = params[0].detach() if len(params) == 1 else torch.cat([p.detach() for p in params], 0)
            c = src.to(dtype).contiguous()
        self._store[key] = (ver, c)
        return c

    def clear(self) -> None:
        """Drop the copies this cache made itself (they are re-cast on next use)."""
        self._store.clear()

    def invalidate(self) -> None:
        """The master parameters were changed by something other than the owner of the bound
        source (a checkpoint load, a broadcast, a re-initialisation): drop the cache's own
        copies AND re-cast the bound flat copy, whose views the kernels would otherwise keep
        reading with the old values."""
        self._store.clear()
        src = self._source
        if src is not None and getattr(src, "master", None) is not None:
            src.refresh_compute_copies()


def _drop_copies_after_optimizer_step(optimizer, args, kwargs) -> None:
    for cache in list(CopyCache._live):
        cache.clear()


register_optimizer_step_post_hook(_drop_copies_after_optimizer_step)

GLOBAL_COPY_CACHE = CopyCache()


def _compute_dtype(x: torch.Tensor) -> torch.dtype:
    if torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    return x.dtype


class LoRAModule(nn.Module):
    def __init__(self, in_dim, out_dim, rank=8, bias=False, w_a_override=None, w_b_override=None):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.rank = rank
        self.alpha = rank * 2
        self.bias = bias
        self.w_a = w_a_override if w_a_override is not None else nn.Linear(in_dim, rank, bias=False)
        self.w_b = w_b_override if w_b_override is not None else nn.Linear(rank, out_dim, bias=False)

    @property
    def scale(self) -> float:
        return self.alpha / self.rank

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.w_a.weight, a=math.sqrt(5))
        nn.init.zeros_(self.w_b.weight)

    def forward(self, x):
        dt = _compute_dtype(x)
        if dt not in (torch.bfloat16, torch.float32):
            raise TypeError(f"LoRAModule computes in bfloat16 or float32, not {dt}")
        A, B = self.w_a.weight, self.w_b.weight
        if A.dtype != dt:
            A, B = A.to(dt), B.to(dt)
        return WF.lora_delta(x.to(dt), A, B, self.scale)


class SharedLoRALinear(nn.Module):
    """y = base(x) + offset(x) as ONE fused projection (K-concatenated GEMM).

    `base` may be the same nn.Linear object in many SharedLoRALinear modules (cross-layer
    sharing); `offset` is this layer's LoRAModule. With `grad_in_place=True` (the training
    configuration) the fp32 gradients of base.weight, w_a.weight and w_b.weight are
    accumulated in place into `param.grad` (allocated as fp32 zeros on first use), so the
    shared weight collects all its users' contributions without per-use temporaries; autograd
    then sees no gradient for those parameters (hooks on them do not fire).
    """

    def __init__(self, base: nn.Linear, offset: LoRAModule, grad_in_place: bool = False,
                 cache: Optional[CopyCache] = None):
        super().__init__()
        if base.bias is not None:
            raise ValueError("SharedLoRALinear fuses bias-free projections only")
        if base.out_features != offset.out_dim or base.in_features != offset.in_dim:
            raise ValueError("fused path needs base and adapter of equal widths "
                             "(head-sharing modes keep the eager broadcast_add composition)")
        self.base = base
        self.offset = offset
        self.grad_in_place = grad_in_place
        self._cache = cache if cache is not None else GLOBAL_COPY_CACHE

    @property
    def in_features(self) -> int:
        return self.base.in_features

    @property
    def out_features(self) -> int:
        return self.base.out_features

    def _sink(self, p: torch.Tensor) -> Optional[torch.Tensor]:
        if not p.requires_grad:
            return None
        if p.grad is None:
            p.grad = torch.zeros(p.shape, device=p.device, dtype=torch.float32)
        if p.grad.dtype != torch.float32 or not p.grad.is_contiguous():
            raise RuntimeError("in-place gradient accumulation needs contiguous fp32 .grad buffers")
        return p.grad

    def forward(self, x):
        dt = _compute_dtype(x)
        if dt not in (torch.bfloat16, torch.float32):
            raise TypeError(f"SharedLoRALinear computes in bfloat16 or float32, not {dt}")
        W, A, B = self.base.weight, self.offset.w_a.weight, self.offset.w_b.weight
        s = self.offset.scale
        if self.grad_in_place and torch.is_grad_enabled():
            sinks = (self._sink(W), self._sink(A), self._sink(B))
            c = self._cache
            return WF.lora_linear(x.to(dt), c.get(dt, W), c.get(dt, A), c.get(dt, B), s,
                                  sinks=sinks, anchors=(W, A, B))
        if W.dtype != dt:
            W, A, B = W.to(dt), A.to(dt), B.to(dt)
        return WF.lora_linear(x.to(dt), W, A, B, s)


class FactorizedEmbedding(nn.Module):
    """tokens -> E_small[tokens] @ P^T with E_small [V, r_e] and P = proj.weight [d, r_e]."""

    def __init__(self, vocab_size: int, embed_rank: int, dim: int):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, embed_rank)
        self.proj = nn.Linear(embed_rank, dim, bias=False)

    def forward(self, tokens):
        E, P = self.embed.weight, self.proj.weight
        dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else E.dtype
        if E.dtype != dt:
            E, P = E.to(dt), P.to(dt)
        return factorized_embedding(tokens, E, P)


class FactorizedEmbeddingFunction(torch.autograd.Function):
    """Row gather + projection; backward = projection grads by the GEMM kernels and an fp32
    scatter-add of the gathered-row gradient."""

    @staticmethod
    def forward(ctx, tokens, E, P, sinks, anchor):
        # TMA gather inside the tcgen05 GEMM (the gathered rows never touch memory) where that
        # pays: every one of the d / 256 column tiles of the output gathers the rows again, and
        # a gather4 instruction moves 4 x 128 bytes where a tiled load moves 16 KiB, so for wide
        # outputs one pass of the row-gather kernel followed by the plain GEMM is faster
        fused = E.dtype == torch.bfloat16 and ops.embed_gather_in_gemm_pays(P.shape[0])
        if fused:
            h = ops.embed_fwd(tokens, E, P)
            ctx.save_for_backward(tokens, E, P)
        else:
            G = ops.embed_gather(tokens, E)
            h = ops.linear_fwd(G, P)
            ctx.save_for_backward(tokens, G, P)
        ctx.fused = fused
        ctx.e_shape = E.shape
        ctx.e_dtype = E.dtype
        ctx.sinks = sinks
        return h.view(*tokens.shape, P.shape[0])

    @staticmethod
    def backward(ctx, dH):
        tokens, GE, P = ctx.saved_tensors       # GE: E_small (fused) or the gathered rows
        d = dH.reshape(-1, dH.shape[-1])
        if d.stride(-1) != 1:
            d = d.contiguous()
        dG = ops.lora_linear_bwd_dx([d], [None], [P], [None])
        if ctx.sinks is not None:
            dE, dP = ctx.sinks
        else:
            dP = torch.zeros(P.shape, device=P.device, dtype=torch.float32)
            dE = torch.zeros(ctx.e_shape, device=P.device, dtype=torch.float32)
        if ctx.fused:
            ops.embed_bwd_dproj(tokens, d, GE, dP)
        else:
            ops.lora_linear_bwd_dw(d, None, GE, None, dP, None, None)
        ops.embed_scatter_add(tokens, dG, dE)
        if ctx.sinks is not None:
            return None, None, None, None, None
        return None, dE.to(ctx.e_dtype), dP.to(P.dtype), None, None


def factorized_embedding(tokens: torch.Tensor, E_small: torch.Tensor, P: torch.Tensor,
                         sinks=None, anchors=()) -> torch.Tensor:
    """sinks = (dE, dP) fp32 buffers to accumulate into in place (then E_small / P may be
    detached compute copies and `anchors` the master parameters that tie the graph)."""
    return FactorizedEmbeddingFunction.apply(tokens, E_small, P, sinks, WF._Anchor(tuple(anchors), P))
