"""torch.autograd.Function wrappers of the fused shared-W + LoRA projection.

Shaped like the reference's own kernel-backed Functions (GroupedGemmMg,
torchtitan/experiments/kernels/triton_mg_group_gemm/torchao_pr/mg_grouped_gemm.py:1202-1300:
``forward(ctx, tensors..., non-tensor args)``, ``ctx.save_for_backward``, ``backward`` returning
one entry per forward argument, plus a functional wrapper that calls ``.apply``).

The arithmetic replaces base(x) + LoRAModule.forward(x) and its autograd graph
(torchtitan/models/llama3/model/model.py:111-145,189-192,392-398).

Weight gradients can go two ways:
  * returned to autograd as fresh tensors (default; drop-in for any optimizer setup), or
  * accumulated IN PLACE into caller-owned fp32 buffers ("sinks"), which is how one shared
    base weight collects the contributions of every layer that reuses it without a
    temporary per use. Then ``None`` is returned for those inputs.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch

from . import ops

Sinks = Optional[Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]]


def _flat(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


# When the shared weight is trained (dW wanted together with dA and dB, bf16), the backward
# can go through the layer's own weight gradient G = dY^T x: dB = s G A^T, dA = s B^T G and
# dX = dY (W + s B A). That reads [N, K] matrices (merge W, copy G, two passes over G for the
# adapter gradients) instead of streaming the M token rows again (pre-pass over dY, rank-r
# regions of the weight-gradient launch and of dX), so it pays when M is large against
# N K / (N + K). "auto" decides per projection group; True / False (environment variable
# WSL_DERIVED_ADAPTER_GRADS=1 / 0) force one formulation where eligible.
_env = os.environ.get("WSL_DERIVED_ADAPTER_GRADS", "auto")
DERIVED_ADAPTER_GRADS = {"0": False, "1": True}.get(_env, "auto")

# Which formulation is faster, measured on a B200 with `python bench.py --routes` (fwd+bwd of
# the group through the autograd Function) for every projection group of the four baseline
# configurations at their own token counts: (M, K, (N_0, ...), r) -> through the layer gradient?
ROUTE_TABLE = {
    # configuration 1 (0.6B shape, 32768 tokens, r 16): q|k|v, o, gate|up, down
    (32768, 1024, (2048, 1024, 1024), 16): True,     # 0.82 -> 0.71 ms
    (32768, 2048, (1024,), 16): True,                # 0.43 -> 0.43
    (32768, 1024, (3072, 3072), 16): True,           # 1.11 -> 1.00
    (32768, 3072, (1024,), 16): True,                # 0.66 -> 0.63
    # configuration 2 (1.7B shape, 32768 tokens, r 32)
    (32768, 2048, (2048, 1024, 1024), 32): True,     # 1.41 -> 1.27
    (32768, 2048, (2048,), 32): True,                # 0.77 -> 0.74
    (32768, 2048, (6144, 6144), 32): True,           # 4.12 -> 3.80
    (32768, 6144, (2048,), 32): True,                # 1.96 -> 1.88
    # configuration 3 (4B shape, 32768 tokens, r 64)
    (32768, 2560, (4096, 1024, 1024), 64): True,     # 2.56 -> 2.45
    (32768, 4096, (2560,), 64): True,                # 1.91 -> 1.80
    (32768, 2560, (9728, 9728), 64): True,           # 8.36 -> 8.15
    (32768, 9728, (2560,), 64): True,                # 3.96 -> 3.91
    # configuration 4 (8B shape, 16384 tokens, r 64)
    (16384, 4096, (4096, 1024, 1024), 64): True,     # 2.27 -> 2.23
    (16384, 4096, (4096,), 64): False,               # 1.27 <- 1.36
    (16384, 4096, (12288, 12288), 64): True,         # 8.43 -> 8.34
    (16384, 12288, (4096,), 64): False,              # 3.99 <- 4.07
    # the gate (or up) projection of configuration 4 on its own, the isolated-op headline shape
    (16384, 4096, (12288,), 64): True,               # 3.87 -> 3.76
}

# Shapes outside the table: the form through G trades passes over M-row activations (the
# pre-pass over dY, the rank-r regions) for passes over [N, K] matrices (merged weight, bf16
# copy of G, two reads of G), so what decides is the token count against the input width. In
# the table the form through G wins clearly from M / K ~ 5 upwards and loses below ~ 4.
_MIN_TOKENS_PER_INPUT_WIDTH = 5.0


def derived_route_pays(M: int, K: int, Ns, r: int) -> bool:
    """True when the backward of this projection group should go through the layer's own weight
    gradient (see ROUTE_TABLE)."""
    hit = ROUTE_TABLE.get((int(M), int(K), tuple(int(n) for n in Ns), int(r)))
    if hit is not None:
        return hit
    return M >= _MIN_TOKENS_PER_INPUT_WIDTH * K


class AdapterGradBatch:
    """Collects the adapter-gradient work (dA += s B^T G, dB += s G A^T) of several projection
    groups and runs it in ONE call of two launches instead of one call per group; the products
    are tiny and launch-bound, so a decoder layer hands the same batch to its four groups.

    ``expected`` = number of groups that will report; the batch runs when the last one has.
    If fewer report (a group got no gradient), what is pending runs when the backward pass
    ends (an autograd engine callback), or when ``flush()`` is called.
    """

    def __init__(self, expected: int):
        self.expected = int(expected)
        self.count = 0
        self.s: Optional[float] = None
        self.pending: List[tuple] = []

    def add(self, dWls, As, Bs, dAs, dBs, s: float) -> None:
        if self.s is not None and self.s != s:
            self.flush()
        self.s = s
        if not self.pending:
            # safety net: whatever is still pending when this backward pass ends runs then
            torch.autograd.Variable._execution_engine.queue_callback(self.flush)
        self.pending += list(zip(dWls, As, Bs, dAs, dBs))
        self.count += 1
        if self.count >= self.expected:
            self.flush()

    def nothing_to_add(self) -> None:
        """A group that computed its adapter gradients itself (direct formulation) still counts,
        so that the others do not wait for the end of the backward pass."""
        self.count += 1
        if self.count >= self.expected:
            self.flush()

    def flush(self) -> None:
        todo, self.pending, self.count = self.pending, [], 0
        if not todo:
            return
        for i in range(0, len(todo), ops.MAX_ADAPTER_PROJ):
            g, a, b, da, db = zip(*todo[i:i + ops.MAX_ADAPTER_PROJ])
            ops.lora_adapter_grads_from_dw(g, a, b, da, db, self.s)


class LoRALinearGroupFunction(torch.autograd.Function):
    """P projections that read the same x: y_p = x W_p^T + s (x A_p^T) B_p^T, p < P <= 3.

    forward(ctx, x, s, sinks, anchors, batch, W_0, A_0, B_0, W_1, A_1, B_1, ...) -> (y_0, ..., y_{P-1})

    ``batch`` is None or an AdapterGradBatch shared with other groups (see there).

    ``sinks`` is None or a list of P triples (dW, dA, dB) of fp32 buffers to accumulate into.
    ``anchors`` is a tuple of tensors that only tie the output to the autograd graph (the
    fp32 master parameters when W/A/B are detached compute copies); they get no gradient.
    """

    @staticmethod
    def forward(ctx, x, s, sinks, anchors, batch, *wab):
        P = len(wab) // 3
        ctx.batch = batch
        Ws, As, Bs = list(wab[0::3]), list(wab[1::3]), list(wab[2::3])
        ctx.empty = x.numel() == 0
        if ctx.empty:
            # no tokens: nothing to launch, every gradient contribution is zero
            ctx.P, ctx.x_shape, ctx.sinks = P, x.shape, sinks
            ctx.save_for_backward(*wab)
            return tuple(x.new_zeros(*x.shape[:-1], W.shape[0]) for W in Ws)
        x2 = _flat(x)
        if not x2.is_contiguous() and x2.stride(-1) != 1:
            x2 = x2.contiguous()
        A_cat = As[0] if P == 1 else torch.cat(As, dim=0)
        T_cat = ops.lora_prepass(x2, A_cat, s)
        ys, Ts = [], []
        off = 0
        for p in range(P):
            r = As[p].shape[0]
            Ts.append(T_cat[:, off:off + r])
            off += r
        if P > 1 and x2.dtype == torch.bfloat16 and len({A.shape[0] for A in As}) == 1:
            ys = [y.view(*x.shape[:-1], y.shape[1]) for y in ops.lora_linear_fwd_group(x2, Ws, Ts, Bs)]
        else:
            for p in range(P):
                ys.append(ops.lora_linear_fwd(x2, Ws[p], Ts[p], Bs[p]).view(*x.shape[:-1], Ws[p].shape[0]))
        ctx.derived = _derived_route(x2, sinks, Ws, As)
        ctx.save_for_backward(x2, None if ctx.derived else T_cat, *wab)
        ctx.s = float(s)
        ctx.sinks = sinks
        ctx.P = P
        ctx.x_shape = x.shape
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dYs):
        if ctx.empty:
            if ctx.batch is not None:
                ctx.batch.nothing_to_add()
            wab = ctx.saved_tensors
            dX = wab[0].new_zeros(ctx.x_shape) if ctx.needs_input_grad[0] else None
            grads = [None] * (3 * ctx.P)
            if ctx.sinks is None:
                grads = [torch.zeros_like(w) if need else None
                         for w, need in zip(wab, ctx.needs_input_grad[5:])]
            return (dX, None, None, None, None, *grads)
        x2, T_cat, *wab = ctx.saved_tensors
        return _group_backward(ctx, x2, T_cat, wab, dYs)


def _group_backward(ctx, x2, T_cat, wab, dYs):
    """Backward of P projections that read the same x (shared by LoRALinearGroupFunction and
    the gate|up + SwiGLU Function): returns the gradient tuple of
    (x, s, sinks, anchors, batch, W_0, A_0, B_0, ...)."""
    P = ctx.P
    Ws, As, Bs = list(wab[0::3]), list(wab[1::3]), list(wab[2::3])
    if ctx.derived:
        dY2 = []
        for p in range(P):
            d = dYs[p]
            if d is None:
                d = torch.zeros(x2.shape[0], Ws[p].shape[0], device=x2.device, dtype=x2.dtype)
            d = _flat(d)
            if d.stride(-1) != 1:
                d = d.contiguous()
            dY2.append(d)
        dX = None
        if ctx.needs_input_grad[0]:
            if len({A.shape[0] for A in As}) == 1:
                Weffs = ops.lora_merge_weight(Ws, As, Bs, ctx.s)
            else:
                Weffs = [ops.lora_merge_weight([Ws[p]], [As[p]], [Bs[p]], ctx.s)[0] for p in range(P)]
            dX = ops.lora_linear_bwd_dx(dY2, [None] * P, Weffs, [None] * P).view(ctx.x_shape)
        dWls = ops.bwd_dw_layer_group(dY2, x2, [t[0] for t in ctx.sinks])
        if ctx.batch is not None:
            ctx.batch.add(dWls, As, Bs, [t[1] for t in ctx.sinks], [t[2] for t in ctx.sinks], ctx.s)
        else:
            ops.lora_adapter_grads_from_dw(dWls, As, Bs, [t[1] for t in ctx.sinks],
                                           [t[2] for t in ctx.sinks], ctx.s)
        return (dX, None, None, None, None, *([None] * (3 * P)))
    if ctx.batch is not None:
        ctx.batch.nothing_to_add()
    dY2, Us = [], []
    # the U of all projections side by side, so that dX contracts [U_0 | U_1 | ...] with
    # the stacked A matrices in ONE rank-sum segment instead of one tiny segment each
    r_tot = sum(A.shape[0] for A in As)
    U_cat = torch.empty(x2.shape[0], r_tot, device=x2.device, dtype=x2.dtype)
    off = 0
    for p in range(P):
        d = dYs[p]
        if d is None:
            d = torch.zeros(x2.shape[0], Ws[p].shape[0], device=x2.device, dtype=x2.dtype)
        d = _flat(d)
        if d.stride(-1) != 1:
            d = d.contiguous()
        dY2.append(d)
        r = As[p].shape[0]
        Us.append(ops.lora_bwd_prepass(d, Bs[p], ctx.s, out=U_cat[:, off:off + r]))
        off += r
    dX = None
    if ctx.needs_input_grad[0]:
        if P == 1:
            dX = ops.lora_linear_bwd_dx(dY2, Us, Ws, As)
        else:
            A_cat = torch.cat(As, dim=0)
            dX = ops.lora_linear_bwd_dx(dY2, [U_cat] + [None] * (P - 1), Ws, [A_cat] + [None] * (P - 1))
        dX = dX.view(ctx.x_shape)
    grads: List[Optional[torch.Tensor]] = []
    off = 0
    if (ctx.sinks is not None and P > 1 and x2.dtype == torch.bfloat16
            and all(s[0] is not None and s[1] is not None and s[2] is not None for s in ctx.sinks)):
        # all projections of the group in one weight-gradient launch
        Ts = []
        for p in range(P):
            r = As[p].shape[0]
            Ts.append(T_cat[:, off:off + r])
            off += r
        ops.lora_linear_bwd_dw_group(dY2, Us, x2, Ts, [s[0] for s in ctx.sinks],
                                     [s[1] for s in ctx.sinks], [s[2] for s in ctx.sinks])
        return (dX, None, None, None, None, *([None] * (3 * P)))
    for p in range(P):
        r = As[p].shape[0]
        T = T_cat[:, off:off + r]
        off += r
        if ctx.sinks is not None:
            dW, dA, dB = ctx.sinks[p]
            if dW is not None or dA is not None or dB is not None:
                ops.lora_linear_bwd_dw(dY2[p], Us[p], x2, T, dW, dA, dB)
            grads += [None, None, None]
        else:
            need = ctx.needs_input_grad[5 + 3 * p: 8 + 3 * p]
            dev = x2.device
            dW = torch.zeros(Ws[p].shape, device=dev, dtype=torch.float32) if need[0] else None
            dA = torch.zeros(As[p].shape, device=dev, dtype=torch.float32) if need[1] else None
            dB = torch.zeros(Bs[p].shape, device=dev, dtype=torch.float32) if need[2] else None
            if any(need):
                ops.lora_linear_bwd_dw(dY2[p], Us[p], x2, T, dW, dA, dB)
            grads += [g.to(w.dtype) if g is not None else None
                      for g, w in ((dW, Ws[p]), (dA, As[p]), (dB, Bs[p]))]
    return (dX, None, None, None, None, *grads)


def _derived_route(x2, sinks, Ws, As) -> bool:
    """Whether the backward of this group goes through the layer's own weight gradient."""
    return (DERIVED_ADAPTER_GRADS is not False and sinks is not None and x2.dtype == torch.bfloat16
            and all(t[0] is not None and t[1] is not None and t[2] is not None for t in sinks)
            and all(A.shape[0] in ops.MERGE_RANKS for A in As)
            and (DERIVED_ADAPTER_GRADS is True
                 or derived_route_pays(x2.shape[0], x2.shape[1], [W.shape[0] for W in Ws], As[0].shape[0])))


class LoRAGateUpSwiGLUFunction(torch.autograd.Function):
    """h = silu(x W_g^T + s (x A_g^T) B_g^T) * (x W_u^T + s (x A_u^T) B_u^T): the gate and up
    projections of the MLP and the activation in one launch
    (``w2(F.silu(w1(x)) * w3(x))`` without the w2, torchtitan/experiments/qwen3/model/model.py:251).

    forward(ctx, x, s, sinks, anchors, batch, W_g, A_g, B_g, W_u, A_u, B_u) -> h

    The accumulator tile of the GEMM holds matching columns of gate and up side by side, so the
    activation is applied in the epilogue; gate and up are still written once (bf16) because the
    backward needs them: d gate = dh u silu'(gate), d up = dh silu(gate), then the backward of a
    two-projection group. Results are bit-identical to lora_linear_group followed by swiglu."""

    @staticmethod
    def forward(ctx, x, s, sinks, anchors, batch, Wg, Ag, Bg, Wu, Au, Bu):
        x2 = _flat(x)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        T_cat = ops.lora_prepass(x2, torch.cat((Ag, Au), dim=0), s)
        g, u, h = ops.lora_swiglu_fwd(x2, Wg, Wu, T_cat, Bg, Bu)
        ctx.P = 2
        ctx.batch = batch
        ctx.s = float(s)
        ctx.sinks = sinks
        ctx.x_shape = x.shape
        ctx.derived = _derived_route(x2, sinks, [Wg, Wu], [Ag, Au])
        ctx.save_for_backward(x2, None if ctx.derived else T_cat, Wg, Ag, Bg, Wu, Au, Bu, g, u)
        return h.view(*x.shape[:-1], Wg.shape[0])

    @staticmethod
    def backward(ctx, dh):
        x2, T_cat, *rest = ctx.saved_tensors
        wab, (g, u) = rest[:6], rest[6:]
        d = _flat(dh)
        if not d.is_contiguous():
            d = d.contiguous()
        dg, du = ops.swiglu_bwd(d, g, u)
        return _group_backward(ctx, x2, T_cat, wab, (dg, du))


# The derivative of the activation can ride in the epilogue of the down projection's
# input-gradient GEMM (ops.lora_linear_bwd_dx_swiglu) or run as its own pass over dh, g, u.
# The four epilogue warps of a CTA spend ~16 instructions per element on it, which the main
# loop hides only when the contraction (the model width d) is long: measured on B200 at the
# configuration-4 MLP shape (d = 4096, 16384 tokens) 1.23 ms against 1.58 ms for GEMM + kernel,
# at the configuration-3 shape (d = 2560, 32768 tokens) 1.59 against 1.80 ms, at the
# configuration-2 shape (d = 2048) 1.00 against 0.97 ms and at the configuration-1 shape
# (d = 1024) 0.33 against 0.30 ms. "auto" takes the epilogue form from d = 2560;
# WSL_FUSE_SWIGLU_BWD=0 / 1 forces one.
_env_fuse = os.environ.get("WSL_FUSE_SWIGLU_BWD", "auto")
FUSE_SWIGLU_BWD = {"0": False, "1": True}.get(_env_fuse, "auto")
_FUSE_SWIGLU_BWD_MIN_WIDTH = 2560


def _down_dx_with_activation_grad(d, U2, W, A, g, u):
    """(d gate, d up) from the down projection's output gradient d [M, width]."""
    fuse = FUSE_SWIGLU_BWD if FUSE_SWIGLU_BWD != "auto" else d.shape[1] >= _FUSE_SWIGLU_BWD_MIN_WIDTH
    if fuse:
        return ops.lora_linear_bwd_dx_swiglu(d, U2, W, A, g, u)
    dh = ops.lora_linear_bwd_dx([d], [U2], [W], [A])
    return ops.swiglu_bwd(dh, g, u)


class _GroupCtx:
    """The fields _group_backward reads, for a projection group that is part of a larger Function."""

    def __init__(self, P, derived, s, sinks, batch, x_shape, need_x):
        self.P, self.derived, self.s, self.sinks, self.batch, self.x_shape = P, derived, s, sinks, batch, x_shape
        self.needs_input_grad = (need_x,) + (False,) * (4 + 3 * P)


class LoRAMLPFunction(torch.autograd.Function):
    """The whole SwiGLU MLP, y = down(silu(gate(x)) * up(x)) with a shared base weight plus a
    per-layer adapter on each of the three projections
    (``w2(F.silu(w1(x)) * w3(x))``, torchtitan/experiments/qwen3/model/model.py:251), as one
    autograd node so that the activation can ride in GEMM epilogues both ways:

      forward   gate|up GEMM whose epilogue writes g, u and h = silu(g) u; down GEMM on h
      backward  the down projection's input gradient, then d gate and d up (as one launch whose
                epilogue applies the activation's derivative when FUSE_SWIGLU_BWD is set, else
                the GEMM followed by the stand-alone kernel), the weight gradients of down and
                the backward of the gate|up group

    forward(ctx, x, s, sinks, anchors, batch, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd) -> y
    ``sinks`` = three (dW, dA, dB) triples of fp32 buffers (gate, up, down), accumulated in place;
    ``batch`` = AdapterGradBatch shared with the layer's other groups (this node reports twice).
    Bit-identical to lora_gate_up_swiglu followed by lora_linear_group for the down projection."""

    @staticmethod
    def forward(ctx, x, s, sinks, anchors, batch, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd):
        x2 = _flat(x)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        T_cat = ops.lora_prepass(x2, torch.cat((Ag, Au), dim=0), s)
        g, u, h = ops.lora_swiglu_fwd(x2, Wg, Wu, T_cat, Bg, Bu)
        T2 = ops.lora_prepass(h, Ad, s)
        y = ops.lora_linear_fwd(h, Wd, T2, Bd)
        ctx.s, ctx.sinks, ctx.batch, ctx.x_shape = float(s), sinks, batch, x.shape
        ctx.derived_gu = _derived_route(x2, sinks[:2], [Wg, Wu], [Ag, Au])
        ctx.derived_d = _derived_route(h, sinks[2:], [Wd], [Ad])
        ctx.save_for_backward(x2, None if ctx.derived_gu else T_cat, g, u, h, None if ctx.derived_d else T2,
                              Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd)
        return y.view(*x.shape[:-1], Wd.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, T_cat, g, u, h, T2, Wg, Ag, Bg, Wu, Au, Bu, Wd, Ad, Bd = ctx.saved_tensors
        d = _flat(dy)
        if d.stride(-1) != 1:
            d = d.contiguous()
        dWd, dAd, dBd = ctx.sinks[2]
        if ctx.derived_d:
            W_eff = ops.lora_merge_weight([Wd], [Ad], [Bd], ctx.s)[0]
            dg, du = _down_dx_with_activation_grad(d, None, W_eff, None, g, u)
            dWl = ops.bwd_dw_layer_group([d], h, [dWd])
            if ctx.batch is not None:
                ctx.batch.add(dWl, [Ad], [Bd], [dAd], [dBd], ctx.s)
            else:
                ops.lora_adapter_grads_from_dw(dWl, [Ad], [Bd], [dAd], [dBd], ctx.s)
        else:
            if ctx.batch is not None:
                ctx.batch.nothing_to_add()
            U2 = ops.lora_bwd_prepass(d, Bd, ctx.s)
            dg, du = _down_dx_with_activation_grad(d, U2, Wd, Ad, g, u)
            ops.lora_linear_bwd_dw(d, U2, h, T2, dWd, dAd, dBd)
        gctx = _GroupCtx(2, ctx.derived_gu, ctx.s, ctx.sinks[:2], ctx.batch, ctx.x_shape, ctx.needs_input_grad[0])
        dX = _group_backward(gctx, x2, T_cat, [Wg, Ag, Bg, Wu, Au, Bu], (dg, du))[0]
        return (dX, None, None, None, None) + (None,) * 9


def lora_mlp(x: torch.Tensor, Ws, As, Bs, s: float, sinks=None, anchors: Tuple[torch.Tensor, ...] = (),
             batch: Optional[AdapterGradBatch] = None) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) with Ws = (W_gate, W_up, W_down) etc. One autograd node with
    the activation in the GEMM epilogues (LoRAMLPFunction) where the shapes allow it and the
    weight gradients accumulate in place (``sinks`` complete); else the composition of
    lora_gate_up_swiglu and lora_linear_group, which computes the same bits."""
    x2 = _flat(x)
    Wg, Wu, Wd = Ws
    M = x2.shape[0]
    r = As[0].shape[0]
    fused = (M > 0 and x2.dtype == torch.bfloat16 and sinks is not None
             and all(t is not None for trip in sinks for t in trip)
             and As[1].shape[0] == r and As[2].shape[0] == r and Wg.shape == Wu.shape
             and Wd.shape == (Wg.shape[1], Wg.shape[0])
             and ops.lora_swiglu_supported(M, Wg.shape[0], Wg.shape[1], r)
             and ops.swiglu_bwd_in_dx_supported(M, Wd.shape[0], Wd.shape[1], r))
    if fused:
        return LoRAMLPFunction.apply(x, s, sinks, _Anchor(anchors, x), batch, Wg, As[0], Bs[0], Wu, As[1], Bs[1],
                                     Wd, As[2], Bs[2])
    act = lora_gate_up_swiglu(x, Ws[:2], As[:2], Bs[:2], s, None if sinks is None else sinks[:2], anchors, batch)
    return lora_linear_group(act, [Wd], [As[2]], [Bs[2]], s, None if sinks is None else sinks[2:], anchors, batch)[0]


def lora_gate_up_swiglu(x: torch.Tensor, Ws, As, Bs, s: float, sinks=None,
                        anchors: Tuple[torch.Tensor, ...] = (),
                        batch: Optional[AdapterGradBatch] = None) -> torch.Tensor:
    """silu(gate(x)) * up(x) with Ws = (W_gate, W_up) etc. Takes the one-launch path where the
    shapes allow it (see ops.lora_swiglu_supported), else the grouped forward followed by the
    stand-alone activation kernel; both give the same bits."""
    x2 = _flat(x)
    Wg, Wu = Ws
    if (x2.shape[0] > 0 and x2.dtype == torch.bfloat16 and As[0].shape[0] == As[1].shape[0]
            and Wg.shape == Wu.shape
            and ops.lora_swiglu_supported(x2.shape[0], Wg.shape[0], Wg.shape[1], As[0].shape[0])):
        return LoRAGateUpSwiGLUFunction.apply(x, s, sinks, _Anchor(anchors, x), batch,
                                              Wg, As[0], Bs[0], Wu, As[1], Bs[1])
    gate, up = lora_linear_group(x, Ws, As, Bs, s, sinks, anchors, batch)
    return swiglu(gate, up)


def lora_linear_group(x: torch.Tensor, Ws: Sequence[torch.Tensor], As: Sequence[torch.Tensor],
                      Bs: Sequence[torch.Tensor], s: float, sinks=None,
                      anchors: Tuple[torch.Tensor, ...] = (),
                      batch: Optional[AdapterGradBatch] = None) -> Tuple[torch.Tensor, ...]:
    """Functional form of LoRALinearGroupFunction (q|k|v or gate|up sharing one input)."""
    wab = []
    for W, A, B in zip(Ws, As, Bs):
        wab += [W, A, B]
    return LoRALinearGroupFunction.apply(x, s, sinks, _Anchor(anchors, x), batch, *wab)


def lora_linear(x: torch.Tensor, W: torch.Tensor, A: torch.Tensor, B: torch.Tensor, s: float,
                sinks: Sinks = None, anchors: Tuple[torch.Tensor, ...] = ()) -> torch.Tensor:
    """y = x W^T + s (x A^T) B^T through the fused kernels; differentiable in x, W, A, B."""
    return lora_linear_group(x, [W], [A], [B], s, None if sinks is None else [sinks], anchors)[0]


class _AnchorFn(torch.autograd.Function):
    """Zero-size tensor that requires grad iff one of the anchors does. It lets a Function
    whose weights are detached compute copies still run its backward when x itself does not
    require grad (first layer), so the in-place sinks get filled."""

    @staticmethod
    def forward(ctx, *anchors):
        return anchors[0].new_empty(0)

    @staticmethod
    def backward(ctx, g):
        return (None,) * len(ctx.needs_input_grad)


def _Anchor(anchors: Tuple[torch.Tensor, ...], like: torch.Tensor):
    live = tuple(a for a in anchors if a.requires_grad)
    if not live:
        return None
    return _AnchorFn.apply(*live)


class LoRADeltaFunction(torch.autograd.Function):
    """The adapter alone: s (x A^T) B^T, i.e. LoRAModule.forward
    (torchtitan/models/llama3/model/model.py:189-192) for callers that keep the base
    projection separate (head-sharing modes of the reference)."""

    @staticmethod
    def forward(ctx, x, A, B, s):
        x2 = _flat(x)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        T = ops.lora_prepass(x2, A, s)
        y = ops.linear_fwd(T, B)
        ctx.save_for_backward(x2, T, A, B)
        ctx.s = float(s)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], B.shape[0])

    @staticmethod
    def backward(ctx, dY):
        x2, T, A, B = ctx.saved_tensors
        d = _flat(dY)
        if d.stride(-1) != 1:
            d = d.contiguous()
        U = ops.lora_bwd_prepass(d, B, ctx.s)
        dX = None
        if ctx.needs_input_grad[0]:
            dX = ops.lora_linear_bwd_dx([U], [None], [A], [None]).view(ctx.x_shape)
        dA = torch.zeros(A.shape, device=A.device, dtype=torch.float32) if ctx.needs_input_grad[1] else None
        dB = torch.zeros(B.shape, device=B.device, dtype=torch.float32) if ctx.needs_input_grad[2] else None
        if dA is not None or dB is not None:
            ops.lora_linear_bwd_dw(d, U, x2, T, None, dA, dB)
        return (dX, dA.to(A.dtype) if dA is not None else None,
                dB.to(B.dtype) if dB is not None else None, None)


def lora_delta(x: torch.Tensor, A: torch.Tensor, B: torch.Tensor, s: float) -> torch.Tensor:
    return LoRADeltaFunction.apply(x, A, B, s)


class LinearFunction(torch.autograd.Function):
    """Plain y = x W^T on the same kernels (projection without an adapter)."""

    @staticmethod
    def forward(ctx, x, W, sink):
        x2 = _flat(x)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = ops.linear_fwd(x2, W)
        ctx.save_for_backward(x2, W)
        ctx.sink = sink
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], W.shape[0])

    @staticmethod
    def backward(ctx, dY):
        x2, W = ctx.saved_tensors
        d = _flat(dY)
        if d.stride(-1) != 1:
            d = d.contiguous()
        dX = None
        if ctx.needs_input_grad[0]:
            dX = ops.lora_linear_bwd_dx([d], [None], [W], [None]).view(ctx.x_shape)
        gW = None
        if ctx.sink is not None:
            ops.lora_linear_bwd_dw(d, None, x2, None, ctx.sink, None, None)
        elif ctx.needs_input_grad[1]:
            dW = torch.zeros(W.shape, device=W.device, dtype=torch.float32)
            ops.lora_linear_bwd_dw(d, None, x2, None, dW, None, None)
            gW = dW.to(W.dtype)
        return dX, gW, None


def linear(x: torch.Tensor, W: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    return LinearFunction.apply(x, W, sink)


class SwiGLUFunction(torch.autograd.Function):
    """silu(gate) * up in one pass each way (torchtitan/experiments/qwen3/model/model.py:251)."""

    @staticmethod
    def forward(ctx, gate, up):
        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        if gate.numel() == 0:
            return torch.empty_like(gate)
        return ops.swiglu_fwd(gate, up)

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        if gate.numel() == 0:
            return torch.empty_like(gate), torch.empty_like(up)
        return ops.swiglu_bwd(dout, gate, up)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return SwiGLUFunction.apply(gate, up)


class RMSNormFunction(torch.autograd.Function):
    """RMSNorm over the last dimension with an fp32 scale, optionally followed by the rotary
    embedding of the normalised row (q/k head norm + RoPE of
    torchtitan/experiments/qwen3/model/model.py:195-203 in one pass).

    forward(ctx, x, w, eps, rope, sink): rope = None or (cos [seq, D] fp32, sin, heads, seq);
    sink = fp32 [D] buffer to accumulate dw into in place (then no gradient is returned
    for w), or None."""

    @staticmethod
    def forward(ctx, x, w, eps, rope, sink):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if x2.shape[0] == 0:
            y, rstd = torch.empty_like(x2), x2.new_empty(0, dtype=torch.float32)
        else:
            y, rstd = ops.rmsnorm_fwd(x2, w, eps, rope)
        ctx.save_for_backward(x2, w, rstd)
        ctx.rope = rope
        ctx.sink = sink
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        D = x2.shape[-1]
        if x2.shape[0] == 0:
            dw0 = torch.zeros_like(w) if ctx.sink is None and ctx.needs_input_grad[1] else None
            return torch.empty_like(x2).view(ctx.shape), dw0, None, None, None
        dy2 = dy.reshape(-1, D)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        if ctx.sink is not None:
            dx = ops.rmsnorm_bwd(dy2, x2, w, rstd, ctx.sink, ctx.rope)
            return dx.view(ctx.shape), None, None, None, None
        dw = torch.zeros(D, device=x2.device, dtype=torch.float32) if ctx.needs_input_grad[1] else None
        dx = ops.rmsnorm_bwd(dy2, x2, w, rstd, dw, ctx.rope)
        return dx.view(ctx.shape), (dw.to(w.dtype) if dw is not None else None), None, None, None


class AddRMSNormFunction(torch.autograd.Function):
    """The residual add that precedes a norm, and the norm, in one pass:
    forward(ctx, x, res, w, eps, sink) -> (h, y) with h = x + res and y = RMSNorm(h) * w
    (``h = h + attention(...)`` followed by ``ffn_norm(h)``,
    torchtitan/experiments/qwen3/model/model.py:310-313). The backward adds the gradient that
    reaches h through the residual stream to the norm's own dx in the same kernel; it is the
    gradient of both x and res."""

    @staticmethod
    def forward(ctx, x, res, w, eps, sink):
        D = x.shape[-1]
        h2, y2, rstd = ops.add_rmsnorm_fwd(x.reshape(-1, D), res.reshape(-1, D), w, eps)
        ctx.save_for_backward(h2, w, rstd)
        ctx.sink = sink
        ctx.shape = x.shape
        return h2.view(x.shape), y2.view(x.shape)

    @staticmethod
    def backward(ctx, dh, dy):
        h2, w, rstd = ctx.saved_tensors
        D = h2.shape[-1]
        dw = ctx.sink
        if dw is None and ctx.needs_input_grad[2]:
            dw = torch.zeros(D, device=h2.device, dtype=torch.float32)
        if dy is None:
            dx = dh
        elif dh is None:
            dx = ops.rmsnorm_bwd(dy.reshape(-1, D), h2, w, rstd, dw).view(ctx.shape)
        else:
            dx = ops.add_rmsnorm_bwd(dy.reshape(-1, D), h2, dh.reshape(-1, D), w, rstd, dw).view(ctx.shape)
        gw = dw.to(w.dtype) if (ctx.sink is None and dw is not None) else None
        return dx, dx, gw, None, None


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float, sink=None):
    """(x + res, RMSNorm(x + res) * w); see AddRMSNormFunction."""
    return AddRMSNormFunction.apply(x, res, w, eps, sink)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, rope=None, sink=None) -> torch.Tensor:
    return RMSNormFunction.apply(x, w, eps, rope, sink)
