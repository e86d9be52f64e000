"""CPU oracle for the shared-W + LoRA linear hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py
may import this module, and only as the checker (or, in bench.py, as the timed CPU
baseline). The product package never imports it: its path has no CPU implementation.

This is a restatement, in plain eager PyTorch, of the arithmetic the reference
(muchanem/weightshared_torchtitan) performs for this path; each function names the
reference lines it follows (paths relative to the reference project root). The
arithmetic primitives themselves (matmul, RMSNorm, SDPA) live in the third-party
dependency ``torch`` (this build pins against torch 2.11.0, the version the golden
fixtures under tests/golden/ were generated with).

Parity pins: the reference has NO test, golden vector or fixture for LoRAModule,
broadcast_add or any weight-shared model (none of its tests import them). The pins are
therefore outputs of the reference's own modules, imported and run in the build
container by tests/golden/make_golden.py and committed as tests/golden/*.npz;
tests/test_oracle_golden.py checks this restatement against them.

Items that do not exist in the reference and are defined here by composition of its
primitives (stated so in each docstring): cross-layer sharing of W, LoRA on
o/gate/up/down, the factorized embedding.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- the op
def broadcast_add(base: torch.Tensor, delta: torch.Tensor, *, dim: int = -1, g: int = 1) -> torch.Tensor:
    """broadcast(base) + delta over head groups.

    Follows torchtitan/models/llama3/model/model.py:111-145: `base` carries g*D features,
    `delta` H*D; every group of H/g heads reuses one template. With equal widths this is a
    plain add (the case the fused kernel covers).
    """
    if dim < 0:
        dim += base.dim()
    big, small = delta.shape[dim], base.shape[dim]
    if big % small != 0:
        raise AssertionError("delta and base feature dims incompatible")
    per_group = big // small
    d_head = small // g
    shape = list(base.shape)
    shape[dim:dim + 1] = [g, 1, d_head]
    expanded = base.reshape(shape)
    target = list(expanded.shape)
    target[dim + 1] = per_group
    expanded = expanded.expand(target).reshape(delta.shape)
    return expanded + delta


def lora_delta(x: torch.Tensor, A: torch.Tensor, B: torch.Tensor, rank: Optional[int] = None) -> torch.Tensor:
    """s * (x A^T) B^T with alpha = 2*rank, i.e. s = alpha/rank = 2.

    Follows LoRAModule.__init__/forward, torchtitan/models/llama3/model/model.py:148-192
    (alpha at l.162, forward at l.189-192: w_b(w_a(x)) * (alpha / rank)).
    """
    rank = A.shape[0] if rank is None else rank
    alpha = rank * 2
    return F.linear(F.linear(x, A), B) * (alpha / rank)


def lora_linear(x: torch.Tensor, W: torch.Tensor, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """base(x) + LoRA(x): torchtitan/models/llama3/model/model.py:392-398 with N_base == N."""
    return broadcast_add(F.linear(x, W), lora_delta(x, A, B))


def lora_linear_fwd_bwd(x, W, A, B, dY):
    """Forward and all gradients by autograd (base F.linear plus LoRAModule.forward, added):
    returns y, dX, dW, dA, dB."""
    x = x.detach().clone().requires_grad_(True)
    W = W.detach().clone().requires_grad_(True)
    A = A.detach().clone().requires_grad_(True)
    B = B.detach().clone().requires_grad_(True)
    y = lora_linear(x, W, A, B)
    y.backward(dY)
    return y.detach(), x.grad, W.grad, A.grad, B.grad


def shared_w_layers_fwd_bwd(xs: Sequence[torch.Tensor], W: torch.Tensor, As: Sequence[torch.Tensor],
                            Bs: Sequence[torch.Tensor], dYs: Sequence[torch.Tensor]):
    """L uses of ONE base weight W, each with its own adapter (config 0 of the baseline).

    Cross-layer sharing is not in the reference; it is defined here the way the reference
    shares parameters elsewhere (the same nn.Linear object referenced by several owners,
    torchtitan/models/llama3/model/model.py:154-182), so autograd sums the L weight
    gradients into one W.grad. Returns ys, dXs, dW (summed), dAs, dBs.
    """
    Wp = W.detach().clone().requires_grad_(True)
    ys, dXs, dAs, dBs = [], [], [], []
    leaves = []
    for x, A, B in zip(xs, As, Bs):
        xl = x.detach().clone().requires_grad_(True)
        Al = A.detach().clone().requires_grad_(True)
        Bl = B.detach().clone().requires_grad_(True)
        leaves.append((xl, Al, Bl))
        ys.append(lora_linear(xl, Wp, Al, Bl))
    total = sum((y * dY).sum() for y, dY in zip(ys, dYs))
    total.backward()
    for xl, Al, Bl in leaves:
        dXs.append(xl.grad)
        dAs.append(Al.grad)
        dBs.append(Bl.grad)
    return [y.detach() for y in ys], dXs, Wp.grad, dAs, dBs


def factorized_embedding(tokens: torch.Tensor, E_small: torch.Tensor, P: torch.Tensor) -> torch.Tensor:
    """E_small[tokens] @ P^T with P stored as an nn.Linear(r_e, d) weight [d, r_e].

    Not in the reference (torchtitan/experiments/qwen3/model/model.py:350,441 is a plain
    nn.Embedding(V, dim)); defined as nn.Embedding(V, r_e) followed by
    nn.Linear(r_e, d, bias=False).
    """
    return F.linear(F.embedding(tokens, E_small), P)


# ------------------------------------------------------------ seeded input generators
def config0_inputs(seed: int = 1234, M: int = 2048, K: int = 1024, N: int = 1024, r: int = 16,
                   L: int = 4, dtype=torch.float32) -> Dict[str, object]:
    """Inputs of baseline configuration 0: x ~ N(0,1), W ~ N(0, 0.02^2), A ~ U(+-1/sqrt(K)),
    B ~ N(0, 0.02^2) (non-zero), dY ~ N(0,1); L layers share W. CPU generator, so the same
    seed gives the same tensors on every machine."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    xs, As, Bs, dYs = [], [], [], []
    bound = 1.0 / math.sqrt(K)
    for _ in range(L):
        xs.append(torch.randn(M, K, generator=g).to(dtype))
        As.append(((torch.rand(r, K, generator=g) * 2 - 1) * bound).to(dtype))
        Bs.append((torch.randn(N, r, generator=g) * 0.02).to(dtype))
        dYs.append(torch.randn(M, N, generator=g).to(dtype))
    return {"W": W, "xs": xs, "As": As, "Bs": Bs, "dYs": dYs, "s": 2.0}


def projection_inputs(seed: int, M: int, N: int, K: int, r: int, dtype=torch.float32):
    """One projection with the value distributions of the baseline configurations."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    A = ((torch.rand(r, K, generator=g) * 2 - 1) / math.sqrt(K)).to(dtype)
    B = (torch.randn(N, r, generator=g) * 0.02).to(dtype)
    dY = torch.randn(M, N, generator=g).to(dtype)
    return x, W, A, B, dY


# ------------------------------------------------------- weight-shared Qwen3 decoder
@dataclass
class DecoderArgs:
    """Shapes of torchtitan/experiments/qwen3/__init__.py:31-104 plus the sharing knobs."""
    dim: int = 1024
    hidden_dim: int = 3072
    n_layers: int = 28
    n_unique: int = 4
    n_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    rank: int = 16
    vocab_size: int = 151936
    embed_rank: int = 256
    norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    max_seq_len: int = 4096


PROJ_NAMES = ("wq", "wk", "wv", "wo", "w1", "w3", "w2")   # q, k, v, o, gate, up, down


def proj_shapes(a: DecoderArgs) -> Dict[str, Tuple[int, int]]:
    """(out, in) of each projection: torchtitan/experiments/qwen3/model/model.py:148-155,246-248."""
    q = a.n_heads * a.head_dim
    kv = a.n_kv_heads * a.head_dim
    return {"wq": (q, a.dim), "wk": (kv, a.dim), "wv": (kv, a.dim), "wo": (a.dim, q),
            "w1": (a.hidden_dim, a.dim), "w3": (a.hidden_dim, a.dim), "w2": (a.dim, a.hidden_dim)}


def rope_cache(head_dim: int, seq_len: int, theta: float, device="cpu") -> torch.Tensor:
    """[seq, 2*head_dim] = cos | sin of position * inverse frequency, halves repeated.
    Follows precompute_rope_cache, torchtitan/experiments/qwen3/model/model.py:20-37."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=inv.dtype), inv).float()
    ang = torch.cat([ang, ang], dim=-1)
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


def apply_rope(q: torch.Tensor, k: torch.Tensor, cache: torch.Tensor):
    """x*cos + rotate_half(x)*sin on [b, s, h, d]; torchtitan/experiments/qwen3/model/model.py:40-90."""
    d = q.shape[-1]
    c = cache[: q.shape[1]].view(1, q.shape[1], 1, 2 * d)
    cos, sin = c[..., :d].to(q.dtype), c[..., d:].to(q.dtype)

    def rot(t):
        return torch.cat((-t[..., d // 2:], t[..., : d // 2]), dim=-1)

    return (q * cos + rot(q) * sin).type_as(q), (k * cos + rot(k) * sin).type_as(k)


def init_decoder_params(a: DecoderArgs, seed: int = 1235, device="cpu") -> Dict[str, torch.Tensor]:
    """fp32 master parameters with the baseline's value distributions; generated on the CPU
    generator so every rank and every implementation gets identical values.

    Names: blocks.{u}.{proj}.weight (shared base, u < n_unique), layers.{l}.{proj}.w_a /
    .w_b (per-layer adapter, LoRAModule naming), layers.{l}.{attention_norm,ffn_norm,
    q_norm,k_norm}, embed.E_small, embed.P, norm, output.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    p: Dict[str, torch.Tensor] = {}
    shapes = proj_shapes(a)
    for u in range(a.n_unique):
        for name, (o, i) in shapes.items():
            p[f"blocks.{u}.{name}.weight"] = torch.randn(o, i, generator=g) * 0.02
    for l in range(a.n_layers):
        for name, (o, i) in shapes.items():
            p[f"layers.{l}.{name}.w_a"] = (torch.rand(a.rank, i, generator=g) * 2 - 1) / math.sqrt(i)
            p[f"layers.{l}.{name}.w_b"] = torch.randn(o, a.rank, generator=g) * 0.02
        p[f"layers.{l}.attention_norm"] = torch.ones(a.dim)
        p[f"layers.{l}.ffn_norm"] = torch.ones(a.dim)
        p[f"layers.{l}.q_norm"] = torch.ones(a.head_dim)
        p[f"layers.{l}.k_norm"] = torch.ones(a.head_dim)
    p["embed.E_small"] = torch.randn(a.vocab_size, a.embed_rank, generator=g)
    p["embed.P"] = torch.randn(a.dim, a.embed_rank, generator=g) * 0.02
    p["norm"] = torch.ones(a.dim)
    p["output"] = torch.randn(a.vocab_size, a.dim, generator=g) * (a.dim ** -0.5)
    return {k: v.to(device) for k, v in p.items()}


def decoder_forward(a: DecoderArgs, p: Dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    """Logits [b, s, V] of the weight-shared Qwen3-shape decoder, eager PyTorch.

    The block follows torchtitan/experiments/qwen3/model/model.py:105-218 (attention with
    q/k RMSNorm, RoPE, causal SDPA), 221-256 (SwiGLU), 288-321 (pre-norm residual block),
    436-447 (embed -> layers -> norm -> output); every nn.Linear of the block is replaced by
    lora_linear with the base weight of block (layer mod n_unique). Run it under
    torch.autocast(bfloat16) to get the reference's mixed precision
    (torchtitan/distributed/utils.py:219-239).
    """
    b, s = tokens.shape
    h = factorized_embedding(tokens, p["embed.E_small"], p["embed.P"])
    cache = rope_cache(a.head_dim, s, a.rope_theta, device=h.device)

    def proj(l: int, name: str, x: torch.Tensor) -> torch.Tensor:
        u = l % a.n_unique
        return lora_linear(x, p[f"blocks.{u}.{name}.weight"], p[f"layers.{l}.{name}.w_a"],
                           p[f"layers.{l}.{name}.w_b"])

    for l in range(a.n_layers):
        xn = F.rms_norm(h, (a.dim,), p[f"layers.{l}.attention_norm"], a.norm_eps)
        q = proj(l, "wq", xn).view(b, s, -1, a.head_dim)
        k = proj(l, "wk", xn).view(b, s, -1, a.head_dim)
        v = proj(l, "wv", xn).view(b, s, -1, a.head_dim)
        q = F.rms_norm(q, (a.head_dim,), p[f"layers.{l}.q_norm"], a.norm_eps)
        k = F.rms_norm(k, (a.head_dim,), p[f"layers.{l}.k_norm"], a.norm_eps)
        q, k = apply_rope(q, k, cache)
        rep = a.n_heads // a.n_kv_heads
        k = k.unsqueeze(3).expand(b, s, a.n_kv_heads, rep, a.head_dim).reshape(b, s, a.n_heads, a.head_dim)
        v = v.unsqueeze(3).expand(b, s, a.n_kv_heads, rep, a.head_dim).reshape(b, s, a.n_heads, a.head_dim)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True)
        o = o.transpose(1, 2).contiguous().view(b, s, -1)
        h = h + proj(l, "wo", o)
        xn = F.rms_norm(h, (a.dim,), p[f"layers.{l}.ffn_norm"], a.norm_eps)
        h = h + proj(l, "w2", F.silu(proj(l, "w1", xn)) * proj(l, "w3", xn))
    h = F.rms_norm(h, (a.dim,), p["norm"], a.norm_eps)
    return F.linear(h, p["output"])


def decoder_loss(a: DecoderArgs, p: Dict[str, torch.Tensor], tokens: torch.Tensor,
                 labels: torch.Tensor) -> torch.Tensor:
    """Mean token cross-entropy on fp32 logits: torchtitan/components/loss.py:18-22."""
    logits = decoder_forward(a, p, tokens)
    return F.cross_entropy(logits.flatten(0, 1).float(), labels.flatten(0, 1))


def max_rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Per-tensor max|a-b| / max|b| (the parity metric of the baseline)."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-300))
