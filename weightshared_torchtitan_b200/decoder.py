"""Weight-shared Qwen3-shape decoder: the caller of the fused projections in a training step.

Host-side PyTorch around the kernels. The block structure (pre-norm residual block, q/k
RMSNorm, RoPE, causal SDPA, SwiGLU, final norm, untied output head, mean-token
cross-entropy) follows torchtitan/experiments/qwen3/model/model.py:105-321,436-447 and
torchtitan/components/loss.py:18-22. What differs from the reference model is exactly the
hot path: every projection is y = x W^T + s (x A^T) B^T with W taken from shared block
(layer mod n_unique) and a per-layer adapter, q|k|v and gate|up are issued as groups that
read x once, and the token embedding is factorized.

The attention core (causal SDPA) stays a PyTorch library call; RMSNorm (+ residual add,
+ rotary embedding), SwiGLU and the softmax cross-entropy run as the library's row kernels
where they cover the width, else as the PyTorch calls.

Parameters are fp32 masters; compute is bf16 (the reference's autocast policy,
torchtitan/distributed/utils.py:219-239) with fp32 accumulation; parameter gradients are
fp32 and accumulate in place into `param.grad` (views of one flat arena when the model is
wrapped by dp.GradArena).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import functional as WF
from . import ops
from .modules import CopyCache, FactorizedEmbedding, LoRAModule, factorized_embedding


@dataclass
class DecoderConfig:
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
    loss_chunk: int = 8192      # tokens per slice of the output head + cross-entropy


# Shapes of torchtitan/experiments/qwen3/__init__.py:31-104 with the sharing/rank settings of
# the baseline configurations 1-4.
CONFIGS: Dict[str, DecoderConfig] = {
    "qwen3-0.6b-ws": DecoderConfig(1024, 3072, 28, 4, 16, 8, 128, 16, 151936, 256, max_seq_len=4096),
    "qwen3-1.7b-ws": DecoderConfig(2048, 6144, 28, 7, 16, 8, 128, 32, 151936, 512, max_seq_len=4096),
    "qwen3-4b-ws": DecoderConfig(2560, 9728, 36, 6, 32, 8, 128, 64, 151936, 512, max_seq_len=8192),
    "qwen3-8b-ws": DecoderConfig(4096, 12288, 36, 4, 32, 8, 128, 64, 151936, 1024, max_seq_len=8192),
}

PROJ_NAMES = ("wq", "wk", "wv", "wo", "w1", "w3", "w2")


def proj_shapes(c: DecoderConfig) -> Dict[str, Tuple[int, int]]:
    q, kv = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
    return {"wq": (q, c.dim), "wk": (kv, c.dim), "wv": (kv, c.dim), "wo": (c.dim, q),
            "w1": (c.hidden_dim, c.dim), "w3": (c.hidden_dim, c.dim), "w2": (c.dim, c.hidden_dim)}


class SharedBlock(nn.Module):
    """The seven base projections of one unique block; layers reference these objects."""

    def __init__(self, c: DecoderConfig):
        super().__init__()
        for name, (o, i) in proj_shapes(c).items():
            setattr(self, name, nn.Linear(i, o, bias=False))


class DecoderLayer(nn.Module):
    """Per-layer state: adapters (LoRAModule naming of the reference: <proj>_offset.w_a /
    .w_b), norms, and references to the shared block's base projections (<proj>_base)."""

    def __init__(self, c: DecoderConfig, block: SharedBlock):
        super().__init__()
        for name, (o, i) in proj_shapes(c).items():
            setattr(self, f"{name}_base", getattr(block, name))
            setattr(self, f"{name}_offset", LoRAModule(i, o, rank=c.rank))
        self.attention_norm = nn.RMSNorm(c.dim, eps=c.norm_eps)
        self.ffn_norm = nn.RMSNorm(c.dim, eps=c.norm_eps)
        self.q_norm = nn.RMSNorm(c.head_dim, eps=c.norm_eps)
        self.k_norm = nn.RMSNorm(c.head_dim, eps=c.norm_eps)


def rope_tables(head_dim: int, seq_len: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def _rms(norm: nn.RMSNorm, x: torch.Tensor, rope=None) -> torch.Tensor:
    """RMSNorm (optionally + rotary embedding) through the fused row kernel; widths the
    kernel does not cover use the PyTorch call with the scale cast to the activation dtype.
    rope = (cos, sin, heads, seq) with fp32 [seq, head_dim] tables."""
    D = x.shape[-1]
    w = norm.weight
    if w.dtype == torch.float32 and ops.rmsnorm_supported(D, x.dtype, rope is not None):
        sink = None
        if torch.is_grad_enabled() and w.requires_grad and x.requires_grad:
            if w.grad is None:
                w.grad = torch.zeros_like(w)
            sink = w.grad
        return WF.rmsnorm(x, w if sink is None else w.detach(), norm.eps, rope, sink)
    y = F.rms_norm(x, norm.normalized_shape, w.to(x.dtype), norm.eps)
    if rope is not None:
        cos, sin, heads, seq = rope
        c = cos[:seq].to(x.dtype).view(1, seq, 1, D)
        s_ = sin[:seq].to(x.dtype).view(1, seq, 1, D)
        y = _rope(y, c, s_)
    return y


def _add_rms(norm: nn.RMSNorm, h: torch.Tensor, delta: torch.Tensor):
    """(h + delta, norm(h + delta)): the residual add folded into the norm kernel where the
    kernel covers the width, else the two PyTorch-level steps."""
    D = h.shape[-1]
    w = norm.weight
    if (w.dtype == torch.float32 and h.is_cuda and h.dtype == delta.dtype and h.shape == delta.shape
            and ops.rmsnorm_supported(D, h.dtype)):
        sink = None
        if torch.is_grad_enabled() and w.requires_grad and (h.requires_grad or delta.requires_grad):
            if w.grad is None:
                w.grad = torch.zeros_like(w)
            sink = w.grad
        return WF.add_rmsnorm(h, delta, w if sink is None else w.detach(), norm.eps, sink)
    h = h + delta
    return h, _rms(norm, h)


def _rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    d = t.shape[-1]
    rot = torch.cat((-t[..., d // 2:], t[..., : d // 2]), dim=-1)
    return t * cos + rot * sin


class _HeadLossFunction(torch.autograd.Function):
    """Output head + mean cross-entropy, sliced over tokens so that the fp32 logits of only
    `chunk` tokens exist at a time. Forward already computes d(loss)/d(h) and the head
    weight gradient (accumulated into `sink`); backward scales dH by the incoming gradient.
    GEMMs and the softmax-cross-entropy row kernel are the library's."""

    @staticmethod
    def forward(ctx, h, Wc, labels, sink, chunk, anchor):
        M = h.shape[0]
        V = Wc.shape[0]
        dH = torch.empty_like(h)
        total = torch.zeros((), device=h.device, dtype=torch.float32)
        # reduction='mean' of F.cross_entropy divides by the number of COUNTED rows: labels
        # outside [0, V) (ignore_index = -100: padding, packed documents) contribute neither
        # loss nor gradient nor to the divisor. The count stays on the device.
        inv_count = ((labels >= 0) & (labels < V)).sum().clamp_min(1).to(torch.float32).reciprocal().reshape(1)
        for m0 in range(0, M, chunk):
            hs = h[m0:m0 + chunk]
            # logits in the compute dtype (bf16 under the reference's autocast, cast up inside
            # the loss kernel), overwritten in place by their gradient
            logits = ops.linear_fwd(hs, Wc)
            total += ops.ce_fwd_bwd(logits, labels[m0:m0 + chunk], 1.0, inv_count).sum()
            dH[m0:m0 + chunk] = ops.lora_linear_bwd_dx([logits], [None], [Wc], [None])
            if sink is not None:
                ops.lora_linear_bwd_dw(logits, None, hs, None, sink, None, None)
            del logits
        ctx.save_for_backward(dH)
        return total * inv_count[0]

    @staticmethod
    def backward(ctx, g):
        (dH,) = ctx.saved_tensors
        return dH * g.to(dH.dtype), None, None, None, None, None


class WeightSharedDecoder(nn.Module):
    def __init__(self, c: DecoderConfig):
        super().__init__()
        self.config = c
        self.tok_embeddings = FactorizedEmbedding(c.vocab_size, c.embed_rank, c.dim)
        self.blocks = nn.ModuleList([SharedBlock(c) for _ in range(c.n_unique)])
        self.layers = nn.ModuleList([DecoderLayer(c, self.blocks[l % c.n_unique]) for l in range(c.n_layers)])
        self.norm = nn.RMSNorm(c.dim, eps=c.norm_eps)
        self.output = nn.Linear(c.dim, c.vocab_size, bias=False)
        self.compute_dtype = torch.bfloat16
        self._cache = CopyCache()
        self._rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        # Called during backward with a ready-rank k as soon as every parameter gradient of
        # rank <= k is final (see grad_ready_rank); lets the owner of the gradient arena start
        # exchanging finished ranges while backward still runs. None = nobody listens.
        self.grad_ready_hook = None

    # ------------------------------------------------------------------ initialisation
    @torch.no_grad()
    def init_weights(self, seed: int = 1235) -> None:
        """Value distributions of the baseline configurations (W ~ N(0, 0.02^2),
        A ~ U(+-1/sqrt(K)), B ~ N(0, 0.02^2) non-zero, E_small ~ N(0,1), P ~ N(0, 0.02^2),
        head ~ N(0, 1/dim)); device generator, same seed on every rank gives identical
        replicas."""
        dev = self.output.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        for blk in self.blocks:
            for name in PROJ_NAMES:
                getattr(blk, name).weight.normal_(0.0, 0.02, generator=g)
        for lyr in self.layers:
            for name in PROJ_NAMES:
                off = getattr(lyr, f"{name}_offset")
                bound = 1.0 / math.sqrt(off.in_dim)
                off.w_a.weight.uniform_(-bound, bound, generator=g)
                off.w_b.weight.normal_(0.0, 0.02, generator=g)
            for n in (lyr.attention_norm, lyr.ffn_norm, lyr.q_norm, lyr.k_norm):
                n.weight.fill_(1.0)
        self.tok_embeddings.embed.weight.normal_(0.0, 1.0, generator=g)
        self.tok_embeddings.proj.weight.normal_(0.0, 0.02, generator=g)
        self.norm.weight.fill_(1.0)
        self.output.weight.normal_(0.0, self.config.dim ** -0.5, generator=g)
        self.post_optimizer_hook()

    @torch.no_grad()
    def load_named_params(self, p: Dict[str, torch.Tensor]) -> None:
        """Copy a parameter dictionary in the flat naming used by the parity tests
        (blocks.{u}.{proj}.weight, layers.{l}.{proj}.w_a / .w_b, norms, embed.*, output)."""
        for u, blk in enumerate(self.blocks):
            for name in PROJ_NAMES:
                getattr(blk, name).weight.copy_(p[f"blocks.{u}.{name}.weight"])
        for l, lyr in enumerate(self.layers):
            for name in PROJ_NAMES:
                off = getattr(lyr, f"{name}_offset")
                off.w_a.weight.copy_(p[f"layers.{l}.{name}.w_a"])
                off.w_b.weight.copy_(p[f"layers.{l}.{name}.w_b"])
            for n in ("attention_norm", "ffn_norm", "q_norm", "k_norm"):
                getattr(lyr, n).weight.copy_(p[f"layers.{l}.{n}"])
        self.tok_embeddings.embed.weight.copy_(p["embed.E_small"])
        self.tok_embeddings.proj.weight.copy_(p["embed.P"])
        self.norm.weight.copy_(p["norm"])
        self.output.weight.copy_(p["output"])
        self.post_optimizer_hook()

    # ------------------------------------------------------------------------ helpers
    def grad_ready_rank(self, name: str) -> int:
        """Order in which parameter gradients become final during one step (smaller = earlier).
        The output head's gradient is complete when the loss has been computed (rank 0, before
        backward starts); backward then walks the layers from last to first, so layer l is rank
        n_layers - l, together with the final norm (rank 1) and with the shared block whose
        FIRST user is layer l (every later user has already contributed); the embedding comes
        last."""
        L = self.config.n_layers
        head = name.split(".", 2)
        if head[0] == "output":
            return 0
        if head[0] == "norm":
            return 1
        if head[0] in ("layers", "blocks"):
            return L - int(head[1])
        return L + 1

    def _notify_on_grad(self, t: torch.Tensor, rank: int) -> None:
        """When the gradient of `t` has been computed, everything of ready-rank <= rank is final."""
        hook = self.grad_ready_hook
        if hook is not None and t.requires_grad:
            def fire(grad, _hook=hook, _rank=rank):
                _hook(_rank)
                return None
            t.register_hook(fire)

    def post_optimizer_hook(self) -> None:
        """The master weights changed: the compute-dtype copies must follow before the next
        forward (the reference's post_optimizer_hook slot, torchtitan/train.py:288-295). Copies
        the cache made itself are dropped and re-cast on next use; when the cache is bound to a
        flat arena (TrainStep) the arena's flat copy is re-cast here, in one pass. Call this
        after anything that writes the parameters behind the optimizer's back: a state-dict
        load, dp.broadcast_parameters, a re-initialisation."""
        self._cache.invalidate()

    @staticmethod
    def _sink(p: torch.Tensor) -> torch.Tensor:
        if p.grad is None:
            p.grad = torch.zeros(p.shape, device=p.device, dtype=torch.float32)
        return p.grad

    def _group(self, lyr: DecoderLayer, names, x, batch=None, mlp: bool = False):
        dt = self.compute_dtype
        Ws, As, Bs, sinks, anchors = [], [], [], [], []
        train = torch.is_grad_enabled()
        for n in names:
            W = getattr(lyr, f"{n}_base").weight
            off = getattr(lyr, f"{n}_offset")
            A, B = off.w_a.weight, off.w_b.weight
            Ws.append(self._cache.get(dt, W))
            As.append(self._cache.get(dt, A))
            Bs.append(self._cache.get(dt, B))
            if train:
                sinks.append((self._sink(W), self._sink(A), self._sink(B)))
                anchors += [W, A, B]
        s = getattr(lyr, f"{names[0]}_offset").scale
        if mlp:   # names = (gate, up, down): the activation rides in the GEMM epilogues
            return WF.lora_mlp(x, Ws, As, Bs, s, sinks if train else None, tuple(anchors), batch)
        return WF.lora_linear_group(x, Ws, As, Bs, s, sinks if train else None, tuple(anchors), batch)

    # ------------------------------------------------------------------------ forward
    def hidden(self, tokens: torch.Tensor) -> torch.Tensor:
        """Final-norm hidden states [b, s, dim] in the compute dtype."""
        c = self.config
        dt = self.compute_dtype
        b, s = tokens.shape
        emb = self.tok_embeddings
        E, P = emb.embed.weight, emb.proj.weight
        if torch.is_grad_enabled():
            h = factorized_embedding(tokens, self._cache.get(dt, E), self._cache.get(dt, P),
                                     sinks=(self._sink(E), self._sink(P)), anchors=(E, P))
        else:
            h = factorized_embedding(tokens, self._cache.get(dt, E), self._cache.get(dt, P))
        if self._rope is None or self._rope[0].shape[0] != s or self._rope[0].device != h.device:
            cos, sin = rope_tables(c.head_dim, s, c.rope_theta, h.device)
            self._rope = (cos.contiguous(), sin.contiguous())       # fp32 [s, head_dim]
        cos, sin = self._rope
        L = c.n_layers
        # layer 0 (and the shared block it is the first user of) is final once the gradient of
        # the embedding output exists
        self._notify_on_grad(h, L)
        pending = None   # output of the previous layer's down projection, not yet added to h
        for li, lyr in enumerate(self.layers):
            if pending is not None:
                # the gradient of the previous layer's output exists only after this layer's
                # whole backward (its first norm included): layers >= li are final then
                self._notify_on_grad(pending, L - li)
            # the layer's four projection groups hand their adapter-gradient work to one batch
            ab = WF.AdapterGradBatch(4) if torch.is_grad_enabled() else None
            # every residual add is folded into the norm that reads the sum
            if pending is None:
                xn = _rms(lyr.attention_norm, h)
            else:
                h, xn = _add_rms(lyr.attention_norm, h, pending)
            q, k, v = self._group(lyr, ("wq", "wk", "wv"), xn, ab)
            q = _rms(lyr.q_norm, q.view(b, s, c.n_heads, c.head_dim), (cos, sin, c.n_heads, s))
            k = _rms(lyr.k_norm, k.view(b, s, c.n_kv_heads, c.head_dim), (cos, sin, c.n_kv_heads, s))
            v = v.view(b, s, c.n_kv_heads, c.head_dim)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=c.n_heads != c.n_kv_heads)
            o = o.transpose(1, 2).reshape(b, s, c.n_heads * c.head_dim)
            h, xn = _add_rms(lyr.ffn_norm, h, self._group(lyr, ("wo",), o, ab)[0])
            pending = self._group(lyr, ("w1", "w3", "w2"), xn, ab, mlp=True)
        if pending is None:
            return _rms(self.norm, h)
        return _add_rms(self.norm, h, pending)[1]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """fp32 logits [b, s, V] (evaluation / parity use; training uses loss())."""
        h = self.hidden(tokens)
        Wc = self._cache.get(self.compute_dtype, self.output.weight)
        logits = ops.linear_fwd(h.reshape(-1, h.shape[-1]), Wc, out_f32=True)
        return logits.view(*tokens.shape, -1)

    def loss(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """Mean token cross-entropy; differentiable (head gradients accumulate in place)."""
        h = self.hidden(tokens)
        h2 = h.reshape(-1, h.shape[-1])
        W = self.output.weight
        train = torch.is_grad_enabled()
        return _HeadLossFunction.apply(h2, self._cache.get(self.compute_dtype, W), labels.reshape(-1),
                                       self._sink(W) if train else None, self.config.loss_chunk,
                                       WF._Anchor((W,), h2) if train else None)


def flops_per_token(c: DecoderConfig, seq_len: int) -> Dict[str, float]:
    """Executed algorithmic FLOPs per token, fwd+bwd: projections 6 N K + 6 r (K + N) each
    (every layer counted, shared or not), attention 12 l h q t as in the reference formula
    (torchtitan/models/llama3/model/args.py:91), output head 6 d V, embedding 6 r_e d."""
    lin = sum(6 * o * i + 6 * c.rank * (o + i) for (o, i) in proj_shapes(c).values()) * c.n_layers
    attn = 12 * c.n_layers * c.n_heads * c.head_dim * seq_len
    head = 6 * c.dim * c.vocab_size
    emb = 6 * c.embed_rank * c.dim
    return {"linear": float(lin), "attention": float(attn), "head": float(head), "embed": float(emb),
            "total": float(lin + attn + head + emb)}
