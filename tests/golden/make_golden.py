"""Generate the golden fixtures in this directory from the REFERENCE's own modules.

Run in the build container only (it imports the reference from its checkout, which does
not exist on the GPU machines):

    python tests/golden/make_golden.py [/path/to/reference/checkout]

It imports LoRAModule and broadcast_add (torchtitan/models/llama3/model/model.py:111-192)
and the Qwen3 decoder (torchtitan/experiments/qwen3/model/model.py), runs them on CPU in
fp32 with seeded inputs and writes small .npz files:

  lora_small.npz    one projection, full inputs and outputs (y, dX, dW, dA, dB)
  lora_cfg0.npz     baseline configuration 0 (M=2048, K=N=1024, r=16, 4 layers sharing W):
                    strided samples and float64 checksums of every output; inputs are
                    regenerated from the seed by oracle.lora_oracle.config0_inputs and a
                    sample of them is stored to prove the regeneration matches
  broadcast_add.npz head-sharing cases of broadcast_add (g = 1, 2)
  decoder_tiny.npz  a tiny weight-shared Qwen3-shape decoder assembled from the reference's
                    blocks: tokens, loss, logits sample, gradient samples

The reference never calls LoRAModule.reset_parameters here (it raises NameError: `math`
is not imported in that file); weights are set explicitly.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("WSL_REFERENCE_CHECKOUT", "reference")
sys.path.insert(0, REF)
sys.path.insert(1, ROOT)

from torchtitan.models.llama3.model.model import LoRAModule, broadcast_add  # noqa: E402
from torchtitan.experiments.qwen3.model.model import Qwen3Model  # noqa: E402
from torchtitan.experiments.qwen3.model.args import Qwen3ModelArgs  # noqa: E402

from oracle import lora_oracle as O  # noqa: E402

torch.set_num_threads(os.cpu_count() or 1)


class RefLoRALinear(nn.Module):
    """base nn.Linear + reference LoRAModule joined by the reference broadcast_add, exactly
    the q/k/v composition of torchtitan/models/llama3/model/model.py:376-398."""

    def __init__(self, base: nn.Linear, rank: int):
        super().__init__()
        self.base = base
        self.offset = LoRAModule(base.in_features, base.out_features, rank=rank)

    def forward(self, x):
        return broadcast_add(self.base(x), self.offset(x), dim=-1, g=1)


def ref_projection(W, A, B):
    base = nn.Linear(W.shape[1], W.shape[0], bias=False)
    m = RefLoRALinear(base, A.shape[0])
    with torch.no_grad():
        base.weight.copy_(W)
        m.offset.w_a.weight.copy_(A)
        m.offset.w_b.weight.copy_(B)
    return m


def sample(t: torch.Tensor, sr: int, sc: int) -> np.ndarray:
    return t.detach()[::sr, ::sc].contiguous().numpy()


def checks(t: torch.Tensor) -> np.ndarray:
    d = t.detach().double()
    return np.array([d.sum().item(), d.abs().sum().item(), (d * d).sum().item()])


def make_small():
    x, W, A, B, dY = O.projection_inputs(seed=77, M=96, N=72, K=80, r=8)
    m = ref_projection(W, A, B)
    xr = x.clone().requires_grad_(True)
    y = m(xr)
    y.backward(dY)
    np.savez(os.path.join(HERE, "lora_small.npz"), x=x.numpy(), W=W.numpy(), A=A.numpy(), B=B.numpy(),
             dY=dY.numpy(), y=y.detach().numpy(), dX=xr.grad.numpy(), dW=m.base.weight.grad.numpy(),
             dA=m.offset.w_a.weight.grad.numpy(), dB=m.offset.w_b.weight.grad.numpy())


def make_cfg0():
    inp = O.config0_inputs()
    W = inp["W"]
    base = nn.Linear(W.shape[1], W.shape[0], bias=False)
    with torch.no_grad():
        base.weight.copy_(W)
    mods, xs, ys = [], [], []
    for x, A, B in zip(inp["xs"], inp["As"], inp["Bs"]):
        m = RefLoRALinear(base, A.shape[0])   # every layer references the SAME base module
        with torch.no_grad():
            m.offset.w_a.weight.copy_(A)
            m.offset.w_b.weight.copy_(B)
        xr = x.clone().requires_grad_(True)
        mods.append(m)
        xs.append(xr)
        ys.append(m(xr))
    total = sum((y * dY).sum() for y, dY in zip(ys, inp["dYs"]))
    total.backward()
    out = {"in_W": sample(W, 61, 67), "in_x0": sample(inp["xs"][0], 127, 61),
           "in_A3": sample(inp["As"][3], 3, 67), "in_B2": sample(inp["Bs"][2], 61, 3),
           "in_dY1": sample(inp["dYs"][1], 127, 61),
           "dW_s": sample(base.weight.grad, 31, 29), "dW_c": checks(base.weight.grad)}
    for l, (m, xr, y) in enumerate(zip(mods, xs, ys)):
        out[f"y{l}_s"] = sample(y, 97, 89)
        out[f"y{l}_c"] = checks(y)
        out[f"dX{l}_s"] = sample(xr.grad, 97, 89)
        out[f"dX{l}_c"] = checks(xr.grad)
        out[f"dA{l}"] = m.offset.w_a.weight.grad.numpy()[:, ::7].copy()
        out[f"dA{l}_c"] = checks(m.offset.w_a.weight.grad)
        out[f"dB{l}"] = m.offset.w_b.weight.grad.numpy()[::7].copy()
        out[f"dB{l}_c"] = checks(m.offset.w_b.weight.grad)
    np.savez(os.path.join(HERE, "lora_cfg0.npz"), **out)


def make_broadcast_add():
    g = torch.Generator().manual_seed(5)
    out = {}
    for name, (gg, H, D) in {"g1": (1, 4, 8), "g2": (2, 8, 4)}.items():
        base = torch.randn(3, 5, gg * D, generator=g)
        delta = torch.randn(3, 5, H * D, generator=g)
        out[f"{name}_base"] = base.numpy()
        out[f"{name}_delta"] = delta.numpy()
        out[f"{name}_out"] = broadcast_add(base, delta, dim=-1, g=gg).numpy()
        out[f"{name}_g"] = np.array(gg)
    np.savez(os.path.join(HERE, "broadcast_add.npz"), **out)


TINY = dict(dim=64, hidden_dim=160, n_layers=4, n_unique=2, n_heads=4, n_kv_heads=2, head_dim=16,
            rank=8, vocab_size=512, embed_rank=32, max_seq_len=24)


def make_decoder():
    a = O.DecoderArgs(**TINY)
    p = O.init_decoder_params(a, seed=4321)
    # non-trivial norm weights so they are exercised
    g = torch.Generator().manual_seed(99)
    for k in list(p):
        if k.endswith("norm"):
            p[k] = 1.0 + 0.1 * torch.randn(p[k].shape, generator=g)
    args = Qwen3ModelArgs(dim=a.dim, n_layers=a.n_layers, n_heads=a.n_heads, n_kv_heads=a.n_kv_heads,
                          vocab_size=a.vocab_size, head_dim=a.head_dim, hidden_dim=a.hidden_dim,
                          norm_eps=a.norm_eps, rope_theta=a.rope_theta, max_seq_len=a.max_seq_len)
    model = Qwen3Model(args)
    bases = {}
    for u in range(a.n_unique):
        for name, (o, i) in O.proj_shapes(a).items():
            lin = nn.Linear(i, o, bias=False)
            with torch.no_grad():
                lin.weight.copy_(p[f"blocks.{u}.{name}.weight"])
            bases[(u, name)] = lin
    with torch.no_grad():
        for l in range(a.n_layers):
            blk = model.layers[str(l)]
            for name in O.PROJ_NAMES:
                m = RefLoRALinear(bases[(l % a.n_unique, name)], a.rank)
                m.offset.w_a.weight.copy_(p[f"layers.{l}.{name}.w_a"])
                m.offset.w_b.weight.copy_(p[f"layers.{l}.{name}.w_b"])
                owner = blk.attention if name in ("wq", "wk", "wv", "wo") else blk.feed_forward
                setattr(owner, name, m)
            blk.attention_norm.weight.copy_(p[f"layers.{l}.attention_norm"])
            blk.ffn_norm.weight.copy_(p[f"layers.{l}.ffn_norm"])
            blk.attention.q_norm.weight.copy_(p[f"layers.{l}.q_norm"])
            blk.attention.k_norm.weight.copy_(p[f"layers.{l}.k_norm"])
        emb = nn.Embedding(a.vocab_size, a.embed_rank)
        emb.weight.copy_(p["embed.E_small"])
        proj = nn.Linear(a.embed_rank, a.dim, bias=False)
        proj.weight.copy_(p["embed.P"])
        model.tok_embeddings = nn.Sequential(emb, proj)
        model.norm.weight.copy_(p["norm"])
        model.output.weight.copy_(p["output"])
    tg = torch.Generator().manual_seed(7)
    tokens = torch.randint(0, a.vocab_size, (2, a.max_seq_len), generator=tg)
    labels = torch.randint(0, a.vocab_size, (2, a.max_seq_len), generator=tg)
    logits = model(tokens)
    loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1).float(), labels.flatten(0, 1))
    loss.backward()
    out = {"tokens": tokens.numpy(), "labels": labels.numpy(), "loss": np.array(loss.item()),
           "logits_s": logits.detach()[:, ::5, ::37].contiguous().numpy(),
           "norm_scale_seed": np.array(99)}
    for (u, name), lin in bases.items():
        out[f"g.blocks.{u}.{name}.weight"] = lin.weight.grad.numpy()
    for l in (0, a.n_layers - 1):
        blk = model.layers[str(l)]
        out[f"g.layers.{l}.wq.w_a"] = blk.attention.wq.offset.w_a.weight.grad.numpy()
        out[f"g.layers.{l}.wq.w_b"] = blk.attention.wq.offset.w_b.weight.grad.numpy()
        out[f"g.layers.{l}.w2.w_a"] = blk.feed_forward.w2.offset.w_a.weight.grad.numpy()
        out[f"g.layers.{l}.w2.w_b"] = blk.feed_forward.w2.offset.w_b.weight.grad.numpy()
        out[f"g.layers.{l}.ffn_norm"] = blk.ffn_norm.weight.grad.numpy()
        out[f"g.layers.{l}.q_norm"] = blk.attention.q_norm.weight.grad.numpy()
    out["g.embed.P"] = proj.weight.grad.numpy()
    out["g.embed.E_small_rows"] = emb.weight.grad[tokens.flatten()[:8]].numpy()
    out["g.output_s"] = model.output.weight.grad[::17, ::3].contiguous().numpy()
    np.savez(os.path.join(HERE, "decoder_tiny.npz"), **out)


if __name__ == "__main__":
    print("torch", torch.__version__, "reference at", REF)
    make_small()
    make_broadcast_add()
    make_cfg0()
    make_decoder()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
