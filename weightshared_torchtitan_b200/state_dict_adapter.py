"""State-dict interop between WeightSharedDecoder and a reference Qwen3 model that went through
SharedLoRAConverter (torchtitan/experiments/qwen3/model/model.py:105-448 after converter.py).

The converted reference model names its parameters

    tok_embeddings.embed.weight / tok_embeddings.proj.weight          (FactorizedEmbedding)
    layers.{l}.attention.{wq,wk,wv,wo}.base.weight                    (shared: layer l mod n_unique)
    layers.{l}.attention.{wq,wk,wv,wo}.offset.w_a.weight / .w_b.weight
    layers.{l}.attention.{q_norm,k_norm}.weight
    layers.{l}.feed_forward.{w1,w2,w3}.base.weight / .offset.w_{a,b}.weight
    layers.{l}.{attention_norm,ffn_norm}.weight,  norm.weight,  output.weight

(the scheme of the reference's own adapters, torchtitan/models/llama3/model/state_dict_adapter.py:24-41:
a flat key map, no tensor is re-laid out). A base weight shared by several layers appears under
every layer that uses it, as nn.Module.state_dict() of the converted model does; `deduplicate`
gives the form a checkpoint writer wants: every shared tensor once, plus an alias table.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .decoder import PROJ_NAMES, WeightSharedDecoder

_OWNER = {"wq": "attention", "wk": "attention", "wv": "attention", "wo": "attention",
          "w1": "feed_forward", "w2": "feed_forward", "w3": "feed_forward"}


def to_reference(model: WeightSharedDecoder) -> Dict[str, torch.Tensor]:
    """Parameters of the decoder under the converted reference model's names (no copies: shared
    base weights are the same tensor object under every layer that uses them)."""
    c = model.config
    sd: Dict[str, torch.Tensor] = {
        "tok_embeddings.embed.weight": model.tok_embeddings.embed.weight,
        "tok_embeddings.proj.weight": model.tok_embeddings.proj.weight,
        "norm.weight": model.norm.weight,
        "output.weight": model.output.weight,
    }
    for l, lyr in enumerate(model.layers):
        blk = model.blocks[l % c.n_unique]
        for n in PROJ_NAMES:
            pre = f"layers.{l}.{_OWNER[n]}.{n}"
            off = getattr(lyr, f"{n}_offset")
            sd[f"{pre}.base.weight"] = getattr(blk, n).weight
            sd[f"{pre}.offset.w_a.weight"] = off.w_a.weight
            sd[f"{pre}.offset.w_b.weight"] = off.w_b.weight
        sd[f"layers.{l}.attention.q_norm.weight"] = lyr.q_norm.weight
        sd[f"layers.{l}.attention.k_norm.weight"] = lyr.k_norm.weight
        sd[f"layers.{l}.attention_norm.weight"] = lyr.attention_norm.weight
        sd[f"layers.{l}.ffn_norm.weight"] = lyr.ffn_norm.weight
    return sd


@torch.no_grad()
def from_reference(model: WeightSharedDecoder, sd: Dict[str, torch.Tensor], check_shared: bool = True) -> None:
    """Loads a converted reference model's state dict into the decoder. Every layer's copy of a
    shared base weight must be the same values (they are one tensor in the reference model)."""
    own = to_reference(model)
    missing = sorted(set(own) - set(sd))
    unexpected = sorted(set(sd) - set(own))
    if missing or unexpected:
        raise KeyError(f"state dict does not fit: missing {missing[:4]}..., unexpected {unexpected[:4]}...")
    done: Dict[int, str] = {}
    for k, dst in own.items():
        src = sd[k]
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{k}: shape {tuple(src.shape)} != {tuple(dst.shape)}")
        first = done.get(id(dst))
        if first is not None:
            if check_shared and not torch.equal(sd[first].to(dst.device, dst.dtype), src.to(dst.device, dst.dtype)):
                raise ValueError(f"{k} and {first} share one base weight here but differ in the state dict")
            continue
        dst.copy_(src.to(dst.device, dst.dtype))
        done[id(dst)] = k
    # the compute-dtype copies follow the new masters, also the flat copy of a model that a
    # TrainStep has already bound to its arena
    model.post_optimizer_hook()


def deduplicate(sd: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    """(unique, aliases): every tensor once under the first key that names it, and
    alias key -> first key for the others (cross-layer shared base weights)."""
    unique: Dict[str, torch.Tensor] = {}
    aliases: Dict[str, str] = {}
    seen: Dict[Tuple[int, int, Tuple[int, ...]], str] = {}
    for k, t in sd.items():
        ident = (t.data_ptr(), t.numel(), tuple(t.shape))
        if ident in seen and t.numel() > 0:
            aliases[k] = seen[ident]
        else:
            seen[ident] = k
            unique[k] = t
    return unique, aliases


def expand(unique: Dict[str, torch.Tensor], aliases: Dict[str, str]) -> Dict[str, torch.Tensor]:
    """Inverse of deduplicate."""
    sd = dict(unique)
    for k, first in aliases.items():
        sd[k] = unique[first]
    return sd
