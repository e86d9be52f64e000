"""Model-converter plug-in: swap a Qwen3-style model's projections for the fused path.

Mirrors the reference's converter seam, torchtitan/protocols/model_converter.py:15-84: a
converter has ``__init__(job_config, parallel_dims)``, ``convert(model)`` (in place, before
parallelisation and weight init, so it also works on meta-device models) and
``post_optimizer_hook(model)``; converters are registered by name with
``register_model_converter`` and built with ``build_model_converters``. The precedent for a
converter that swaps ``nn.Linear`` modules is Float8Converter,
torchtitan/components/quantization/float8.py:149-176.

What convert() does to a model shaped like torchtitan/experiments/qwen3/model/model.py
(``model.layers`` a ModuleDict/ModuleList of blocks with ``attention.{wq,wk,wv,wo}`` and
``feed_forward.{w1,w2,w3}``, ``model.tok_embeddings``):
  * layer l keeps its own LoRAModule per projection but takes its base nn.Linear from layer
    (l mod n_unique): cross-layer weight sharing by sharing the module object, the
    mechanism the reference uses for its own parameter sharing (model.py:154-182);
  * every projection becomes SharedLoRALinear(base, offset) (one fused GEMM);
  * tok_embeddings becomes FactorizedEmbedding(vocab, embed_rank, dim) when embed_rank > 0.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Type

import torch.nn as nn

from .modules import GLOBAL_COPY_CACHE, FactorizedEmbedding, LoRAModule, SharedLoRALinear

ATTN_PROJ = ("wq", "wk", "wv", "wo")
FFN_PROJ = ("w1", "w2", "w3")


@dataclass
class SharedLoRAConfig:
    """The knobs the converter reads from ``job_config.shared_lora`` (any object with these
    attributes; missing ones fall back to the defaults). The reference's JobConfig has no such
    section; ``job_config_ext.JobConfig`` adds it through the reference's own extension
    mechanism, ``--experimental.custom_args_module weightshared_torchtitan_b200.job_config_ext``
    (torchtitan/config/manager.py:86-155), after which ``--shared_lora.rank 64`` etc. and a
    ``[shared_lora]`` TOML table are parsed like any built-in section."""
    n_unique: int = 4
    rank: int = 16
    embed_rank: int = 0          # 0 keeps the full embedding
    grad_in_place: bool = False  # True: fp32 in-place weight gradients (use dp.GradArena)


class SharedLoRAConverter:
    def __init__(self, job_config=None, parallel_dims=None):
        src = getattr(job_config, "shared_lora", None)
        d = SharedLoRAConfig()
        self.config = SharedLoRAConfig(**{k: getattr(src, k, getattr(d, k)) for k in d.__dataclass_fields__})
        self.parallel_dims = parallel_dims

    def convert(self, model: nn.Module) -> nn.Module:
        c = self.config
        layers = list(model.layers.values()) if hasattr(model.layers, "values") else list(model.layers)
        if c.n_unique < 1 or c.n_unique > len(layers):
            raise ValueError(f"n_unique must be in [1, {len(layers)}]")
        for l, blk in enumerate(layers):
            donor = layers[l % c.n_unique]
            for owner_name, names in (("attention", ATTN_PROJ), ("feed_forward", FFN_PROJ)):
                owner, d_owner = getattr(blk, owner_name), getattr(donor, owner_name)
                for n in names:
                    cur = getattr(d_owner, n)
                    base = cur.base if isinstance(cur, SharedLoRALinear) else cur
                    if not isinstance(base, nn.Linear):
                        raise TypeError(f"{owner_name}.{n} of layer {l} is not an nn.Linear")
                    off = LoRAModule(base.in_features, base.out_features, rank=c.rank)
                    off.to(device=base.weight.device, dtype=base.weight.dtype)
                    setattr(owner, n, SharedLoRALinear(base, off, grad_in_place=c.grad_in_place))
        emb = getattr(model, "tok_embeddings", None)
        if c.embed_rank > 0 and isinstance(emb, nn.Embedding):
            fe = FactorizedEmbedding(emb.num_embeddings, c.embed_rank, emb.embedding_dim)
            fe.to(device=emb.weight.device, dtype=emb.weight.dtype)
            model.tok_embeddings = fe
        return model

    def post_optimizer_hook(self, model):
        """Weights changed: compute-dtype copies are re-cast on next use (the cache keys on
        the tensors' version counters; clearing only releases the stale copies early)."""
        GLOBAL_COPY_CACHE.clear()


_registry_model_converter_cls: Dict[str, Type] = {}


def register_model_converter(converter_cls: Type, name: str):
    """Same contract as the reference's register_model_converter (model_converter.py:41-50)."""
    assert name not in _registry_model_converter_cls, f"A model converter '{name}' is already registered."
    _registry_model_converter_cls[name] = converter_cls


class ModelConvertersContainer:
    """Applies the converters named in ``job_config.model.converters`` in order
    (reference: ModelConvertersContainer, model_converter.py:53-84)."""

    def __init__(self, job_config, parallel_dims=None):
        names = list(getattr(getattr(job_config, "model", None), "converters", []) or [])
        self.converters = [_registry_model_converter_cls[n](job_config, parallel_dims) for n in names]

    def convert(self, model: nn.Module):
        for c in self.converters:
            c.convert(model)

    def post_optimizer_hook(self, model):
        for c in self.converters:
            c.post_optimizer_hook(model)


def build_model_converters(job_config, parallel_dims=None) -> ModelConvertersContainer:
    return ModelConvertersContainer(job_config, parallel_dims)


register_model_converter(SharedLoRAConverter, "shared_lora")


def register_with_torchtitan() -> bool:
    """Also enter the converter under the name ``shared_lora`` in the trainer's own registry,
    torchtitan.protocols.model_converter (register_model_converter, l.41-50), so that
    ``--model.converters shared_lora`` selects it. Returns False when torchtitan cannot be
    imported. Runs by itself when this module is imported inside a process that already
    loaded torchtitan (``--experimental.custom_import weightshared_torchtitan_b200.converter``,
    torchtitan/train.py:78-79); importing torchtitan just for this would cost seconds."""
    try:
        from torchtitan.protocols import model_converter as mc
    except Exception:   # noqa: BLE001 - absent, or a checkout that does not import here
        return False
    if "shared_lora" not in mc._registry_model_converter_cls:
        mc.register_model_converter(SharedLoRAConverter, "shared_lora")
    return True


if "torchtitan" in sys.modules:
    register_with_torchtitan()
