"""A TrainSpec that lets the reference trainer drive the fused path.

The reference selects a model family by name (``--model.name``) from a registry of TrainSpec
records (torchtitan/protocols/train_spec.py:42-80: model class, flavors, parallelize function
and the builders of optimizer, scheduler, data loader, tokenizer, loss). Its own ``qwen3`` spec
cannot run as shipped: ``parallelize_qwen3`` reads ``job_config.training.compile``, a field the
config no longer has (torchtitan/experiments/qwen3/infra/parallelize.py:51,78,119). This module
registers ``qwen3_shared_lora``: the reference's Qwen3Model, flavors and builders, with a
parallelize function for the one strategy this path uses, replicated data parallelism:

    torchrun ... -m torchtitan.train --model.name qwen3_shared_lora --model.flavor 8B \\
        --experimental.custom_import weightshared_torchtitan_b200.train_spec \\
        --experimental.custom_args_module weightshared_torchtitan_b200.job_config_ext \\
        --model.converters shared_lora --shared_lora.n_unique 4 --shared_lora.rank 64

With DDP the module-level API returns weight gradients to autograd (``grad_in_place`` off), so
the reference's ``replicate(..., bucket_cap_mb=100)`` hooks see them
(torchtitan/models/llama3/infra/parallelize.py:428-444); the flat-arena exchange of dp.GradArena
belongs to this package's own TrainStep.
"""
from __future__ import annotations

import sys

SPEC_NAME = "qwen3_shared_lora"


def parallelize_shared_lora(model, parallel_dims, job_config):
    """Replicated data parallelism only; every other strategy is refused rather than ignored."""
    for flag in ("tp_enabled", "cp_enabled", "pp_enabled", "dp_shard_enabled", "ep_enabled"):
        if getattr(parallel_dims, flag, False):
            raise NotImplementedError(f"{SPEC_NAME} covers replicated data parallelism; {flag} is set")
    if getattr(parallel_dims, "dp_replicate_enabled", False):
        from torch.distributed._composable.replicate import replicate
        replicate(model, device_mesh=parallel_dims.world_mesh["dp_replicate"], bucket_cap_mb=100)
    return model


def register_with_torchtitan() -> bool:
    """Enter the spec and the converter in the trainer's registries. False when torchtitan (with
    its Qwen3 experiment) cannot be imported."""
    try:
        from torchtitan.components.loss import build_cross_entropy_loss
        from torchtitan.components.lr_scheduler import build_lr_schedulers
        from torchtitan.components.optimizer import build_optimizers
        from torchtitan.components.tokenizer import build_hf_tokenizer
        from torchtitan.components.validate import build_validator
        from torchtitan.datasets.hf_datasets import build_hf_dataloader
        from torchtitan.experiments.qwen3 import Qwen3Model, qwen3_configs
        from torchtitan.protocols import train_spec as ts
    except Exception:   # noqa: BLE001 - absent, or a checkout that does not import here
        return False
    from . import converter
    converter.register_with_torchtitan()
    if SPEC_NAME not in ts._train_specs:
        ts.register_train_spec(ts.TrainSpec(
            name=SPEC_NAME, model_cls=Qwen3Model, model_args=qwen3_configs,
            parallelize_fn=parallelize_shared_lora, pipelining_fn=None,
            build_optimizers_fn=build_optimizers, build_lr_schedulers_fn=build_lr_schedulers,
            build_dataloader_fn=build_hf_dataloader, build_tokenizer_fn=build_hf_tokenizer,
            build_loss_fn=build_cross_entropy_loss, build_validator_fn=build_validator))
    return True


if "torchtitan" in sys.modules:
    register_with_torchtitan()
