"""JobConfig extension that gives the reference trainer a ``shared_lora`` section.

The reference merges a user module's ``JobConfig`` dataclass into its own when started with
``--experimental.custom_args_module <module>`` (torchtitan/config/manager.py:86-155,
torchtitan/config/job_config.py:703-708): fields that exist only here are added, so

    torchrun ... -m torchtitan.train --job.config_file cfg.toml \\
        --experimental.custom_import weightshared_torchtitan_b200.converter \\
        --experimental.custom_args_module weightshared_torchtitan_b200.job_config_ext \\
        --model.converters shared_lora --shared_lora.n_unique 4 --shared_lora.rank 64 \\
        --shared_lora.embed_rank 1024 --shared_lora.grad_in_place

reaches ``converter.SharedLoRAConverter`` as ``job_config.shared_lora``. Plain dataclasses
only: the reference builds its command-line parser from the field types and docstrings.
"""
from dataclasses import dataclass, field


@dataclass
class SharedLoRA:
    n_unique: int = 4
    """Number of unique blocks; layer l takes its base projections from layer l mod n_unique"""

    rank: int = 16
    """Rank r of the per-layer adapters on q, k, v, o, gate, up and down"""

    embed_rank: int = 0
    """Inner width r_e of the factorized token embedding; 0 keeps the full embedding"""

    grad_in_place: bool = False
    """Accumulate fp32 weight gradients in place into param.grad (use with dp.GradArena)"""


@dataclass
class JobConfig:
    shared_lora: SharedLoRA = field(default_factory=SharedLoRA)
