"""Configuration of the GRPO recipe.

The reference has no reinforcement-learning recipe; this one follows the layout of its train
recipe config (optimus_dl/recipe/train/config.py) so that model, transforms, optimizer, loggers
and checkpointing are configured the same way, and adds a ``grpo`` section.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ...core.registry import RegistryConfigStrict
from ...parallel.collective import DistributedConfig


@dataclass
class GRPOCommonConfig:
    exp_name: str = "grpo"
    seed: int = 42
    data_seed: int = 42
    output_path: str = "outputs/grpo"
    use_gpu: bool = True
    distributed: DistributedConfig = field(default_factory=lambda: DistributedConfig(sharding_world_size=None))
    log_freq: int = 1
    save_freq: int = 0            # persistent checkpoint every N iterations (0 = never)
    last_save_freq: int = 0


@dataclass
class GRPOSection:
    num_prompts: int = 64          # prompts per step over all ranks
    prompt_length: int = 256
    group_size: int = 8            # completions sampled per prompt
    max_new_tokens: int = 512
    temperature: float = 1.0
    top_k: int | None = None
    top_p: float | None = None
    eos_token_id: int | None = None
    clip_eps: float = 0.2
    kl_coef: float = 0.04
    updates_per_rollout: int = 1
    micro_batch_size: int = 8      # sequences per forward/backward
    rollout_batch_size: int = 64   # sequences decoded together
    advantage_eps: float = 1e-6
    use_kv_cache: bool = True
    use_cuda_graph: bool = True
    reward: Any = field(default_factory=lambda: {"_name": "even_fraction"})
    prompts: Any = field(default_factory=lambda: {"_name": "uniform_random"})


@dataclass
class GRPOOptimization:
    iterations: int = 100
    optimizer: Any = field(default_factory=lambda: {"_name": "adamw", "lr": 1e-6, "weight_decay": 0.0})
    clip_grad_norm: float | None = 1.0
    amp: Any = None


@dataclass
class GRPOConfig(RegistryConfigStrict):
    args: dict = field(default_factory=dict)
    common: GRPOCommonConfig = field(default_factory=GRPOCommonConfig)
    model: Any = "???"
    grpo: GRPOSection = field(default_factory=GRPOSection)
    optimization: GRPOOptimization = field(default_factory=GRPOOptimization)
    lr_scheduler: Any = None
    loggers: Any = None
    model_transforms: list = field(default_factory=list)
    model_builder: Any = field(default_factory=lambda: {"_name": "base"})
    optimizer_builder: Any = field(default_factory=lambda: {"_name": "base"})
    scheduler_builder: Any = field(default_factory=lambda: {"_name": "base"})
    checkpoint_manager: Any = field(default_factory=lambda: {"_name": "base"})
    logger_manager: Any = field(default_factory=lambda: {"_name": "base"})
