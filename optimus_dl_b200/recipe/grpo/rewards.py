"""Reward functions and prompt sources of the GRPO recipe (registries ``grpo_reward`` and ``grpo_prompts``)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ...core.registry import RegistryConfig, make_registry

_REWARDS, register_reward, build_reward = make_registry("grpo_reward")
_PROMPTS, register_prompts, build_prompts = make_registry("grpo_prompts")


@dataclass
class EvenFractionConfig(RegistryConfig):
    pass


@register_reward("even_fraction", EvenFractionConfig)
class EvenFractionReward:
    """Deterministic reward: the fraction of generated ids that are even (over the unmasked positions)."""

    def __init__(self, cfg: Any = None, **_: Any):
        self.cfg = cfg

    def __call__(self, prompts: torch.Tensor, completions: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        even = ((completions % 2) == 0) & mask
        return even.sum(-1).float() / mask.sum(-1).clamp(min=1).float()


@dataclass
class TargetTokenConfig(RegistryConfig):
    token_id: int = 0


@register_reward("target_token_fraction", TargetTokenConfig)
class TargetTokenReward:
    """Fraction of generated ids equal to ``token_id`` (a sharper learning signal for smoke tests)."""

    def __init__(self, cfg: Any = None, **_: Any):
        self.token_id = int(cfg.token_id) if cfg is not None else 0

    def __call__(self, prompts: torch.Tensor, completions: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        hit = (completions == self.token_id) & mask
        return hit.sum(-1).float() / mask.sum(-1).clamp(min=1).float()


@dataclass
class UniformRandomPromptsConfig(RegistryConfig):
    low: int = 0
    high: int | None = None        # default: the model's vocabulary size


@register_prompts("uniform_random", UniformRandomPromptsConfig)
class UniformRandomPrompts:
    """Prompts of uniform random token ids, a different slice of one seeded stream per rank and step."""

    def __init__(self, cfg: Any = None, vocab_size: int = 0, seed: int = 0, rank: int = 0, world_size: int = 1, **_: Any):
        self.low = int(cfg.low) if cfg is not None else 0
        high = cfg.get("high") if cfg is not None and hasattr(cfg, "get") else None
        self.high = int(high) if high is not None else int(vocab_size)
        self.seed, self.rank, self.world = int(seed), int(rank), int(world_size)

    def __call__(self, step: int, n_local: int, length: int, device: torch.device) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + step) & 0x7FFFFFFF)
        all_ids = torch.randint(self.low, self.high, (n_local * self.world, length), generator=g)
        return all_ids[self.rank * n_local:(self.rank + 1) * n_local].to(device)
