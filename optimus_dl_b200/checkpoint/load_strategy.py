"""What to restore from a checkpoint (optimus_dl/modules/checkpoint/load_strategy.py:15-85)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class LoadStrategy:
    load_model: bool = True
    load_optimizer: bool = True
    load_scheduler: bool = True
    load_data_sources: bool = True
    load_dataloaders: bool = True
    load_metrics: bool = True
    load_iteration: bool = True
    extra_ignore_keys: list[str] = field(default_factory=list)

    @classmethod
    def from_cfg(cls, cfg) -> "LoadStrategy":
        if cfg is None:
            return cls()
        if isinstance(cfg, cls):
            return cfg
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: (list(cfg[k]) if k == "extra_ignore_keys" else cfg[k]) for k in keys if k in cfg})
