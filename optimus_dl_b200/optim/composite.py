"""``composite``: several optimizers behind one ``torch.optim.Optimizer`` face
(optimus_dl/modules/optim/composite.py:55-330).

Parameters are routed to named sub-optimizers by regular expressions on their names
(``params_regexp``; at most one entry may use ``None`` = everything not matched before). The
composite owns one ``state`` mapping that every child shares and its ``param_groups`` are the very
dict objects of the children, so ``state_dict()`` / ``load_state_dict()`` / LR schedulers see a
single ordinary optimizer. Each group is tagged with ``composite_optimizer_path`` (outermost name
first) and ``composite_optimizer_name``.
"""

from __future__ import annotations

import dataclasses
import re
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

import torch
from torch.optim.optimizer import Optimizer

from ..core.registry import RegistryConfig, RegistryConfigStrict
from . import build_optimizer, register_optimizer


@dataclass
class CompositeOptimizerConfigEntry(RegistryConfig):
    params_regexp: str | None = ".*"
    optimizer_config: Any = field(default_factory=dict)


@dataclass
class CompositeOptimizerConfig(RegistryConfigStrict):
    optimizers: dict = field(default_factory=dict)


class CompositeOptimizer(Optimizer):
    def __init__(self, optimizers: Iterable[Optimizer] | dict[str, Optimizer], **kwargs: Any):
        if isinstance(optimizers, dict):
            self.optimizers: dict[str, Optimizer] = dict(sorted(optimizers.items()))
        else:
            self.optimizers = {str(i): o for i, o in enumerate(optimizers)}
        if not self.optimizers:
            raise ValueError("At least one optimizer must be provided.")
        merged: list[dict] = []
        for name, child in self.optimizers.items():
            for group in child.param_groups:
                group.setdefault("composite_optimizer_path", [])
                group["composite_optimizer_path"].insert(0, name)
                group["composite_optimizer_name"] = name
                merged.append(group)
        super().__init__(merged, {})
        # Optimizer.__init__ copies nothing here: ``merged`` holds the children's own dicts, and
        # add_param_group keeps them, so a scheduler writing group["lr"] reaches the child.
        self._share_state(self.state)

    def _share_state(self, state: Any) -> None:
        for child in self.optimizers.values():
            child.state = state
            if isinstance(child, CompositeOptimizer):
                child._share_state(state)

    def step(self, closure: Callable[[], float] | None = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for child in self.optimizers.values():
            child.step()
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        for child in self.optimizers.values():
            child.zero_grad(set_to_none=set_to_none)

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        super().load_state_dict(state_dict)   # rebuilds self.param_groups and self.state as new objects
        self._relink()

    def _relink(self) -> None:
        cursor = 0
        for child in self.optimizers.values():
            n = len(child.param_groups)
            mine = self.param_groups[cursor:cursor + n]
            cursor += n
            child.state = self.state
            child.param_groups.clear()
            child.param_groups.extend(mine)
        for child in self.optimizers.values():
            if isinstance(child, CompositeOptimizer):
                child._relink()

    def __repr__(self) -> str:
        return "CompositeOptimizer(" + ", ".join(f"{k}={v!r}" for k, v in self.optimizers.items()) + ")"


def _is_named(p: Any) -> bool:
    return isinstance(p, tuple) and len(p) == 2 and isinstance(p[0], str) and isinstance(p[1], torch.Tensor)


def get_subgroup(params: Any, predicate: Callable[[str, torch.Tensor], bool]) -> list:
    """Filter named parameters (``[(name, tensor)]`` or ``[{"params": [(name, tensor)], ...}]``) by a predicate;
    groups that end up empty are dropped, other group keys are kept."""
    params = list(params)
    if any(isinstance(p, torch.Tensor) for p in params):
        raise ValueError("CompositeOptimizer requires named optimizers with regex matching, not a flat list of parameters.")
    if params and all(_is_named(p) for p in params):
        return [(n, t) for n, t in params if predicate(n, t)]
    out = []
    for group in params:
        assert isinstance(group, dict) and "params" in group, "Each parameter group dict must have a 'params' key."
        assert all(_is_named(p) for p in group["params"]), \
            "If using dicts, each 'params' entry must be a list of (name, tensor) tuples."
        kept = [(n, t) for n, t in group["params"] if predicate(n, t)]
        if kept:
            out.append({**{k: v for k, v in group.items() if k != "params"}, "params": kept})
    return out


def _iter_named(params: list) -> Iterable[tuple[str, torch.Tensor]]:
    for item in params:
        if _is_named(item):
            yield item
        else:
            yield from item["params"]


@register_optimizer("composite", CompositeOptimizerConfig)
def make_composite_optimizer(cfg: Any, params: Any, **kwargs: Any) -> CompositeOptimizer:
    params = list(params)
    names = {id(t): n for n, t in _iter_named(params)}
    entries = dict(cfg.optimizers)

    def regexp_of(entry: Any) -> str | None:  # an explicit ``None`` means "everything that is left"
        if dataclasses.is_dataclass(entry):
            return getattr(entry, "params_regexp", ".*")
        return entry["params_regexp"] if "params_regexp" in entry else ".*"

    def optimizer_config_of(entry: Any) -> Any:
        return entry.optimizer_config if dataclasses.is_dataclass(entry) else entry["optimizer_config"]

    assert sum(1 for e in entries.values() if regexp_of(e) is None) <= 1, \
        "Only one optimizer can have params_regexp set to None (match all remaining)."
    order = sorted(entries.items(), key=lambda kv: (regexp_of(kv[1]) is None, kv[0]))
    claimed: set[int] = set()
    built: dict[str, Optimizer] = {}
    for name, entry in order:
        rx = regexp_of(entry)
        if rx is None:
            sub = get_subgroup(params, lambda n, t: id(t) not in claimed)
        else:
            pattern = re.compile(rx)
            sub = get_subgroup(params, lambda n, t, pattern=pattern: pattern.match(n) is not None)
        if not sub:
            raise ValueError(f"Optimizer '{name}' with regex '{rx}' did not match any parameters.")
        for n, t in _iter_named(sub):
            if id(t) in claimed:
                raise ValueError(f"Parameter '{n}' matched by multiple optimizers (currently matched by '{name}').")
            claimed.add(id(t))
        built[name] = build_optimizer(optimizer_config_of(entry), params=sub, **kwargs)
    missing = [n for i, n in names.items() if i not in claimed]
    if missing:
        raise ValueError(f"The following parameters were not matched by any optimizer regex: {missing}")
    return CompositeOptimizer(built)
