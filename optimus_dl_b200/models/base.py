"""``BaseModel``: the interface every model family implements
(optimus_dl/modules/model/base.py:52-131).

Forward contract: ``model(**batch) -> {"logits": Tensor}``. Models here additionally accept
``skip_lm_head=True`` and then return ``{"hidden": normed_states}`` so that the criterion can run the
fused linear + cross-entropy kernel path without materialising ``[tokens, vocab]`` logits.
"""

from __future__ import annotations

import logging
from typing import Any, Callable

import torch.nn

logger = logging.getLogger(__name__)


class BaseModel(torch.nn.Module):
    supports_fused_head = False

    def __init__(self) -> None:
        super().__init__()

    @classmethod
    def register_arch(cls, arch_name: str) -> Callable[[Callable[[], Any]], Any]:
        raise NotImplementedError("populated when the class is registered in the model registry")

    def make_parameter_groups(self) -> Any:
        """Optimizer parameter groups; default is one group with every named parameter."""
        return {"params": list(self.named_parameters())}

    def fully_shard(self, **fsdp_kwargs: Any) -> list[torch.nn.Module]:
        """Return the sub-modules that each form one sharding group (besides the root)."""
        logger.warning("Model does not define sharding groups; the whole model becomes one group.")
        return []

    def apply_tp(self, mesh: Any, **kwargs: Any) -> None:
        """Shard parameters for tensor parallelism over ``mesh`` (no-op by default)."""
        logger.warning("%s does not support tensor parallelism", type(self).__name__)

    def _fanout(self, hook: str) -> None:
        cache_name = f"_{hook}_modules"
        mods = getattr(self, cache_name, None)
        if mods is None:
            mods = [m for m in self.modules() if m is not self and callable(getattr(m, hook, None))]
            object.__setattr__(self, cache_name, mods)
        for m in mods:
            getattr(m, hook)()

    def pre_optimizer_step(self) -> None:
        self._fanout("pre_optimizer_step")

    def post_optimizer_step(self) -> None:
        self._fanout("post_optimizer_step")
