"""``causal_lm``: run the model on the batch and expose logits, targets, mask and the classification
view (optimus_dl/modules/metrics/sources/causal_lm.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..source import MetricSource, MetricSourceConfig, StandardProtocols as P, register_metric_source


@dataclass
class CausalLMSourceConfig(MetricSourceConfig):
    padding_token_id: int = -100


@register_metric_source("causal_lm", CausalLMSourceConfig)
class CausalLMSource(MetricSource):
    provides = {P.LOGITS, P.LOGITS_TARGETS, P.LOGITS_MASK, P.CLASSIFICATION, P.INPUT_TOKENS}

    @torch.no_grad()
    def __call__(self, dependencies: dict[str, Any], model: Any = None, batch: dict | None = None, **kwargs: Any):
        from ...criterion.cross_entropy import CrossEntropyCriterion

        inputs, targets = CrossEntropyCriterion.prepare_batch(batch)
        logits = model(**inputs)["logits"]
        pad = int(self.cfg.padding_token_id)
        if pad != -100:
            targets = torch.where(targets == pad, torch.full_like(targets, -100), targets)
        mask = targets != -100
        return {P.LOGITS: logits, P.LOGITS_TARGETS: targets, P.LOGITS_MASK: mask, P.INPUT_TOKENS: inputs["input_ids"],
                P.CLASSIFICATION: {"predictions": logits.argmax(-1), "targets": targets, "mask": mask}}
