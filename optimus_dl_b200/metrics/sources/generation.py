"""``generation``: sample continuations of the batch's prompts (greedy, temperature, top-k, top-p; stops
per sequence at EOS) and expose them as ``generated_tokens``
(optimus_dl/modules/metrics/sources/generation.py:20-177). Uses the KV-cache decoder of
``recipe/generation.py`` when the model supports it, else re-runs the full prefix per token."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..source import MetricSource, MetricSourceConfig, StandardProtocols as P, register_metric_source


@dataclass
class GenerationSourceConfig(MetricSourceConfig):
    max_new_tokens: int = 50
    temperature: float = 1.0
    top_k: int | None = None
    top_p: float | None = None
    do_sample: bool = False          # the reference's switch: False = greedy search (its default)
    greedy: bool | None = None       # explicit override; None = derived from do_sample
    eos_token_id: int | None = None
    prompt_length: int | None = None
    use_kv_cache: bool = True


def sample_next(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None, top_p: float | None = None,
                greedy: bool = False, generator: torch.Generator | None = None) -> torch.Tensor:
    """Pick next tokens from ``logits (B, V)``."""
    if greedy or temperature == 0:
        return logits.argmax(-1)
    logits = logits.float() / max(temperature, 1e-6)
    if top_k is not None and top_k > 0:
        kth = torch.topk(logits, min(int(top_k), logits.shape[-1])).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0 < top_p < 1:
        sl, si = torch.sort(logits, descending=True)
        cp = torch.softmax(sl, -1).cumsum(-1)
        drop = cp - torch.softmax(sl, -1) > top_p
        sl = sl.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, si, sl)
    return torch.multinomial(torch.softmax(logits, -1), 1, generator=generator).squeeze(-1)


@register_metric_source("generation", GenerationSourceConfig)
class GenerationSource(MetricSource):
    provides = {P.GENERATED_TOKENS}

    @torch.no_grad()
    def __call__(self, dependencies: dict[str, Any], model: Any = None, batch: dict | None = None, **kwargs: Any):
        ids = batch["input_ids"]
        if self.cfg.prompt_length:
            ids = ids[:, : int(self.cfg.prompt_length)]
        from ...recipe.generation import generate

        out = generate(model, ids, max_new_tokens=int(self.cfg.max_new_tokens), temperature=float(self.cfg.temperature),
                       top_k=self.cfg.top_k, top_p=self.cfg.top_p, greedy=(bool(self.cfg.greedy) if self.cfg.greedy is not None else not bool(self.cfg.do_sample)),
                       eos_token_id=self.cfg.eos_token_id, use_kv_cache=bool(self.cfg.use_kv_cache))
        return {P.GENERATED_TOKENS: out}
