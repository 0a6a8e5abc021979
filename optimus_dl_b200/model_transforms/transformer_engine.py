"""``transformer_engine`` transform (optimus_dl/modules/model_transforms/transformer_engine.py:278-375).

The reference swaps ``nn.Linear`` / norm modules for NVIDIA Transformer Engine modules so that an
FP8 recipe has something to act on. Here FP8 execution is built in: the transform marks the weights
of the transformer blocks' linear layers as FP8-capable (``weight._fp8 = True``), and inside an
``FP8Recipe.autocast()`` context (``amp/fp8.py``) those layers run the block-scaled e4m3 GEMM of
``ops/fp8.py``. Modules and parameter names are untouched, so checkpoints stay interchangeable
with bf16 runs. The reference's knobs are accepted: ``replace_linear`` gates the marking;
``replace_norm`` marks the pre-norms of the converted blocks so that they emit the 1x128-quantised input of
the linear layers they feed from the norm launch itself; ``replace_attention`` has nothing to replace (the
attention kernels are already this package's own) and is ignored with a log line; ``linear_kwargs`` may carry
``skip_first_layers`` / ``skip_last_layers`` (blocks kept in bf16) and ``include_lm_head``.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch.nn as nn

from . import register_model_transform
from .base import BaseModelTransform
from .config import ModelTransformConfig

logger = logging.getLogger(__name__)


@dataclass
class TransformerEngineTransformConfig(ModelTransformConfig):
    enabled: bool = True
    replace_linear: bool = True
    replace_norm: bool = True
    replace_attention: bool = False
    linear_kwargs: Any = None
    norm_kwargs: Any = None
    attention_kwargs: Any = None
    replace_inplace: bool = True
    verbose: bool = False


def mark_fp8_norms(model: nn.Module, skip_first: int = 0, skip_last: int = 0) -> int:
    """Set ``_fp8_out`` on the pre-norms (``ln_1`` / ``ln_2``) of pre-norm blocks whose width fits the 128-wide
    scale blocks: under the block-scaled recipe they then write the e4m3 form of their output as well."""
    from ..models.blocks.layer_norms import RMSNorm

    blocks = list(getattr(getattr(model, "transformer", None), "h", []))
    n = 0
    for i, block in enumerate(blocks):
        if i < skip_first or i >= len(blocks) - skip_last:
            continue
        for name in ("ln_1", "ln_2"):
            mod = getattr(block, name, None)
            if isinstance(mod, RMSNorm) and mod.weight.numel() % 128 == 0:
                mod._fp8_out = True
                n += 1
    return n


def mark_fp8_linears(model: nn.Module, skip_first: int = 0, skip_last: int = 0, include_lm_head: bool = False,
                     verbose: bool = False) -> int:
    """Set ``weight._fp8`` on the block linears whose shapes fit the 128-wide scale blocks; returns the count."""
    blocks = list(getattr(getattr(model, "transformer", None), "h", []))
    n = 0
    for i, block in enumerate(blocks):
        if i < skip_first or i >= len(blocks) - skip_last:
            continue
        for name, mod in block.named_modules():
            if isinstance(mod, nn.Linear) and mod.in_features % 128 == 0 and mod.out_features % 16 == 0:
                mod.weight._fp8 = True
                n += 1
                if verbose:
                    logger.info("fp8: transformer.h.%d.%s [%d x %d]", i, name, mod.out_features, mod.in_features)
    if include_lm_head and hasattr(model, "lm_head") and model.lm_head.in_features % 128 == 0:
        model.lm_head.weight._fp8 = True
        n += 1
    return n


@register_model_transform("transformer_engine", TransformerEngineTransformConfig)
class TransformerEngineTransform(BaseModelTransform):
    def apply(self, model: nn.Module, **kwargs: Any) -> nn.Module:
        cfg = self.cfg
        if not bool(cfg.get("enabled", True)):
            return model
        if bool(cfg.get("replace_attention", False)):
            logger.info("transformer_engine: attention already runs this package's kernels; nothing to replace")
        if not bool(cfg.get("replace_linear", True)):
            return model
        kw = dict(cfg.get("linear_kwargs") or {})
        if bool(cfg.get("replace_norm", True)):
            n = mark_fp8_norms(model, int(kw.get("skip_first_layers", 0)), int(kw.get("skip_last_layers", 0)))
            logger.info("transformer_engine: %d pre-norms emit the quantised input of their linear layers", n)
        n = mark_fp8_linears(model, int(kw.get("skip_first_layers", 0)), int(kw.get("skip_last_layers", 0)),
                             bool(kw.get("include_lm_head", False)), bool(cfg.get("verbose", False)))
        logger.info("transformer_engine: %d linear layers marked for block-scaled fp8 execution", n)
        return model
