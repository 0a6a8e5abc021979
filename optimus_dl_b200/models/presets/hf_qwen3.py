"""``preset_hfqwen3``: Qwen-3 from a Hugging Face checkpoint (optimus_dl/modules/model/presets/hf_qwen3.py:25-183).
Per-head QK-norm weights follow the rotary row order, so they are permuted like the projections."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

from .. import register_model
from ..qwen3 import Qwen3, Qwen3Config
from . import utils

logger = logging.getLogger(__name__)


def __getattr__(name: str) -> Any:
    return utils.lazy_hub_class(__name__, name)


@dataclass
class HFQwen3Config(Qwen3Config):
    hf_model_name: str = "Qwen/Qwen3-4B-Thinking-2507"
    load_weights: bool = True


RULES = utils.COMMON_RULES + utils.PRENORM_RULES + utils.QK_NORM_RULES


def qwen3_from_hf(cfg: Any, hf_config: Any, hf_state_dict: dict | None) -> Qwen3:
    utils.update_config_from_hf(cfg, hf_config)
    cfg.rmsnorm_eps = getattr(hf_config, "rms_norm_eps", getattr(hf_config, "layer_norm_epsilon", 1e-6))
    cfg.attention_bias = bool(getattr(hf_config, "attention_bias", False))
    sw = getattr(hf_config, "sliding_window", None)
    cfg.sliding_window = sw if getattr(hf_config, "use_sliding_window", False) else None
    model = Qwen3(cfg)
    if hf_state_dict is not None:
        utils.load_weights(model, hf_state_dict, RULES, cfg)
    return model


@register_model("preset_hfqwen3", HFQwen3Config)
def make_hf_qwen3_model(cfg: Any, **_: Any) -> Qwen3:
    logger.info("loading HF model %s", cfg.hf_model_name)
    hf_config = utils.load_hf_config(cfg.hf_model_name, globals().get("AutoConfig"))
    sd = utils.load_hf_state_dict(cfg.hf_model_name, globals().get("AutoModelForCausalLM")) if cfg.load_weights else None
    return qwen3_from_hf(cfg, hf_config, sd)
