"""``preset_hfllama2``: a Llama whose shape (and weights) come from a Hugging Face Llama checkpoint
(optimus_dl/modules/model/presets/hf_llama.py:25-127)."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

from .. import register_model
from ..llama2 import Llama, LlamaConfig
from . import utils

logger = logging.getLogger(__name__)


def __getattr__(name: str) -> Any:
    return utils.lazy_hub_class(__name__, name)


@dataclass
class HFLlamaConfig(LlamaConfig):
    hf_model_name: str = "meta-llama/Llama-2-7b-hf"
    load_weights: bool = True      # False: only the shape is taken, weights stay randomly initialised
    head_dim: int | None = None


RULES = utils.COMMON_RULES + utils.PRENORM_RULES


def llama_from_hf(cfg: Any, hf_config: Any, hf_state_dict: dict | None) -> Llama:
    utils.update_config_from_hf(cfg, hf_config)
    model = Llama(cfg)
    if hf_state_dict is not None:
        utils.load_weights(model, hf_state_dict, RULES, cfg)
    return model


@register_model("preset_hfllama2", HFLlamaConfig)
def make_hf_llama_model(cfg: Any, **_: Any) -> Llama:
    logger.info("loading HF model %s", cfg.hf_model_name)
    hf_config = utils.load_hf_config(cfg.hf_model_name, globals().get("AutoConfig"))
    sd = utils.load_hf_state_dict(cfg.hf_model_name, globals().get("AutoModelForCausalLM")) if cfg.load_weights else None
    return llama_from_hf(cfg, hf_config, sd)
