"""``preset_hfolmo3``: OLMo-3 from a Hugging Face checkpoint (optimus_dl/modules/model/presets/hf_olmo3.py:25-191).
QK-norm spans the full projection width here, so its weights are permuted head by head."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

from .. import register_model
from ..olmo3 import Olmo3, Olmo3Config
from . import utils

logger = logging.getLogger(__name__)


def __getattr__(name: str) -> Any:
    return utils.lazy_hub_class(__name__, name)


@dataclass
class HFOlmo3Config(Olmo3Config):
    hf_model_name: str = "allenai/Olmo-3-1025-7B"
    load_weights: bool = True


RULES = utils.COMMON_RULES + utils.QK_NORM_RULES + utils.POSTNORM_RULES


def olmo3_from_hf(cfg: Any, hf_config: Any, hf_state_dict: dict | None) -> Olmo3:
    utils.update_config_from_hf(cfg, hf_config)
    cfg.rmsnorm_eps = getattr(hf_config, "rms_norm_eps", 1e-6)
    cfg.sliding_window = getattr(hf_config, "sliding_window", 4096)
    default_types = (["sliding_attention"] * 3 + ["full_attention"]) * (cfg.n_layer // 4 + 1)
    cfg.layer_types = list(getattr(hf_config, "layer_types", None) or default_types[: cfg.n_layer])
    cfg.attention_bias = bool(getattr(hf_config, "attention_bias", False))
    model = Olmo3(cfg)
    if hf_state_dict is not None:
        utils.load_weights(model, hf_state_dict, RULES, cfg)
    return model


@register_model("preset_hfolmo3", HFOlmo3Config)
def make_hf_olmo3_model(cfg: Any, **_: Any) -> Olmo3:
    logger.info("loading HF model %s", cfg.hf_model_name)
    hf_config = utils.load_hf_config(cfg.hf_model_name, globals().get("AutoConfig"))
    sd = utils.load_hf_state_dict(cfg.hf_model_name, globals().get("AutoModelForCausalLM")) if cfg.load_weights else None
    return olmo3_from_hf(cfg, hf_config, sd)
