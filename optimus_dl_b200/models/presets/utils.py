"""Conversion of Hugging Face causal-LM checkpoints to this package's parameter layout
(optimus_dl/modules/model/presets/utils.py:15-219).

Two differences need care: parameter names, and rotary embeddings — Hugging Face rotates the pair
``(x[i], x[i + hd/2])`` while this package rotates neighbouring elements ``(x[2i], x[2i+1])``, so
the output rows of the query / key projections (and per-head QK-norm weights) are re-ordered per
head. The mapping is a table of ``Rule`` rows applied by ``convert_state_dict``.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch

logger = logging.getLogger(__name__)


def permute_rope_weight(w: torch.Tensor, n_heads: int, head_dim: int, interleaved: bool = True) -> torch.Tensor:
    """Re-order rows from half-split to interleaved rotary layout. ``w`` is ``[n_heads * head_dim, ...]``
    or a per-head vector ``[head_dim]`` shared by all heads; other shapes are returned untouched."""
    if not interleaved:
        return w
    if w.shape[0] == head_dim:
        heads = 1
    elif w.shape[0] == n_heads * head_dim:
        heads = n_heads
    else:
        logger.warning("unexpected shape %s for a rotary permutation (head_dim %d, heads %d): left as is",
                       tuple(w.shape), head_dim, n_heads)
        return w
    half = head_dim // 2
    v = w.reshape(heads, 2, half, *w.shape[1:])          # [head, (first|second half), i, ...]
    return v.transpose(1, 2).reshape(w.shape)            # [head, i, (first|second), ...] -> x[2i], x[2i+1]


@dataclass(frozen=True)
class Rule:
    src: str                      # Hugging Face key, ``{i}`` = layer index
    dst: str                      # local key
    rope_heads: str | None = None  # config attribute with the head count when rows follow the rotary layout
    per_layer: bool = True
    optional: bool = False


class WeightMapper:
    """Copies tensors of a Hugging Face state dict into a local state dict and keeps score."""

    def __init__(self, hf_sd: dict[str, torch.Tensor], local_sd: dict[str, torch.Tensor]):
        self.hf_sd, self.local_sd = hf_sd, local_sd
        self.loaded_keys: set[str] = set()

    def copy(self, src_key: str, dest_key: str, permute: bool = False, n_heads: int | None = None,
             head_dim: int | None = None, transpose: bool = False, dim: int = 0) -> None:
        if src_key not in self.hf_sd:
            if dest_key in self.local_sd:
                logger.warning("Missing key in HF model: %s", src_key)
            return
        w = self.hf_sd[src_key]
        if transpose:
            w = w.t()
        if permute:
            assert n_heads is not None and head_dim is not None
            w = permute_rope_weight(w, n_heads, head_dim) if dim == 0 else permute_rope_weight(w.t(), n_heads, head_dim).t()
        if dest_key not in self.local_sd:
            logger.warning("Extra key in HF model not in local model: %s", dest_key)
            return
        dst = self.local_sd[dest_key]
        if dst.shape != w.shape:
            logger.warning("Shape mismatch for %s: %s vs %s. Attempting reshape.", dest_key, tuple(dst.shape), tuple(w.shape))
            w = w.reshape(dst.shape)
        with torch.no_grad():
            dst.copy_(w)
        self.loaded_keys.add(dest_key)

    def apply(self, rules: list[Rule], cfg: Any) -> None:
        for rule in rules:
            layers = range(int(cfg.n_layer)) if rule.per_layer else [None]
            for i in layers:
                src = rule.src.format(i=i) if i is not None else rule.src
                dst = rule.dst.format(i=i) if i is not None else rule.dst
                if rule.optional and src not in self.hf_sd:
                    continue
                if rule.rope_heads is not None:
                    self.copy(src, dst, permute=True, n_heads=int(getattr(cfg, rule.rope_heads)), head_dim=int(cfg.head_dim))
                else:
                    self.copy(src, dst)

    def validate(self, tie_word_embeddings: bool = False, ignore_patterns: list[str] | None = None) -> set[str]:
        missing = set(self.local_sd) - self.loaded_keys
        missing = {k for k in missing if "inv_freq" not in k and not any(p in k for p in (ignore_patterns or []))}
        if tie_word_embeddings:
            for a, b in (("transformer.wte.weight", "lm_head.weight"), ("lm_head.weight", "transformer.wte.weight")):
                if a in self.loaded_keys:
                    missing.discard(b)
        if missing:
            logger.warning("Missing keys in loaded model: %s", sorted(missing))
        else:
            logger.info("All weights loaded successfully.")
        return missing


def update_config_from_hf(cfg: Any, hf: Any, head_dim_fallback: int | None = None) -> None:
    """Fill the shape fields of a local model config from a ``transformers`` config."""
    cfg.n_layer = hf.num_hidden_layers
    cfg.n_head = hf.num_attention_heads
    cfg.n_embd = hf.hidden_size
    cfg.vocab_size = hf.vocab_size
    cfg.sequence_length = getattr(hf, "max_position_embeddings", 2048)
    cfg.block_size = cfg.sequence_length
    cfg.rmsnorm_eps = getattr(hf, "rms_norm_eps", getattr(hf, "layer_norm_epsilon", 1e-5))
    cfg.intermediate_size = getattr(hf, "intermediate_size", None)
    cfg.tie_word_embeddings = bool(getattr(hf, "tie_word_embeddings", False))
    scaling = next((v for v in (getattr(hf, "rope_scaling", None), getattr(hf, "rope_parameters", None))
                    if isinstance(v, dict) and v), None)
    theta = getattr(hf, "rope_theta", None)
    if theta is None and scaling is not None:
        theta = scaling.get("rope_theta")
    if hasattr(cfg, "rope_theta") and theta is not None:
        cfg.rope_theta = float(theta)
    if scaling is not None:
        if hasattr(cfg, "rope_scaling"):
            cfg.rope_scaling = dict(scaling)
        if hasattr(cfg, "rope_parameters"):
            cfg.rope_parameters = dict(scaling)
    cfg.n_kv_head = getattr(hf, "num_key_value_heads", None) or hf.num_attention_heads
    hd = getattr(hf, "head_dim", None)
    cfg.head_dim = hd if isinstance(hd, int) else (head_dim_fallback or cfg.n_embd // cfg.n_head)


def lazy_hub_class(module_name: str, name: str) -> Any:
    """Module ``__getattr__`` of the preset modules: ``AutoConfig`` and ``AutoModelForCausalLM`` are module-level
    names there (callers can substitute them) that import ``transformers`` on first use only."""
    if name in ("AutoConfig", "AutoModelForCausalLM"):
        import transformers

        return getattr(transformers, name)
    raise AttributeError(f"module {module_name!r} has no attribute {name!r}")


def load_hf_config(name_or_path: str, auto_config: Any = None) -> Any:
    """``auto_config``: the class to ask (a preset module's ``AutoConfig`` when something replaced it)."""
    if auto_config is None:
        from transformers import AutoConfig as auto_config

    return auto_config.from_pretrained(name_or_path)


def load_hf_state_dict(name_or_path: str, auto_model: Any = None) -> dict[str, torch.Tensor]:
    if auto_model is None:
        from transformers import AutoModelForCausalLM as auto_model

    model = auto_model.from_pretrained(name_or_path, dtype=torch.float32, low_cpu_mem_usage=True)
    return model.state_dict()


COMMON_RULES = [
    Rule("model.embed_tokens.weight", "transformer.wte.weight", per_layer=False),
    Rule("model.norm.weight", "transformer.ln_f.weight", per_layer=False),
    Rule("lm_head.weight", "lm_head.weight", per_layer=False, optional=True),
    Rule("model.layers.{i}.self_attn.q_proj.weight", "transformer.h.{i}.attn.wq.weight", rope_heads="n_head"),
    Rule("model.layers.{i}.self_attn.k_proj.weight", "transformer.h.{i}.attn.wk.weight", rope_heads="n_kv_head"),
    Rule("model.layers.{i}.self_attn.v_proj.weight", "transformer.h.{i}.attn.wv.weight"),
    Rule("model.layers.{i}.self_attn.o_proj.weight", "transformer.h.{i}.attn.wo.weight"),
    Rule("model.layers.{i}.self_attn.q_proj.bias", "transformer.h.{i}.attn.wq.bias", rope_heads="n_head", optional=True),
    Rule("model.layers.{i}.self_attn.k_proj.bias", "transformer.h.{i}.attn.wk.bias", rope_heads="n_kv_head", optional=True),
    Rule("model.layers.{i}.self_attn.v_proj.bias", "transformer.h.{i}.attn.wv.bias", optional=True),
    Rule("model.layers.{i}.self_attn.o_proj.bias", "transformer.h.{i}.attn.wo.bias", optional=True),
    Rule("model.layers.{i}.mlp.gate_proj.weight", "transformer.h.{i}.mlp.w1.weight"),
    Rule("model.layers.{i}.mlp.up_proj.weight", "transformer.h.{i}.mlp.w2.weight"),
    Rule("model.layers.{i}.mlp.down_proj.weight", "transformer.h.{i}.mlp.c_proj.weight"),
]

PRENORM_RULES = [
    Rule("model.layers.{i}.input_layernorm.weight", "transformer.h.{i}.ln_1.weight"),
    Rule("model.layers.{i}.post_attention_layernorm.weight", "transformer.h.{i}.ln_2.weight"),
]

QK_NORM_RULES = [
    Rule("model.layers.{i}.self_attn.q_norm.weight", "transformer.h.{i}.attn.q_norm.weight", rope_heads="n_head"),
    Rule("model.layers.{i}.self_attn.k_norm.weight", "transformer.h.{i}.attn.k_norm.weight", rope_heads="n_kv_head"),
]

POSTNORM_RULES = [
    Rule("model.layers.{i}.post_attention_layernorm.weight", "transformer.h.{i}.post_attention_layernorm.weight"),
    Rule("model.layers.{i}.post_feedforward_layernorm.weight", "transformer.h.{i}.post_feedforward_layernorm.weight"),
]


def load_weights(model: torch.nn.Module, hf_sd: dict[str, torch.Tensor], rules: list[Rule], cfg: Any) -> set[str]:
    """Copy ``hf_sd`` into ``model`` following ``rules``; returns the local keys that stayed untouched."""
    mapper = WeightMapper(hf_sd, model.state_dict())
    mapper.apply(rules, cfg)
    if bool(cfg.tie_word_embeddings) and "lm_head.weight" not in mapper.loaded_keys:
        mapper.copy("model.embed_tokens.weight", "lm_head.weight")
    return mapper.validate(tie_word_embeddings=bool(cfg.tie_word_embeddings))
