"""Metric sources: causal_lm, generation, model_info."""

from .causal_lm import CausalLMSource, CausalLMSourceConfig  # noqa: F401
from .generation import GenerationSource, GenerationSourceConfig  # noqa: F401
from .model_info import ModelInfoSource, ModelInfoSourceConfig  # noqa: F401
