"""Model families and the ``model`` registry (``_name``: gpt2, llama2, qwen3, olmo3, preset_hf*)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseModel
from .config import ModelConfig

_MODELS_REGISTRY, register_model, build_model = make_registry("model")
bootstrap_module(__name__)
