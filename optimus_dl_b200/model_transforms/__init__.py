"""Model transforms and the ``model_transform`` registry (``_name``: ddp, fully_shard,
tensor_parallel, compile, activation_checkpoint, load_weights, transformer_engine)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseModelTransform
from .config import ModelTransformConfig

_TRANSFORMS_REGISTRY, register_model_transform, build_model_transform = make_registry("model_transform", BaseModelTransform)
bootstrap_module(__name__)
