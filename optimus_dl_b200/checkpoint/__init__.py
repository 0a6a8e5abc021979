"""Checkpointing: manager, mid-evaluation state, load strategy."""

from ..core.registry import make_registry
from .load_strategy import LoadStrategy
from .checkpoint_manager import CheckpointManager, CheckpointManagerConfig, CheckpointPath
from .eval_checkpoint_manager import EvaluationCheckpointManager

_CKPT_REGISTRY, register_checkpoint_manager, build_checkpoint_manager = make_registry("checkpoint_manager")
register_checkpoint_manager("base", CheckpointManagerConfig)(CheckpointManager)
