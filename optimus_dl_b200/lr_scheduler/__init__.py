"""Learning-rate schedules and the ``lr_scheduler`` registry (``_name``: cosine_annealing,
linear_warmup, wsd)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseLRScheduler, BaseLRSchedulerConfig

_LR_REGISTRY, register_lr_scheduler, build_lr_scheduler = make_registry("lr_scheduler", BaseLRScheduler)
bootstrap_module(__name__)
