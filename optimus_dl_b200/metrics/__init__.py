"""Meters, metric engine, metric sources and their registries."""

from .base import (  # noqa: F401
    BaseMeter,
    MeterEntry,
    MeterGroup,
    compute_meters,
    load_state_dict,
    log_meter,
    meters_group,
    reset_meters,
    state_dict,
    step_meters,
)
from .common import (  # noqa: F401
    cached_lambda,
    log_averaged,
    log_averaged_exponent,
    log_event_end,
    log_event_occurence,
    log_event_start,
    log_gathered,
    log_max,
    log_min,
    log_summed,
)
from . import engine, metrics, source  # noqa: E402,F401
from .sources import causal_lm as _s1, generation as _s2, model_info as _s3  # noqa: E402,F401
from .engine import MetricEngine  # noqa: E402,F401
