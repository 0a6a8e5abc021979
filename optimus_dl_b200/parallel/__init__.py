"""Distributed runtime: collectives, symmetric peer memory, FSDP/TP/SP engines."""

from .collective import (  # noqa: F401
    Collective,
    DistributedConfig,
    FakeCollective,
    MeshCollective,
    build_best_collective,
    reset_collective,
)
