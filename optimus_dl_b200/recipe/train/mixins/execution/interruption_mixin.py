"""Interruption handling (optimus_dl/recipe/train/mixins/execution/interruption_mixin.py:12-75): on
``KeyboardInterrupt`` a final checkpoint is written through the supplied callback."""

from __future__ import annotations

import logging
from typing import Any, Callable

logger = logging.getLogger(__name__)


class TrainingInterruptionMixin:
    def handle_training_interruption(self, iteration: int, save_callback: Callable[[int], Any] | None = None) -> None:
        logger.warning("training interrupted at iteration %d", iteration)
        if save_callback is None:
            return
        try:
            save_callback(iteration)
            logger.info("final checkpoint written at iteration %d", iteration)
        except Exception as e:  # the interrupt must still propagate cleanly
            logger.error("could not write the final checkpoint: %s", e)
