"""Process teardown: close loggers' backends, kill child processes, and arm a watchdog that
force-exits if interpreter shutdown stalls (optimus_dl/core/multiprocess.py:13-151)."""

from __future__ import annotations

import logging
import os
import sys
import threading
import time

from .environment import OPTIMUS_EXIT_TIMEOUT

logger = logging.getLogger(__name__)


def _kill_loky_workers() -> None:
    try:
        from joblib.externals.loky import get_reusable_executor

        get_reusable_executor().shutdown(wait=False, kill_workers=True)
    except Exception:
        pass


def _finish_wandb() -> None:
    if "wandb" in sys.modules:
        try:
            import wandb

            if wandb.run is not None:
                wandb.finish()
        except Exception:
            pass


def _finish_mlflow() -> None:
    if "mlflow" in sys.modules:
        try:
            import mlflow

            if mlflow.active_run() is not None:
                mlflow.end_run()
        except Exception:
            pass


def _kill_children(rounds: int = 10) -> None:
    try:
        import psutil
    except ImportError:
        return
    me = psutil.Process(os.getpid())
    for i in range(rounds):
        children = me.children(recursive=True)
        if not children:
            return
        for c in children:
            try:
                c.terminate() if i < rounds // 2 else c.kill()
            except psutil.Error:
                pass
        psutil.wait_procs(children, timeout=0.5)


def _watchdog(timeout: float) -> None:
    def run() -> None:
        time.sleep(timeout)
        os._exit(0)

    threading.Thread(target=run, daemon=True, name="optimus-exit-watchdog").start()


def finalize_process(exit_timeout: float | None = None) -> None:
    """Best-effort cleanup at the end of an entry point; never raises."""
    _kill_loky_workers()
    _finish_wandb()
    _finish_mlflow()
    _kill_children()
    t = OPTIMUS_EXIT_TIMEOUT.get() if exit_timeout is None else exit_timeout
    if t and t > 0:
        _watchdog(float(t))


# names the reference exports for the individual teardown steps (optimus_dl/core/multiprocess.py:101-151)
force_terminate_joblib = _kill_loky_workers
finish_wandb = _finish_wandb
finish_mlflow = _finish_mlflow
