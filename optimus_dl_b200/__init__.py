"""B200-native LLM training framework with the capabilities of Optimus-DL.

Importing the package does what the reference's package init does
(optimus_dl/__init__.py:31-42): one intra-op CPU thread per process (data workers and ranks
multiply; override with ``OPTIMUS_DL_NUM_THREADS``), a version string, and a bootstrap pass that
imports every component package so that all ``@register_*`` decorators have run.
"""

import os as _os

__version__ = "0.1.0"

_BOOTSTRAPPED = False


def bootstrap() -> None:
    """Import all registry-bearing sub-packages (idempotent)."""
    global _BOOTSTRAPPED
    if _BOOTSTRAPPED:
        return
    _BOOTSTRAPPED = True
    import importlib

    for name in ("models", "criterion", "optim", "lr_scheduler", "data", "tokenizer", "metrics", "loggers",
                 "model_transforms", "checkpoint", "recipe.train", "recipe.metrics", "recipe.eval", "recipe.serve",
                 "recipe.pretokenize", "recipe.grpo"):
        try:
            importlib.import_module(f"{__name__}.{name}")
        except ModuleNotFoundError as err:  # optional third-party dependency of one component
            if err.name and err.name.startswith(__name__):
                raise
            import logging

            logging.getLogger(__name__).debug("component %s skipped: %s", name, err)


def _init() -> None:
    from .core import aliases

    aliases.install()      # the reference's module paths that differ from this tree resolve to the modules here
    from .core import config_utils  # noqa: F401  (registers the eval / env / hash resolvers of the config system)
    threads = _os.environ.get("OPTIMUS_DL_NUM_THREADS", "1")
    try:
        import torch

        if int(threads) > 0:
            torch.set_num_threads(int(threads))
    except Exception:  # noqa: BLE001 - torch missing or refusing the value must not break the import
        pass
    if _os.environ.get("OPTIMUS_DL_NO_BOOTSTRAP") != "1":
        bootstrap()


_init()
