"""Logging setup, tqdm wrappers that stay quiet off a TTY, and ``*_once`` helpers
(optimus_dl/core/log.py:15-224)."""

from __future__ import annotations

import logging
import os
import sys
from functools import lru_cache

from .environment import OPTIMUS_DEBUG

_FMT = "%(asctime)s | %(levelname)-7s | %(name)s | %(message)s"


def _console_handler(use_rich: bool | None) -> logging.Handler:
    tty = sys.stderr.isatty()
    if use_rich is None:
        use_rich = tty
    if use_rich:
        try:
            from rich.logging import RichHandler

            return RichHandler(rich_tracebacks=True, show_path=False)
        except ImportError:
            pass
    try:
        import colorlog  # optional

        h = colorlog.StreamHandler()
        h.setFormatter(colorlog.ColoredFormatter("%(log_color)s" + _FMT))
        return h
    except ImportError:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(_FMT))
        return h


def setup_logging(level: int | str | None = None, log_path: str | None = None, use_rich: bool | None = None,
                  keep_console: bool = True) -> None:
    """Configure the root logger. With ``log_path`` writes ``info.log``, ``error.log`` (and
    ``debug.log`` when ``OPTIMUS_DEBUG`` is set) into that directory."""
    if level is None:
        level = logging.DEBUG if OPTIMUS_DEBUG.get() else logging.INFO
    root = logging.getLogger()
    root.setLevel(level)
    for h in list(root.handlers):
        if getattr(h, "_optimus", False):
            root.removeHandler(h)
    handlers: list[logging.Handler] = []
    if keep_console or log_path is None:
        handlers.append(_console_handler(use_rich))
    if log_path is not None:
        os.makedirs(log_path, exist_ok=True)
        for name, lvl in (("info.log", logging.INFO), ("error.log", logging.ERROR)):
            fh = logging.FileHandler(os.path.join(log_path, name))
            fh.setLevel(lvl)
            fh.setFormatter(logging.Formatter(_FMT))
            handlers.append(fh)
        if OPTIMUS_DEBUG.get():
            fh = logging.FileHandler(os.path.join(log_path, "debug.log"))
            fh.setLevel(logging.DEBUG)
            fh.setFormatter(logging.Formatter(_FMT))
            handlers.append(fh)
    for h in handlers:
        h._optimus = True  # type: ignore[attr-defined]
        root.addHandler(h)


def tqdm(iterable=None, *args, **kwargs):
    """``tqdm`` that prints sparse plain lines when stderr is not a terminal."""
    from tqdm import tqdm as _tqdm

    if not sys.stderr.isatty():
        kwargs.setdefault("mininterval", 30.0)
        kwargs.setdefault("ascii", True)
        kwargs.setdefault("ncols", 100)
    return _tqdm(iterable, *args, **kwargs)


def trange(*args, **kwargs):
    return tqdm(range(*args), **kwargs)


@lru_cache(maxsize=None)
def _once(logger_name: str, level: int, msg: str) -> None:
    logging.getLogger(logger_name).log(level, msg)


def log_once(logger: logging.Logger, level: int, msg: str) -> None:
    _once(logger.name, level, msg)


def warn_once(logger: logging.Logger, msg: str) -> None:
    _once(logger.name, logging.WARNING, msg)


def info_once(logger: logging.Logger, msg: str) -> None:
    _once(logger.name, logging.INFO, msg)


def debug_once(logger: logging.Logger, msg: str) -> None:
    _once(logger.name, logging.DEBUG, msg)


def error_once(logger: logging.Logger, msg: str) -> None:
    _once(logger.name, logging.ERROR, msg)
