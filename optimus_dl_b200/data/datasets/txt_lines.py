"""``txt_lines``: lines of a local text file or URL, sharded by line index across ranks
(optimus_dl/modules/data/datasets/txt_lines.py:21-168). Remote files are cached under
``cache_dir`` keyed by the sha256 of the URL."""

from __future__ import annotations

import hashlib
import os
import urllib.request
from dataclasses import dataclass
from typing import Any

from ...core.registry import RegistryConfigStrict
from . import register_dataset
from .base import BaseDataset


@dataclass
class TxtLinesDatasetConfig(RegistryConfigStrict):
    file_link: str = "???"
    cache_dir: str = "~/.cache/optimus_dl/txt_lines"
    skip_empty_lines: bool = True
    field: str = "text"
    lines_per_item: int = 1


@register_dataset("txt_lines", TxtLinesDatasetConfig)
class TxtLinesDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        self.path = self._resolve(cfg.file_link, os.path.expanduser(cfg.cache_dir))
        self._lines: list[str] | None = None
        self.index = self.limit = 0

    @staticmethod
    def _resolve(link: str, cache_dir: str) -> str:
        if link.startswith(("http://", "https://")):
            os.makedirs(cache_dir, exist_ok=True)
            path = os.path.join(cache_dir, hashlib.sha256(link.encode()).hexdigest() + ".txt")
            if not os.path.exists(path):
                tmp = path + ".tmp"
                urllib.request.urlretrieve(link, tmp)
                os.replace(tmp, path)
            return path
        return os.path.expanduser(link)

    def _load(self) -> list[str]:
        """All items of the file; this rank's share is ``[start, limit)`` with ``total // world_size`` items per rank
        (the remainder is left out, so every rank has equally many: optimus_dl/modules/data/datasets/txt_lines.py:
        115-127)."""
        if self._lines is None:
            with open(self.path, encoding="utf-8") as f:
                lines = [l.rstrip("\n") for l in f]
            if self.cfg.skip_empty_lines:
                lines = [l for l in lines if l.strip()]
            n = int(self.cfg.lines_per_item)
            if n > 1:
                lines = ["\n".join(lines[i:i + n]) for i in range(0, len(lines), n)]
            self._lines = lines
            per = len(lines) // self.world_size
            self.start, self.limit = per * self.rank, per * (self.rank + 1)
        return self._lines

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        st = initial_state or {}
        assert st.get("rank", self.rank) == self.rank and st.get("world_size", self.world_size) == self.world_size, \
            "txt_lines must be resumed with the same rank and world size"
        self._load()
        self.index = int(st["index"]) if "index" in st else self.start      # a position in the whole file

    def get_state(self) -> dict[str, Any]:
        return {"index": self.index, "file_link": self.cfg.file_link, "skip_empty_lines": bool(self.cfg.skip_empty_lines),
                "rank": self.rank, "world_size": self.world_size}

    def next(self) -> dict[str, Any]:
        lines = self._load()
        if self.index >= self.limit:
            raise StopIteration
        item = {self.cfg.field: lines[self.index]}
        self.index += 1
        return item
