"""Size-bounded shard writer for tokenised documents (optimus_dl/recipe/pretokenize/sharder.py:23-183).

On-disk format (read back by ``data/datasets/tokenized_dataset.py``): ``<name>_<10-digit idx>.npy``
holds the shard's tokens as one flat array, ``<name>_<idx>_lens.npy`` the document lengths
(uint32), and ``index.json`` lists ``{file, lens_file, num_tokens, num_docs, shard_idx}`` per shard
plus ``total_tokens`` and the producing config. Tokens are staged in a preallocated numpy buffer
of the shard's byte budget instead of a Python list.
"""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any

import numpy as np

logger = logging.getLogger(__name__)


class Sharder:
    def __init__(self, output_config: Any, proc_config: Any):
        self.output_dir = Path(str(output_config.dir))
        self.output_name = str(output_config.name)
        self.max_shard_bytes = int(float(proc_config.shard_size_mb) * 1024 * 1024)    # fractions of a MB are allowed
        self._dtype = np.dtype(np.uint16 if str(proc_config.dtype) == "uint16" else np.uint32)
        self._cap = max(self.max_shard_bytes // self._dtype.itemsize, 1)
        self._buf = np.empty(min(self._cap, 1 << 20), dtype=self._dtype)
        self._n = 0
        self._lens: list[int] = []
        self.shard_idx = 0
        self.file_metadata: list[dict[str, Any]] = []
        self.total_tokens = 0

    # ------------------------------------------------------------------ state
    def get_state(self) -> dict[str, Any]:
        return {"shard_idx": self.shard_idx, "file_metadata": [dict(m) for m in self.file_metadata],
                "total_tokens": self.total_tokens, "current_shard_tokens": self._buf[: self._n].copy(),
                "current_shard_doc_lens": list(self._lens)}

    def load_state(self, state: dict[str, Any]) -> None:
        self.shard_idx = int(state.get("shard_idx", 0))
        self.file_metadata = [dict(m) for m in state.get("file_metadata", [])]
        self.total_tokens = int(state.get("total_tokens", 0))
        cur = np.asarray(state.get("current_shard_tokens", []), dtype=self.dtype)
        self._reserve(len(cur))
        self._buf[: len(cur)] = cur
        self._n = len(cur)
        self._lens = [int(x) for x in state.get("current_shard_doc_lens", [])]

    @property
    def dtype(self) -> np.dtype:
        return self._dtype

    @dtype.setter
    def dtype(self, value: Any) -> None:
        """Changing the token type converts what is already staged."""
        value = np.dtype(value)
        if value != self._dtype:
            self._buf, self._dtype = self._buf.astype(value), value
            self._cap = max(self.max_shard_bytes // value.itemsize, 1)

    @property
    def current_shard_tokens(self) -> list[int]:
        """The staged tokens of the open shard as a list (a copy: for inspection and state, not for appending)."""
        return self._buf[: self._n].tolist()

    @property
    def current_shard_doc_lens(self) -> list[int]:
        return list(self._lens)

    @property
    def current_shard_size_bytes(self) -> int:
        return self._n * np.dtype(self.dtype).itemsize

    def _reserve(self, n: int) -> None:
        if n > len(self._buf):
            new = np.empty(max(n, min(2 * len(self._buf), max(self._cap, n))), dtype=self.dtype)
            new[: self._n] = self._buf[: self._n]
            self._buf = new

    # ------------------------------------------------------------------ writing
    def add(self, doc_tokens: Any) -> bool:
        """Append one document; returns True when a shard was written first to make room."""
        doc = np.asarray(doc_tokens)
        flushed = False
        if self._n and (self._n + len(doc)) * np.dtype(self.dtype).itemsize > self.max_shard_bytes:
            self.flush()
            flushed = True
        self._reserve(self._n + len(doc))
        self._buf[self._n:self._n + len(doc)] = doc
        self._n += len(doc)
        self._lens.append(len(doc))
        return flushed

    def flush(self) -> None:
        if not self._n:
            return
        self.output_dir.mkdir(parents=True, exist_ok=True)
        shard = f"{self.output_name}_{self.shard_idx:010d}.npy"
        lens = f"{self.output_name}_{self.shard_idx:010d}_lens.npy"
        logger.info("saving shard %s (%s tokens, %s docs)", shard, f"{self._n:,}", f"{len(self._lens):,}")
        np.save(self.output_dir / shard, self._buf[: self._n])
        np.save(self.output_dir / lens, np.asarray(self._lens, dtype=np.uint32))
        self.file_metadata.append({"file": shard, "lens_file": lens, "num_tokens": int(self._n),
                                   "num_docs": len(self._lens), "shard_idx": self.shard_idx})
        self.total_tokens += int(self._n)
        self.shard_idx += 1
        self._n = 0
        self._lens = []

    def finalize(self, final_config: dict[str, Any]) -> None:
        self.flush()
        self.output_dir.mkdir(parents=True, exist_ok=True)
        index = {"files": self.file_metadata, "total_tokens": self.total_tokens, "config": final_config}
        (self.output_dir / "index.json").write_text(json.dumps(index, indent=2))
        logger.info("done: %s tokens in %d shards; index at %s", f"{self.total_tokens:,}", len(self.file_metadata),
                    self.output_dir / "index.json")
