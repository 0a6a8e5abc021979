"""Documents -> token lists, in a deterministic and resumable order
(optimus_dl/recipe/pretokenize/processor.py:23-440).

Per file: texts are read, passed through a seeded shuffle buffer and tokenised. With
``num_proc > 1`` a pool of worker processes (spawn context) tokenises chunks of texts while the
parent keeps reading; results are consumed in submission order, so the output does not depend on
the worker count. Progress is ``(file index, documents emitted from that file)``: a resumed run
re-reads the interrupted file and skips what was already emitted — the shuffle is seeded per file,
so the order repeats exactly.
"""

from __future__ import annotations

import logging
import multiprocessing as mp
import random
from collections import deque
from typing import Any, Iterator

from ...core import conf
from .source import FileReader

logger = logging.getLogger(__name__)

_WORKER_TOKENIZER = None
CHUNK = 256


def _worker_init(tokenizer_cfg: Any) -> None:
    global _WORKER_TOKENIZER
    import torch

    torch.set_num_threads(1)
    from ...tokenizer import build_tokenizer

    _WORKER_TOKENIZER = build_tokenizer(conf.create(tokenizer_cfg) if isinstance(tokenizer_cfg, dict) else tokenizer_cfg)


def _worker_encode(texts: list[str]) -> list[list[int]]:
    return [list(_WORKER_TOKENIZER.encode(t)) for t in texts]


def shuffled(texts: Iterator[str], buffer_size: int | None, init_seed: int) -> Iterator[str]:
    """Block shuffle: collect ``buffer_size`` texts, shuffle them with a generator seeded ``init_seed + block index``,
    hand them out, start the next block (the order optimus_dl/recipe/pretokenize/processor.py:70-90 produces, so
    one seed gives the same shards in both code bases). ``None`` keeps the file's order."""
    if buffer_size is None:
        yield from texts
        return
    block, buf = 0, []
    for t in texts:
        buf.append(t)
        if len(buf) >= buffer_size:
            random.Random(init_seed + block).shuffle(buf)
            yield from buf
            block, buf = block + 1, []
    if buf:
        random.Random(init_seed + block).shuffle(buf)
        yield from buf


class TokenProcessor:
    def __init__(self, files: list[str], config: Any):
        self.files = list(files)
        self.config = config
        self.reader = FileReader(config.processing, config.dataset)
        self.num_proc = max(int(config.processing.num_proc), 1)
        self.file_idx = 0
        self.docs_in_file = 0
        self.total_docs_yielded = 0
        self._pool = None
        self._tokenizer = None

    # ------------------------------------------------------------------ state
    def get_state(self) -> dict[str, Any]:
        """Position under the reference's keys (optimus_dl/recipe/pretokenize/processor.py:237-247): the file being
        read, the index of the last document taken from it (``None`` before the first) and the running total; an
        interrupted run can be continued by either code base. ``file_idx`` / ``docs_in_file`` say the same in this
        package's earlier spelling."""
        return {"yielded_doc_idx": self.docs_in_file - 1 if self.docs_in_file > 0 else None,
                "yielded_file_idx": self.file_idx, "total_docs_yielded": self.total_docs_yielded,
                "file_idx": self.file_idx, "docs_in_file": self.docs_in_file}

    def load_state(self, state: dict[str, Any]) -> None:
        if "yielded_file_idx" in state:
            self.file_idx = int(state.get("yielded_file_idx") or 0)
            last = state.get("yielded_doc_idx")
            self.docs_in_file = int(last) + 1 if last is not None else 0
        else:
            self.file_idx = int(state.get("file_idx", 0))
            self.docs_in_file = int(state.get("docs_in_file", 0))
        self.total_docs_yielded = int(state.get("total_docs_yielded", 0))

    @property
    def progress(self) -> int:
        return self.file_idx

    # ------------------------------------------------------------------ iteration
    def _texts_of(self, idx: int) -> Iterator[str]:
        size = self.config.processing.shuffle_buffer_size
        return shuffled(self.reader.read_texts(self.files[idx]), int(size) if size is not None else None,
                        idx * 100 + int(self.config.processing.seed))

    def _tokenizer_cfg(self) -> Any:
        t = self.config.tokenizer
        return conf.to_container(t, resolve=True) if conf.is_config(t) else t

    def _encode_stream(self, texts: Iterator[str]) -> Iterator[list[int]]:
        if self.num_proc == 1:
            if self._tokenizer is None:
                from ...tokenizer import build_tokenizer

                self._tokenizer = build_tokenizer(self.config.tokenizer)
            for t in texts:
                yield list(self._tokenizer.encode(t))
            return
        if self._pool is None:
            self._pool = mp.get_context("spawn").Pool(self.num_proc, initializer=_worker_init,
                                                      initargs=(self._tokenizer_cfg(),))
        pending: deque = deque()
        chunk: list[str] = []
        for t in texts:
            chunk.append(t)
            if len(chunk) == CHUNK:
                pending.append(self._pool.apply_async(_worker_encode, (chunk,)))
                chunk = []
                while len(pending) > 2 * self.num_proc:
                    yield from pending.popleft().get()
        if chunk:
            pending.append(self._pool.apply_async(_worker_encode, (chunk,)))
        while pending:
            yield from pending.popleft().get()

    def __iter__(self) -> Iterator[list[int]]:
        try:
            while self.file_idx < len(self.files):
                skip = self.docs_in_file
                for n, toks in enumerate(self._encode_stream(self._texts_of(self.file_idx))):
                    if n < skip:
                        continue
                    self.docs_in_file = n + 1
                    if toks:
                        self.total_docs_yielded += 1
                        yield toks
                self.file_idx += 1
                self.docs_in_file = 0
        finally:
            self.close()

    def close(self) -> None:
        if self._pool is not None:
            self._pool.terminate()
            self._pool.join()
            self._pool = None
