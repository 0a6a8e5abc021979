"""Where the documents come from: file discovery and readers
(optimus_dl/recipe/pretokenize/source.py:27-304).

``FileFinder`` lists the files of a dataset and narrows them to the requested split, in this order:
an explicit ``file_pattern``; the ``configs: [{config_name, data_files: [{split, path}]}]`` table in
the YAML front matter of ``README.md``; the conventional ``data/<split>-*``, ``data/<split>_*``,
``data/<split>/*`` layouts. The list is sorted, then shuffled with the processing seed. The
repository can be a Hugging Face dataset id (listed and downloaded through ``huggingface_hub``) or
a local directory with the same layout. ``FileReader`` yields the text column of parquet (row-group
streaming), JSON-lines (optionally gzip-compressed) and plain ``.txt`` (one document per line) files.
"""

from __future__ import annotations

import fnmatch
import gzip
import json
import logging
import os
import random
from pathlib import Path
from typing import Any, Iterator

import yaml

try:  # module-level names so that callers (and tests) can substitute the two hub calls
    from huggingface_hub import hf_hub_download, list_repo_files
except ImportError:  # pragma: no cover - local directories need no hub client
    hf_hub_download = list_repo_files = None

logger = logging.getLogger(__name__)

DATA_SUFFIXES = (".parquet", ".jsonl", ".json", ".jsonl.gz", ".txt")


class _Repo:
    """Uniform view of a dataset repository: a local directory or a hub id."""

    def __init__(self, repo_id: str, cache_dir: str | None):
        self.repo_id, self.cache_dir = repo_id, cache_dir
        self.local = Path(repo_id) if os.path.isdir(repo_id) else None

    def list_files(self) -> list[str]:
        if self.local is not None:
            return sorted(str(p.relative_to(self.local)).replace(os.sep, "/") for p in self.local.rglob("*") if p.is_file())
        if list_repo_files is None:
            raise ImportError(f"{self.repo_id!r} is not a local directory and huggingface_hub is not installed")
        return list(list_repo_files(repo_id=self.repo_id, repo_type="dataset"))

    def fetch(self, name: str) -> Path:
        if self.local is not None:
            return self.local / name
        if hf_hub_download is None:
            raise ImportError(f"{self.repo_id!r} is not a local directory and huggingface_hub is not installed")
        return Path(hf_hub_download(repo_id=self.repo_id, filename=name, repo_type="dataset", cache_dir=self.cache_dir))


class FileFinder:
    def __init__(self, config: Any, seed: int):
        self.config, self.seed = config, int(seed)
        self.repo = _Repo(str(config.repo_id), config.get("cache_dir") if hasattr(config, "get") else config.cache_dir)

    @staticmethod
    def _data_files(names: list[str], pattern: str | None = None) -> list[str]:
        return sorted(n for n in names if n.endswith(DATA_SUFFIXES) and (pattern is None or fnmatch.fnmatch(n, pattern)))

    def _from_readme(self, names: list[str]) -> list[str] | None:
        if "README.md" not in names:
            return None
        try:
            content = self.repo.fetch("README.md").read_text(encoding="utf-8")
        except Exception as err:  # noqa: BLE001
            logger.warning("could not read README.md: %s", err)
            return None
        parts = content.split("---")
        if not content.startswith("---") or len(parts) < 3:
            return None
        try:
            meta = yaml.safe_load(parts[1])
        except yaml.YAMLError as err:
            logger.warning("README.md front matter does not parse: %s", err)
            return None
        if not isinstance(meta, dict) or "configs" not in meta:
            return None
        want = self.config.get("config_name") if hasattr(self.config, "get") else self.config.config_name
        entry = next((c for c in meta["configs"] if c.get("config_name") == want), None)
        if entry is None:
            logger.warning("no config named %r in README.md", want)
            return None
        data_files = entry.get("data_files") or []
        if isinstance(data_files, (str, list)) and data_files and not isinstance(data_files[0], dict):
            data_files = [{"split": "all", "path": p} for p in ([data_files] if isinstance(data_files, str) else data_files)]
        out: list[str] = []
        for item in data_files:
            if item.get("split") in (self.config.split, "all"):
                paths = item["path"] if isinstance(item["path"], list) else [item["path"]]
                for pat in paths:
                    out.extend(fnmatch.filter(names, pat))
        return out

    def get_files(self) -> list[str]:
        names = self.repo.list_files()
        logger.info("%d files in %s before filtering", len(names), self.config.repo_id)
        pattern = self.config.get("file_pattern") if hasattr(self.config, "get") else self.config.file_pattern
        if pattern is not None:
            files = self._data_files(names, pattern)
        else:
            files = self._from_readme(names) or []
            if not files:
                cname = self.config.get("config_name") if hasattr(self.config, "get") else self.config.config_name
                assert cname is None, "config_name is not supported without metadata file"
                split = self.config.split
                patterns = ["data/*"] if not split or split == "all" else [f"data/{split}-*", f"data/{split}_*",
                                                                          f"data/{split}/*"]
                files = [f for p in patterns for f in self._data_files(names, p)]
        if not files:
            logger.warning("no files found for split %r", self.config.split)
            return []
        # order before the shuffle as optimus_dl/recipe/pretokenize/source.py:60-97 leaves it: every pattern's matches
        # sorted, the patterns one after the other
        files = list(dict.fromkeys(files))
        random.Random(self.seed).shuffle(files)
        logger.info("%d files to process", len(files))
        return files


class FileReader:
    def __init__(self, config: Any, dataset_config: Any):
        self.text_column = str(config.text_column)
        self.repo = _Repo(str(dataset_config.repo_id),
                          dataset_config.get("cache_dir") if hasattr(dataset_config, "get") else dataset_config.cache_dir)

    def read_texts(self, file_path: str) -> Iterator[str]:
        local = self.repo.fetch(file_path)
        name = str(local)
        try:
            if name.endswith(".parquet"):
                yield from self._parquet(local)
            elif name.endswith((".jsonl", ".json", ".jsonl.gz")):
                yield from self._jsonl(local)
            elif name.endswith(".txt"):
                with open(local, encoding="utf-8") as f:
                    for line in f:
                        if line.strip():
                            yield line.rstrip("\n")
            else:
                logger.warning("skipping unsupported file %s", file_path)
        except Exception as err:  # noqa: BLE001 - one bad file must not end a multi-hour job
            logger.error("failed to read %s: %s", file_path, err)

    def _parquet(self, path: Path) -> Iterator[str]:
        import pyarrow.parquet as pq

        pf = pq.ParquetFile(path)
        if self.text_column not in pf.schema_arrow.names:
            logger.warning("column %r not in %s (has %s)", self.text_column, path, pf.schema_arrow.names)
            return
        for batch in pf.iter_batches(batch_size=4096, columns=[self.text_column]):
            for text in batch.column(0).to_pylist():
                if text:
                    yield text

    def _jsonl(self, path: Path) -> Iterator[str]:
        opener = gzip.open if str(path).endswith(".gz") else open
        with opener(path, "rt", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                try:
                    text = json.loads(line).get(self.text_column)
                except (json.JSONDecodeError, AttributeError):
                    continue
                if text:
                    yield text
