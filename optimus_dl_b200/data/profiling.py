"""Data-pipeline profiler (optimus_dl/modules/data/profiling.py:16-389).

Every node built by a transform is wrapped in a ``ProfilingProxyNode`` when profiling is on. The
profiler keeps, per node, total time inside ``next()`` and *self* time (total minus time spent in
upstream nodes called on the same thread). A node whose upstream runs on another thread
(prefetchers, parallel mappers) is an async boundary: time it spends waiting is reported as
"blocked" rather than "compute". Every ``report_freq`` root batches a table is logged, slowest first.
"""

from __future__ import annotations

import contextvars
import logging
import threading
import time
from contextlib import contextmanager
from typing import Any

from torchdata.nodes import BaseNode

logger = logging.getLogger(__name__)

_current_profiler: contextvars.ContextVar = contextvars.ContextVar("optimus_data_profiler", default=None)
_call_stack = threading.local()


@contextmanager
def scope_profiler(profiler: "PipelineProfiler | None"):
    tok = _current_profiler.set(profiler)
    try:
        yield profiler
    finally:
        _current_profiler.reset(tok)


def current_profiler() -> "PipelineProfiler | None":
    return _current_profiler.get()


class NodeStats:
    __slots__ = ("name", "calls", "total", "self_time", "threads", "parent_threads")

    def __init__(self, name: str):
        self.name, self.calls, self.total, self.self_time = name, 0, 0.0, 0.0
        self.threads: set[int] = set()
        self.parent_threads: set[int] = set()


class NodeSummary:
    """What ``_analyze_bottlenecks`` reports per node: call count, wall time inside ``next()`` and the part of it not
    spent in upstream nodes on the same thread."""
    __slots__ = ("name", "calls", "total_time", "compute_time", "is_async_boundary")

    def __init__(self, name: str, calls: int, total_time: float, compute_time: float, is_async_boundary: bool):
        self.name, self.calls, self.total_time, self.compute_time = name, calls, total_time, compute_time
        self.is_async_boundary = is_async_boundary


class PipelineProfiler:
    def __init__(self, name: str = "pipeline", report_freq: int = 500):
        self.name, self.report_freq = name, max(1, int(report_freq))
        self.stats: dict[int, NodeStats] = {}
        self.root_nodes: list[Any] = []
        self._lock = threading.Lock()
        self._root_batches = 0

    def register(self, node_id: int, name: str) -> NodeStats:
        with self._lock:
            return self.stats.setdefault(node_id, NodeStats(name))

    def record(self, node_id: int, total: float, child: float, is_root: bool, parent_thread: int | None) -> None:
        st = self.stats[node_id]
        with self._lock:
            st.calls += 1
            st.total += total
            st.self_time += max(0.0, total - child)
            st.threads.add(threading.get_ident())
            if parent_thread is not None:
                st.parent_threads.add(parent_thread)
            if is_root:
                self._root_batches += 1
                due = self._root_batches % self.report_freq == 0
            else:
                due = False
        if due:
            self.print_report()

    def is_async_boundary(self, st: NodeStats) -> bool:
        return bool(st.threads and st.parent_threads and not (st.threads & st.parent_threads))

    def report(self) -> str:
        rows = sorted(self.stats.values(), key=lambda s: s.self_time, reverse=True)
        lines = [f"data pipeline '{self.name}' after {self._root_batches} batches:",
                 f"  {'node':<48}{'calls':>10}{'total s':>10}{'self s':>10}{'ms/call':>10}  kind"]
        for s in rows:
            kind = "blocked" if self.is_async_boundary(s) else "compute"
            per = 1e3 * s.self_time / s.calls if s.calls else 0.0
            lines.append(f"  {s.name[:47]:<48}{s.calls:>10}{s.total:>10.2f}{s.self_time:>10.2f}{per:>10.3f}  {kind}")
        if rows:
            lines.append(f"  bottleneck: {rows[0].name}")
        return "\n".join(lines)


    def print_report(self) -> None:
        """Log the report (the periodic summary's entry point)."""
        logger.info("Data Pipeline Profiling Report: %s\n%s", self.name, self.report())

    def _analyze_bottlenecks(self) -> dict[str, "NodeSummary"]:
        """Per-node summary keyed by node name (a second node of the same name gets ``#2``, ...); nodes that were
        never called are left out."""
        out: dict[str, NodeSummary] = {}
        with self._lock:
            rows = list(self.stats.values())
        for st in rows:
            if not st.calls:
                continue
            key, k = st.name, 1
            while key in out:
                k += 1
                key = f"{st.name}#{k}"
            out[key] = NodeSummary(st.name, st.calls, st.total, st.self_time, self.is_async_boundary(st))
        return out

    def pipeline_tree(self) -> str:
        """The chain of nodes below each root, one per line: proxies by the name they were registered under (the
        transform or dataset that built them), the nodes between them by class."""
        lines: list[str] = []

        def walk(node: Any, depth: int) -> None:
            if depth > 64 or node is None:
                return
            if isinstance(node, ProfilingProxyNode):
                lines.append("  " * depth + "[" + " > ".join([*node._enclosing, node._name]) + "]")
                walk(node.node, depth + 1)
                return
            lines.append("  " * depth + type(node).__name__)
            for attr in ("node", "source", "inner", "dataset"):
                child = getattr(node, attr, None)
                if isinstance(child, BaseNode):
                    walk(child, depth + 1)
                    return
            for attr in ("nodes", "source_nodes", "sources"):
                kids = getattr(node, attr, None)
                if isinstance(kids, dict):
                    kids = list(kids.values())
                if isinstance(kids, (list, tuple)) and kids and all(isinstance(c, BaseNode) for c in kids):
                    for c in kids:
                        walk(c, depth + 1)
                    return

        for root in self.root_nodes:
            walk(root, 0)
        return "\n".join(lines)

    def print_pipeline_tree(self) -> None:
        logger.info("Data Pipeline Structure: %s\n%s", self.name, self.pipeline_tree())


class PipelineTracer:
    """``with PipelineTracer(name) as profiler:`` makes ``profiler`` the active one, so transforms built inside the
    block proxy their nodes into it. ``describe`` prints the chain of nodes below one node (debug aid)."""

    def __init__(self, name: str = "pipeline", report_freq: int = 500, profiler: "PipelineProfiler | None" = None):
        self.profiler = profiler if profiler is not None else PipelineProfiler(name, report_freq)
        self._token: Any = None

    def __enter__(self) -> "PipelineProfiler":
        self._token = _current_profiler.set(self.profiler)
        return self.profiler

    def __exit__(self, *exc: Any) -> None:
        _current_profiler.reset(self._token)
        self._token = None

    @staticmethod
    def describe(node: Any, depth: int = 0) -> str:
        out = "  " * depth + repr(type(node).__name__)
        for attr in ("node", "source", "inner"):
            child = getattr(node, attr, None)
            if child is not None:
                out += "\n" + PipelineTracer.describe(child, depth + 1)
                break
        return out


class ProfilingProxyNode(BaseNode):
    def __init__(self, node: BaseNode, name: str, profiler: PipelineProfiler, is_root: bool = False):
        super().__init__()
        self.node, self.name, self.profiler = node, name, profiler
        self._name, self._profiler = name, profiler
        self._enclosing: list[str] = []
        self._creator_thread: int | None = None
        profiler.register(id(self), name)
        self._is_root = False
        if is_root:
            self._is_root = True

    @property
    def _is_root(self) -> bool:
        return self.__dict__.get("_root", False)

    @_is_root.setter
    def _is_root(self, value: bool) -> None:
        """The root is the node whose batches are counted for ``report_freq`` and where the printed tree starts."""
        self.__dict__["_root"] = bool(value)
        roots = self.profiler.root_nodes
        if value and not any(r is self for r in roots):
            roots.append(self)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self.node.reset(initial_state)

    def get_state(self) -> dict[str, Any]:
        return self.node.state_dict()

    def next(self):
        stack = getattr(_call_stack, "frames", None)
        if stack is None:
            stack = _call_stack.frames = []
        parent_thread = stack[-1][1] if stack else self._creator_thread
        frame = [0.0, threading.get_ident()]
        stack.append(frame)
        t0 = time.perf_counter()
        try:
            return next(self.node)
        finally:
            dt = time.perf_counter() - t0
            stack.pop()
            if stack:
                stack[-1][0] += dt
            self.profiler.record(id(self), dt, frame[0], self._is_root, parent_thread)


def maybe_profile(node: BaseNode, name: str) -> BaseNode:
    prof = current_profiler()
    if prof is None:
        return node
    if isinstance(node, ProfilingProxyNode):
        if name != node._name:
            node._enclosing.insert(0, name)      # a transform made of transforms: shown in the tree, timed once
        return node
    return ProfilingProxyNode(node, name, prof)


get_active_profiler = current_profiler   # the reference's name
