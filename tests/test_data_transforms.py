"""Datasets and transforms not covered by the pipeline tests: synthetic and loop datasets, tokenising, chunking,
skipping, shuffling, prefetching, composition, and exact state resume of each
(optimus_dl/modules/data/datasets/*.py, optimus_dl/modules/data/transforms/*.py)."""

import numpy as np
import pytest
import torch
import torchdata.nodes as tn

from optimus_dl_b200.data.datasets import build_dataset
from optimus_dl_b200.data.transforms import build_transform


class _Range(tn.BaseNode):
    def __init__(self, n, make=lambda i: {"input_ids": [i]}):
        super().__init__()
        self.n, self.i, self.make = n, 0, make

    def reset(self, initial_state=None):
        super().reset(initial_state)
        self.i = initial_state["i"] if initial_state else 0

    def get_state(self):
        return {"i": self.i}

    def next(self):
        if self.i >= self.n:
            raise StopIteration
        self.i += 1
        return self.make(self.i - 1)


def _drain(node, limit=10_000):
    out = []
    for _ in range(limit):
        try:
            out.append(next(node))
        except StopIteration:
            break
    return out


def _resume_equals_straight(make_node, consume, total):
    """Run ``total`` items straight; run ``consume``, snapshot, rebuild, restore, run the rest: same items."""
    a = make_node()
    a.reset()
    straight = [next(a) for _ in range(total)]
    b = make_node()
    b.reset()
    head = [next(b) for _ in range(consume)]
    state = b.state_dict()
    c = make_node()
    c.reset(state)
    tail = [next(c) for _ in range(total - consume)]
    return straight, head + tail


def _same(a, b):
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, (np.ndarray, torch.Tensor)):
        return np.array_equal(np.asarray(a), np.asarray(b))
    return a == b


def test_synthetic_tokens_is_deterministic_per_rank_and_resumable():
    cfg = {"_name": "synthetic_tokens", "vocab_size": 50, "length": 9, "num_documents": 6, "seed": 3}
    d0 = build_dataset(cfg, rank=0, world_size=2, seed=1)
    d0.reset()
    docs = _drain(d0)
    assert len(docs) == 6 and all(d["input_ids"].shape == (9,) and d["input_ids"].max() < 50 for d in docs)
    again = build_dataset(cfg, rank=0, world_size=2, seed=1)
    again.reset()
    assert _same(docs, _drain(again))
    other = build_dataset(cfg, rank=1, world_size=2, seed=1)
    other.reset()
    assert not _same(docs, _drain(other))               # ranks draw different documents
    straight, resumed = _resume_equals_straight(lambda: build_dataset(cfg, rank=0, world_size=2, seed=1), 4, 6)
    assert _same(straight, resumed)
    lens_cfg = {"_name": "synthetic_tokens", "vocab_size": 50, "mean_length": 40.0, "min_length": 8, "max_length": 64,
                "num_documents": 200}
    d = build_dataset(lens_cfg)
    d.reset()
    lens = [len(x["input_ids"]) for x in _drain(d)]
    assert min(lens) >= 8 and max(lens) <= 64 and len(set(lens)) > 10


def test_loop_restarts_the_inner_dataset_and_counts_epochs():
    cfg = {"_name": "loop", "inner": {"_name": "synthetic_tokens", "vocab_size": 9, "length": 3, "num_documents": 4}}
    d = build_dataset(cfg)
    d.reset()
    items = [next(d) for _ in range(10)]
    assert _same(items[:4], items[4:8]) and _same(items[:2], items[8:10])
    assert d.get_state()["epoch"] == 2
    straight, resumed = _resume_equals_straight(lambda: build_dataset(cfg), 6, 11)
    assert _same(straight, resumed)
    empty = build_dataset({"_name": "loop", "inner": {"_name": "synthetic_tokens", "num_documents": 0}})
    empty.reset()
    with pytest.raises(RuntimeError):
        next(empty)


def test_tokenize_maps_text_and_can_keep_it():
    texts = ["ab", "", "héllo"]
    src = lambda: _Range(3, lambda i: {"text": texts[i], "meta": i})  # noqa: E731
    base = {"_name": "tokenize", "tokenizer_config": {"_name": "char_tokenize"}, "worker_cfg": {"num_workers": 0}}
    node = build_transform(base).build(src())
    node.reset()
    out = _drain(node)
    assert [list(o["input_ids"]) for o in out][0] == [256, 97, 98, 257]        # BOS, bytes, EOS
    assert list(out[1]["input_ids"]) == [256, 257]
    assert len(out[2]["input_ids"]) == 2 + len("héllo".encode())               # UTF-8 bytes, not characters
    assert all("text" not in o and o["meta"] == i for i, o in enumerate(out))
    keep = build_transform({**base, "keep_text": True, "output_field": "ids"}).build(src())
    keep.reset()
    k = next(keep)
    assert k["text"] == "ab" and list(k["ids"]) == [256, 97, 98, 257]


def test_chunk_tokens_splits_long_documents_with_shift_overlap_budget():
    docs = [{"input_ids": list(range(10))}, {"input_ids": list(range(100, 103))}]
    node = build_transform({"_name": "chunk_tokens", "max_seq_len": 4}).build(_Range(2, lambda i: docs[i]))
    node.reset()
    chunks = [list(c["input_ids"]) for c in _drain(node)]
    assert chunks == [[0, 1, 2, 3, 4], [5, 6, 7, 8, 9], [100, 101, 102]]        # max_seq_len + 1 tokens for the shift
    node = build_transform({"_name": "chunk_tokens", "max_seq_len": 4, "add_one_for_shift": False, "max_chunks": 2}).build(
        _Range(2, lambda i: docs[i]))
    node.reset()
    chunks = [list(c["input_ids"]) for c in _drain(node)]
    assert chunks == [[0, 1, 2, 3], [4, 5, 6, 7], [100, 101, 102]]              # at most two chunks per document
    make = lambda: build_transform({"_name": "chunk_tokens", "max_seq_len": 3}).build(  # noqa: E731
        _Range(5, lambda i: {"input_ids": list(range(10 * i, 10 * i + 9))}))
    straight, resumed = _resume_equals_straight(make, 4, 11)                    # snapshot in the middle of a document
    assert _same(straight, resumed)


def test_skip_transforms_partition_the_stream():
    keep0 = build_transform({"_name": "skip_interleaved", "keep_every": 3, "offset": 0}).build(_Range(10))
    keep1 = build_transform({"_name": "skip_interleaved", "keep_every": 3, "offset": 1}).build(_Range(10))
    keep0.reset(), keep1.reset()
    assert [x["input_ids"][0] for x in _drain(keep0)] == [0, 3, 6, 9]
    assert [x["input_ids"][0] for x in _drain(keep1)] == [1, 4, 7]
    a = build_transform({"_name": "skip_random", "keep_probability": 0.3, "seed": 5}).build(_Range(200))
    b = build_transform({"_name": "skip_random", "keep_probability": 0.3, "seed": 5, "invert": True}).build(_Range(200))
    a.reset(), b.reset()
    ka, kb = [x["input_ids"][0] for x in _drain(a)], [x["input_ids"][0] for x in _drain(b)]
    assert sorted(ka + kb) == list(range(200)) and not set(ka) & set(kb)        # a train / held-out split
    assert 30 < len(ka) < 90
    make = lambda: build_transform({"_name": "skip_random", "keep_probability": 0.5, "seed": 1}).build(_Range(100))  # noqa: E731
    straight, resumed = _resume_equals_straight(make, 7, 30)
    assert _same(straight, resumed)


def test_shuffle_is_a_seeded_permutation_within_the_buffer_and_resumes_exactly():
    make = lambda seed=0: build_transform({"_name": "shuffle", "buffer_size": 8}, seed=seed).build(_Range(40))  # noqa: E731
    n = make()
    n.reset()
    out = [x["input_ids"][0] for x in _drain(n)]
    assert sorted(out) == list(range(40)) and out != list(range(40))
    assert all(abs(v - i) < 40 for i, v in enumerate(out)) and max(out[:8]) < 16   # early items come from the first buffers
    n2 = make()
    n2.reset()
    assert [x["input_ids"][0] for x in _drain(n2)] == out                          # same seed, same order
    straight, resumed = _resume_equals_straight(make, 13, 40)
    assert _same(straight, resumed)


def test_prefetch_and_composition_preserve_order_and_state():
    cfg = {"_name": "compose", "transforms": [
        {"_name": "chunk_tokens", "max_seq_len": 2, "add_one_for_shift": False},
        {"_name": "skip_interleaved", "keep_every": 2, "offset": 1},
        {"_name": "prefetch", "prefetch_factor": 2},
    ]}
    src = lambda: _Range(6, lambda i: {"input_ids": [10 * i, 10 * i + 1, 10 * i + 2, 10 * i + 3]})  # noqa: E731
    node = build_transform(cfg).build(src())
    node.reset()
    got = [list(x["input_ids"]) for x in _drain(node)]
    assert got == [[10 * i + 2, 10 * i + 3] for i in range(6)]                   # second chunk of every document
    straight, resumed = _resume_equals_straight(lambda: build_transform(cfg).build(src()), 2, 6)
    assert _same(straight, resumed)
    assert build_transform({"_name": "compose", "transforms": []}).build(src()) is not None


def test_to_device_converts_arrays_and_leaves_scalars():
    item = {"input_ids": np.arange(6).reshape(2, 3), "seq_lens": [3, 2], "max_seqlen": 3, "name": "x"}
    node = build_transform({"_name": "to_device"}, device=torch.device("cpu")).build(_Range(1, lambda i: item))
    node.reset()
    out = next(node)
    assert isinstance(out["input_ids"], torch.Tensor) and out["input_ids"].dtype == torch.int64
    assert out["max_seqlen"] == 3 and out["name"] == "x"


def test_reference_spellings_of_transform_and_dataset_options(tmp_path, caplog):
    import logging

    node = build_transform({"_name": "skip_interleaved", "skip_count": 2}).build(_Range(10))
    node.reset()
    assert [x["input_ids"][0] for x in _drain(node)] == [0, 3, 6, 9]          # first item, then two dropped each time
    a = build_transform({"_name": "skip_random", "probability": 0.25, "seed": 3}).build(_Range(400))
    a.reset()
    kept = len(_drain(a))
    assert 260 < kept < 340                                                     # an item is dropped with probability 0.25
    for cfg in ({"_name": "prefetch", "prefetch_factor": 2, "snapshot_frequency": 4},
                {"_name": "to_device", "pin_prefetch_factor": 1, "pin_snapshot_frequency": 8, "properties": ["input_ids"]}):
        n = build_transform(cfg, device=torch.device("cpu")).build(_Range(3, lambda i: {"input_ids": np.arange(3), "other": np.arange(2)}))
        n.reset()
        out = _drain(n)
        assert len(out) == 3
    assert isinstance(out[0]["input_ids"], torch.Tensor) and isinstance(out[0]["other"], np.ndarray)   # only listed keys move
    with caplog.at_level(logging.INFO):
        tok = build_transform({"_name": "tokenize", "tokenizer_config": {"_name": "char_tokenize"}, "debug_samples": 1,
                               "worker_cfg": {"num_workers": 0}}).build(_Range(3, lambda i: {"text": "ab"}))
        tok.reset()
        _drain(tok)
    assert caplog.text.count("tokenize sample") == 1
    raw = tmp_path / "tokens.bin"
    np.concatenate([np.zeros(4, np.uint16), np.arange(40, dtype=np.uint16)]).tofile(raw)
    flat = build_dataset({"_name": "tokenized_flat", "files": [str(raw)], "dtype": "np.uint16", "seq_len": 4, "batch_size": 2,
                          "offset": 8})
    flat.reset()
    first = next(flat)
    assert np.asarray(first["input_ids"])[0, 0] == 0 and np.asarray(first["input_ids"]).shape[0] == 2


def test_pipeline_profiler_attributes_time_to_the_slow_stage():
    import time

    from optimus_dl_b200.data import build_data_pipeline
    from optimus_dl_b200.data.profiling import PipelineProfiler, ProfilingProxyNode, get_active_profiler, scope_profiler

    class _Slow(tn.BaseNode):
        def __init__(self, node, delay):
            super().__init__()
            self.node, self.delay = node, delay

        def reset(self, initial_state=None):
            super().reset(initial_state)
            self.node.reset(initial_state)

        def get_state(self):
            return self.node.state_dict()

        def next(self):
            item = next(self.node)
            time.sleep(self.delay)
            return item

    prof = PipelineProfiler("t", report_freq=1000)
    assert get_active_profiler() is None
    with scope_profiler(prof):
        assert get_active_profiler() is prof
    src = ProfilingProxyNode(_Range(5), "source", prof)
    slow = ProfilingProxyNode(_Slow(src, 0.01), "slow_stage", prof)
    top = ProfilingProxyNode(_Slow(slow, 0.0), "top", prof)
    top.reset()
    assert len(_drain(top)) == 5
    by_name = {s.name: s for s in prof.stats.values()}
    assert by_name["slow_stage"].calls >= 5 and by_name["top"].total >= by_name["slow_stage"].total >= by_name["source"].total
    assert by_name["slow_stage"].self_time > 5 * 0.008 and by_name["top"].self_time < by_name["slow_stage"].self_time
    report = prof.report()
    assert "bottleneck: slow_stage" in report and "source" in report
    state = top.state_dict()
    top.reset(state)                                    # the proxies are transparent for state
    # the builder attaches a profiler when the config asks for one
    cfg = {"source": {"_name": "synthetic_tokens", "vocab_size": 11, "length": 5, "num_documents": 8},
           "transform": {"_name": "basic_batcher", "batch_size": 2, "pad_token_id": 0}, "profile": True, "report_freq": 2}
    pipe = build_data_pipeline(cfg, profile_name="train")
    loader = pipe.dataloader if hasattr(pipe, "dataloader") else pipe
    it = iter(loader)
    assert np.asarray(next(it)["input_ids"]).shape[0] == 2


def test_tokenized_flat_streams_files_as_one_sequence_with_equal_spans_per_rank(tmp_path):
    a, b = tmp_path / "a.bin", tmp_path / "b.npy"
    np.arange(0, 50, dtype=np.uint16).tofile(a)
    np.save(b, np.arange(50, 120, dtype=np.uint16))
    cfg = {"_name": "tokenized_flat", "files": [str(a), str(b)], "dtype": "uint16", "batch_size": 2, "seq_len": 8,
           "add_one_for_shift": True}
    whole = build_dataset(cfg)
    whole.reset()
    batches = _drain(whole)
    first = np.asarray(batches[0]["input_ids"])
    assert first.shape == (2, 9)                                  # one extra token per row for the shifted targets
    assert first[0].tolist() == list(range(0, 9)) and first[1].tolist() == list(range(8, 17))
    flat = np.concatenate([np.asarray(x["input_ids"])[:, :8].reshape(-1) for x in batches])
    assert flat.tolist() == list(range(len(flat))) and len(flat) >= 96   # crosses the file boundary without a seam
    halves = []
    for rank in (0, 1):
        d = build_dataset(cfg, rank=rank, world_size=2)
        d.reset()
        halves.append([np.asarray(x["input_ids"])[:, :8].reshape(-1) for x in _drain(d)])
    starts = [h[0][0] for h in halves]
    assert starts == [0, 60] and len(halves[0]) == len(halves[1])   # ranks read disjoint, equally long spans
    straight, resumed = _resume_equals_straight(lambda: build_dataset(cfg), 2, 5)
    assert _same(straight, resumed)
    # the reference's form (the default): (batch, seq_len) blocks in the files' dtype; 5 ranks over 104 tokens read
    # 20 tokens each, and together exactly the first 100 (optimus_dl tests/data/test_tokenized_flat_dataset.py)
    ref_cfg = {k: v for k, v in cfg.items() if k != "add_one_for_shift"}
    no_shift = build_dataset(ref_cfg)
    no_shift.reset()
    blk = np.asarray(next(no_shift)["input_ids"])
    assert blk.shape == (2, 8) and blk.dtype == np.uint16
    assert set(no_shift.state_dict()) >= {"files", "index", "limit", "seq_len", "batch_size", "rank", "world_size"}
    c, d2 = tmp_path / "c.u8", tmp_path / "d.u8"
    np.arange(0, 77, dtype=np.uint8).tofile(c)
    np.arange(77, 104, dtype=np.uint8).tofile(d2)
    got = []
    for rank in range(5):
        ds5 = build_dataset({"_name": "tokenized_flat", "files": [str(c), str(d2)], "dtype": "np.uint8", "batch_size": 1,
                             "seq_len": 5}, rank=rank, world_size=5)
        ds5.reset()
        got += [np.asarray(x["input_ids"]).reshape(-1) for x in _drain(ds5)]
    assert np.concatenate(got).tolist() == list(range(100))
    glob_cfg = {**cfg, "files": str(tmp_path / "*.bin")}
    g = build_dataset(glob_cfg)
    g.reset()
    assert np.asarray(next(g)["input_ids"])[0, 0] == 0


def test_tokenize_single_item_call_and_batcher_state_carries_its_config():
    """``TokenizeTransform._map`` (optimus_dl/modules/data/transforms/tokenize.py) and the ``cfg`` entry of the batcher
    states (optimus_dl/modules/data/transforms/basic_batcher.py:71-79, flat_tokens_batcher.py:109-121)."""
    from optimus_dl_b200.data.transforms.basic_batcher import BasicBatcherConfig, BasicBatcherNode
    from optimus_dl_b200.data.transforms.flat_tokens_batcher import FlatTokensBatcherConfig, FlatTokensBatcherNode
    from optimus_dl_b200.data.transforms.tokenize import TokenizeTransform, TokenizeTransformConfig
    from optimus_dl_b200.tokenizer.implementations.char import CharTokenizerConfig

    plain = TokenizeTransform(TokenizeTransformConfig(tokenizer_config=CharTokenizerConfig(_name="char_tokenize", add_bos=False, add_eos=False)))
    assert plain._map({"text": "abc"})["input_ids"] == [97, 98, 99]
    marked = TokenizeTransform(TokenizeTransformConfig(tokenizer_config=CharTokenizerConfig(_name="char_tokenize")))
    assert marked._map({"text": "€"})["input_ids"] == [256, 226, 130, 172, 257]        # UTF-8 bytes between BOS and EOS

    docs = [{"input_ids": [1]}, {"input_ids": [2]}, {"input_ids": [3]}]
    cfg = BasicBatcherConfig(batch_size=1, pad_token_id=0)
    node = BasicBatcherNode(tn.IterableWrapper(docs), cfg)
    node.reset()
    node.next()
    state = node.get_state()
    assert state["cfg"] == cfg and "source_state" in state
    again = BasicBatcherNode(tn.IterableWrapper(docs), cfg)
    again.reset(state)
    np.testing.assert_array_equal(again.next()["input_ids"], np.array([[2]]))
    fcfg = FlatTokensBatcherConfig(batch_size=1, seq_len=4)
    flat = FlatTokensBatcherNode(tn.IterableWrapper([{"input_ids": np.arange(50)}]), fcfg)
    flat.reset()
    flat.next()
    assert flat.get_state()["cfg"] == fcfg


def _drain(node):
    out = []
    try:
        while True:
            out.append(next(node))
    except StopIteration:
        return out


def test_skip_nodes_take_their_config_and_resume_from_their_counters():
    """Call forms and state keys of optimus_dl/modules/data/transforms/skip.py (node(source, cfg), ``counter``, ``seed``)."""
    from optimus_dl_b200.data.transforms.skip import (SkipInterleavedTransform, SkipInterleavedTransformConfig,
                                                     SkipInterleavedTransformNode, SkipRandomTransform,
                                                     SkipRandomTransformConfig, SkipRandomTransformNode)

    src = lambda n: tn.IterableWrapper(list(range(n)))  # noqa: E731
    one = SkipInterleavedTransformNode(src(10), SkipInterleavedTransformConfig(skip_count=1))
    one.reset()
    assert _drain(one) == [0, 2, 4, 6, 8]
    two = SkipInterleavedTransformNode(src(10), SkipInterleavedTransformConfig(skip_count=2))
    two.reset()
    assert _drain(two) == [0, 3, 6, 9]
    cfg = SkipInterleavedTransformConfig(skip_count=1)
    first = SkipInterleavedTransformNode(src(10), cfg)
    first.reset()
    assert [next(first), next(first)] == [0, 2]
    state = first.get_state()
    assert state["counter"] == 3 and first.counter == 3
    second = SkipInterleavedTransformNode(src(10), cfg)
    second.reset(state)
    assert second.counter == 3 and [next(second), next(second)] == [4, 6]
    source = src(10)
    built = SkipInterleavedTransform(cfg).build(source)
    assert isinstance(built, SkipInterleavedTransformNode) and built.cfg == cfg

    half = SkipRandomTransformConfig(probability=0.5)
    a = SkipRandomTransformNode(src(100), half, seed=42)
    b = SkipRandomTransformNode(src(100), half, seed=42)
    a.reset(), b.reset()
    kept = _drain(a)
    assert kept == _drain(b) and 0 < len(kept) < 100
    part = SkipRandomTransformNode(src(100), half, seed=42)
    part.reset()
    head = [next(part) for _ in range(10)]
    state = part.get_state()
    rest = _drain(part)
    resumed = SkipRandomTransformNode(src(100), half, seed=42)
    resumed.reset(state)
    assert _drain(resumed) == rest and head + rest == kept
    none = SkipRandomTransformNode(src(10), SkipRandomTransformConfig(probability=0.0), seed=42)
    every = SkipRandomTransformNode(src(10), SkipRandomTransformConfig(probability=1.0), seed=42)
    none.reset(), every.reset()
    assert _drain(none) == list(range(10)) and _drain(every) == []
    node = SkipRandomTransform(half, seed=42).build(src(10))
    assert isinstance(node, SkipRandomTransformNode) and node.cfg == half and node.seed == 42


def test_to_device_single_sample_call_touches_only_the_listed_properties():
    """``ToDeviceTransform._map`` and ``properties`` (optimus_dl/modules/data/transforms/to_device.py:21-119)."""
    from optimus_dl_b200.data.transforms.to_device import ToDeviceTransform, ToDeviceTransformConfig

    cpu = torch.device("cpu")
    t = ToDeviceTransform(ToDeviceTransformConfig(pin_memory=False), cpu)
    t.properties = ["input_ids"]
    out = t._map({"input_ids": torch.tensor([1, 2, 3]), "other": "string"})
    assert out["input_ids"].device == cpu and out["other"] == "string"
    listed = ToDeviceTransform(ToDeviceTransformConfig(properties=["a"]), cpu)._map({"a": [1, 2, 3], "b": [4, 5, 6]})
    assert torch.is_tensor(listed["a"]) and listed["a"].tolist() == [1, 2, 3] and listed["b"] == [4, 5, 6]
    every = ToDeviceTransform(ToDeviceTransformConfig(), cpu)._map({"x": np.arange(3), "n": 5})
    assert torch.is_tensor(every["x"]) and every["n"] == 5


def test_profiler_tracer_scope_summaries_tree_and_periodic_report():
    """Surface of optimus_dl/modules/data/profiling.py:16-389: the tracer scope, per-node summaries, the printed tree
    and the report every ``report_freq`` root batches."""
    import io
    import logging
    import time

    from optimus_dl_b200.data import build_data_pipeline
    from optimus_dl_b200.data.profiling import PipelineProfiler, PipelineTracer, ProfilingProxyNode, get_active_profiler

    class Slow(tn.BaseNode):
        def __init__(self, delay):
            super().__init__()
            self.delay, self.n = delay, 0

        def next(self):
            time.sleep(self.delay)
            self.n += 1
            return self.n

        def reset(self, state=None):
            super().reset(state)
            self.n = 0

    class Above(tn.BaseNode):
        def __init__(self, inner, delay):
            super().__init__()
            self.inner, self.delay = inner, delay

        def next(self):
            item = next(self.inner)
            time.sleep(self.delay)
            return item

        def reset(self, state=None):
            super().reset(state)

    assert get_active_profiler() is None
    with PipelineTracer() as scoped:
        assert get_active_profiler() is scoped
    assert get_active_profiler() is None

    prof = PipelineProfiler("nested")
    child = ProfilingProxyNode(Slow(0.03), name="Child", profiler=prof)
    assert "Child" not in prof._analyze_bottlenecks()                    # never called: not listed
    parent = ProfilingProxyNode(Above(child, 0.06), name="Parent", profiler=prof)
    assert next(parent) == 1
    stats = prof._analyze_bottlenecks()
    assert stats["Child"].calls == 1 and stats["Child"].total_time >= 0.027
    assert stats["Parent"].total_time >= 0.08 and abs(stats["Parent"].compute_time - 0.06) < 0.03   # self time excludes the child

    p1, p2 = PipelineProfiler("p1"), PipelineProfiler("p2")               # two profilers do not share counters
    n1, n2 = ProfilingProxyNode(Slow(0), name="Node", profiler=p1), ProfilingProxyNode(Slow(0), name="Node", profiler=p2)
    next(n1), next(n2), next(n2)
    assert p1._analyze_bottlenecks()["Node"].calls == 1 and p2._analyze_bottlenecks()["Node"].calls == 2

    stream = io.StringIO()
    handler = logging.StreamHandler(stream)
    log = logging.getLogger("optimus_dl_b200.data.profiling")
    old_level = log.level
    log.addHandler(handler), log.setLevel(logging.INFO)
    try:
        every2 = PipelineProfiler("freq", report_freq=2)
        root = ProfilingProxyNode(Slow(0), name="FreqNode", profiler=every2, is_root=True)
        next(root)
        assert "Data Pipeline Profiling Report" not in stream.getvalue()
        next(root)
        assert "Data Pipeline Profiling Report: freq" in stream.getvalue() and "FreqNode" in stream.getvalue()
        pipe = build_data_pipeline({"source": {"_name": "synthetic_tokens", "vocab_size": 11, "length": 4, "num_documents": 8},
                                    "transform": {"_name": "compose", "transforms": [{"_name": "prefetch", "prefetch_factor": 2}]},
                                    "profile": True, "report_freq": 10}, profile_name="tree", rank=0, world_size=1, seed=1)
        assert isinstance(pipe.dataloader, ProfilingProxyNode)
        pipe.dataloader._profiler.print_pipeline_tree()
        text = stream.getvalue()
        for word in ("Data Pipeline Structure: tree", "CompositeTransform", "Prefetcher", "SyntheticTokens"):
            assert word in text, word
    finally:
        log.removeHandler(handler), log.setLevel(old_level)


def test_node_states_use_the_reference_keys_and_the_shuffle_stream_is_the_reference_stream(tmp_path):
    """Checkpointed state of the data nodes is interchangeable with the reference's: same keys, same meaning
    (optimus_dl/modules/data/transforms/shuffle.py:74-98, chunk_tokens.py:56-84, flat_tokens_batcher.py:109-121,
    skip.py:118-123, datasets/txt_lines.py:115-168, loop_dataset.py:87-95). The shuffle buffer draws with numpy's
    ``default_rng(seed + 41 * rank).integers(0, len(buffer))`` and pops that element."""
    sh = build_transform({"_name": "shuffle", "buffer_size": 4}, rank=2, seed=9).build(_Range(10))
    sh.reset()
    got = [x["input_ids"][0] for x in _drain(sh)]
    rng, buf, src, want = np.random.default_rng(9 + 2 * 41), [], list(range(10)), []
    while True:
        while src and len(buf) < 4:
            buf.append(src.pop(0))
        if not buf:
            break
        want.append(buf.pop(int(rng.integers(0, len(buf)))))
    assert got == want and sorted(got) == list(range(10))
    sh.reset()
    next(sh)
    st = sh.state_dict()
    assert set(st) >= {"buffer", "cfg", "source_state", "rng_state", "terminated", "rank"} and st["rank"] == 2
    assert st["rng_state"]["bit_generator"] == "PCG64" and st["terminated"] is False and len(st["buffer"]) == 3

    ch = build_transform({"_name": "chunk_tokens", "max_seq_len": 3, "add_one_for_shift": False}).build(
        _Range(2, lambda i: {"input_ids": list(range(10 * i, 10 * i + 8)), "tag": i}))
    ch.reset()
    assert next(ch) == {"input_ids": [0, 1, 2], "tag": 0}
    st = ch.state_dict()
    assert st["buffer"] == [3, 4, 5, 6, 7] and st["rest"] == {"tag": 0} and "cfg" in st and "source_state" in st

    fb = build_transform({"_name": "flat_batcher", "batch_size": 1, "seq_len": 4, "mask_documents": True}).build(
        _Range(3, lambda i: {"input_ids": list(range(10 * i, 10 * i + 4))}))
    fb.reset()
    next(fb)
    st = fb.state_dict()
    assert st["input_buffer"] == [11, 12] and st["label_buffer"] == [12, 13] and st["position_ids_buffer"] == [1, 2]
    assert st["document_ids_buffer"] == [1, 1] and st["_current_doc_id"] == 2 and "cfg" in st
    fb2 = build_transform({"_name": "flat_batcher", "batch_size": 1, "seq_len": 4, "mask_documents": True}).build(
        _Range(3, lambda i: {"input_ids": list(range(10 * i, 10 * i + 4))}))
    fb2.reset(st)
    assert next(fb2)["input_ids"].tolist() == next(fb)["input_ids"].tolist() == [[11, 12, 20, 21]]

    sr = build_transform({"_name": "skip_random", "probability": 0.5}, seed=3).build(_Range(20))
    sr.reset()
    next(sr)
    assert set(sr.state_dict()) == {"rng_state", "source_state"}

    f = tmp_path / "t.txt"
    f.write_text("".join(f"line {i}\n" for i in range(11)))
    parts = [build_dataset({"_name": "txt_lines", "file_link": str(f)}, rank=r, world_size=3) for r in range(3)]
    for p in parts:
        p.reset()
    assert [[x["text"] for x in _drain(p)] for p in parts] == [[f"line {i}" for i in range(a, a + 3)] for a in (0, 3, 6)]
    parts[1].reset()
    next(parts[1])
    st = parts[1].state_dict()
    assert st == {"index": 4, "file_link": str(f), "skip_empty_lines": st["skip_empty_lines"], "rank": 1, "world_size": 3}
    parts[1].reset(st)
    assert next(parts[1])["text"] == "line 4"                       # ``index`` is a position in the whole file
    lp = build_dataset({"_name": "loop", "inner": {"_name": "txt_lines", "file_link": str(f)}}, rank=0, world_size=3)
    lp.reset()
    assert [next(lp)["text"] for _ in range(4)] == ["line 0", "line 1", "line 2", "line 0"]
    assert set(lp.state_dict()) == {"rank", "world_size", "epoch", "inner_state"}


def test_to_device_cuda_chain_order_and_state_nesting(monkeypatch):
    """On a CUDA device the chain is conversion (no state level of its own) -> ``PinMemory`` -> ``Mapper`` (copy) ->
    ``Prefetcher``, with the configured snapshot frequency and prefetch depth
    (optimus_dl/modules/data/transforms/to_device.py:92-119). Built here with stand-ins for the two nodes that need a
    GPU; the copy itself is replaced by an identity."""
    import optimus_dl_b200.data.transforms.to_device as td

    calls = []

    class Pass(tn.BaseNode):
        def __init__(self, source, **kw):
            super().__init__()
            self.source, self.kw = source, kw
            calls.append((type(self).__name__, kw))

        def reset(self, initial_state=None):
            super().reset(initial_state)
            self.source.reset(initial_state["source"] if initial_state else None)

        def get_state(self):
            return {"source": self.source.state_dict()}

        def next(self):
            return next(self.source)

    class FakePin(Pass):
        pass

    class FakePrefetch(Pass):
        pass

    monkeypatch.setattr(td, "PinMemory", FakePin)
    monkeypatch.setattr(td, "Prefetcher", FakePrefetch)
    monkeypatch.setattr(td._Mover, "__call__", lambda self, b: b)
    t = build_transform({"_name": "to_device", "pin_prefetch_factor": 3, "pin_snapshot_frequency": 77}, device=torch.device("cuda", 0))
    node = t.build(_Range(5, lambda i: {"input_ids": np.array([i, i + 1], dtype=np.uint16), "n": i}))
    assert [c[0] for c in calls] == ["FakePin", "FakePrefetch"]
    assert calls[0][1] == {"pin_memory_device": "cuda", "snapshot_frequency": 77}
    assert calls[1][1] == {"prefetch_factor": 3, "snapshot_frequency": 77}
    node.reset()
    first = next(node)
    assert first["input_ids"].dtype == torch.int64 and first["input_ids"].tolist() == [0, 1] and first["n"] == 0
    st = node.state_dict()
    # prefetch -> mapper -> pin -> (conversion: transparent) -> source
    assert st == {"source": {"it_state": {"source": {"source": {"i": 1}}}}}
    node.reset(st)
    assert next(node)["input_ids"].tolist() == [1, 2]
