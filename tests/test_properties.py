"""Property-based checks (hypothesis): invariants that must hold for ANY input of the stated shape, not only for
the hand-picked cases of the other files. Each property names the rule of the reference it restates."""

import json
import math
import tempfile
from pathlib import Path

import numpy as np
import torch
import torchdata.nodes as tn
from hypothesis import HealthCheck, given, settings, strategies as st

from optimus_dl_b200.core import conf
from optimus_dl_b200.data.datasets import build_dataset
from optimus_dl_b200.data.transforms import build_transform
from optimus_dl_b200.metrics import common as mc
from optimus_dl_b200.ops.attention import build_doc_start, mask_from_doc_start

FAST = settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])


class _Docs(tn.BaseNode):
    def __init__(self, docs):
        super().__init__()
        self.docs, self.i = docs, 0

    def reset(self, initial_state=None):
        super().reset(initial_state)
        self.i = initial_state["i"] if initial_state else 0

    def get_state(self):
        return {"i": self.i}

    def next(self):
        if self.i >= len(self.docs):
            raise StopIteration
        self.i += 1
        return {"input_ids": list(self.docs[self.i - 1])}


def _drain(node):
    out = []
    while True:
        try:
            out.append(next(node))
        except StopIteration:
            return out


def _numbered(lens):
    docs, c = [], 0
    for n in lens:
        docs.append(list(range(c, c + n)))
        c += n
    return docs


doc_lens = st.lists(st.integers(1, 40), min_size=1, max_size=12)


@FAST
@given(lens=doc_lens, width=st.integers(1, 16), shift=st.booleans())
def test_chunking_loses_and_reorders_nothing(lens, width, shift):
    """``chunk_tokens``: the chunks of a document, concatenated, are the document; no chunk is longer than
    ``max_seq_len`` (+1 with the shift token) and only the last chunk of a document may be shorter
    (optimus_dl/modules/data/transforms/chunk_tokens.py)."""
    docs = _numbered(lens)
    node = build_transform({"_name": "chunk_tokens", "max_seq_len": width, "add_one_for_shift": shift}).build(_Docs(docs))
    node.reset()
    chunks = [list(c["input_ids"]) for c in _drain(node)]
    cap = width + (1 if shift else 0)
    assert [t for c in chunks for t in c] == [t for d in docs for t in d]
    assert all(1 <= len(c) <= cap for c in chunks)
    for a, b in zip(chunks, chunks[1:]):
        if len(a) < cap:                      # a short chunk ends its document: the next one starts a new document
            assert any(b[0] == d[0] for d in docs)


@FAST
@given(lens=doc_lens, batch=st.integers(1, 3), seq=st.integers(2, 12))
def test_flat_batches_are_the_token_stream_cut_into_rows(lens, batch, seq):
    """``flat_batcher``: every document gives ``tokens[:-1]`` as inputs and ``tokens[1:]`` as labels (a label never
    crosses into the next document, a one-token document gives nothing); the two streams are cut into rows of
    ``seq_len``; positions restart and document ids step by one at every document start; only an incomplete last
    batch is dropped (optimus_dl/modules/data/transforms/flat_tokens_batcher.py)."""
    docs = _numbered(lens)
    node = build_transform({"_name": "flat_batcher", "batch_size": batch, "seq_len": seq, "mask_documents": True}).build(_Docs(docs))
    node.reset()
    inputs = [t for d in docs for t in d[:-1]]
    labels = [t for d in docs for t in d[1:]]
    starts = {d[0] for d in docs if len(d) > 1}
    used = 0
    for b in _drain(node):
        assert b["input_ids"].shape == b["labels"].shape == (batch, seq)
        flat_in, flat_lab = b["input_ids"].reshape(-1).tolist(), b["labels"].reshape(-1).tolist()
        n = batch * seq
        assert flat_in == inputs[used:used + n] and flat_lab == labels[used:used + n]
        assert all(y == x + 1 for x, y in zip(flat_in, flat_lab))
        pos, did = b["position_ids"].reshape(-1).tolist(), b["document_ids"].reshape(-1).tolist()
        assert did[0] == 0
        for j in range(1, n):
            if flat_in[j] in starts:
                assert pos[j] == 0 and did[j] == did[j - 1] + 1
            else:
                assert pos[j] == pos[j - 1] + 1 and did[j] == did[j - 1]
        used += n
    assert len(inputs) - used < batch * seq


@FAST
@given(shards=st.lists(st.lists(st.integers(1, 30), min_size=1, max_size=5), min_size=1, max_size=4),
       world=st.integers(1, 4), shuffle=st.booleans(), seed=st.integers(0, 5))
def test_document_strategy_visits_every_token_once_over_all_ranks(shards, world, shuffle, seed):
    """``tokenized_dataset`` with the ``document`` strategy: the ranks' documents partition the corpus, whatever the
    shard layout, world size, shuffling and seed (optimus_dl/modules/data/datasets/strategies/document.py)."""
    with tempfile.TemporaryDirectory() as d:
        root, files, c = Path(d), [], 0
        for i, lens in enumerate(shards):
            np.save(root / f"s_{i:010d}.npy", np.arange(c, c + sum(lens), dtype=np.uint16))
            np.save(root / f"s_{i:010d}_lens.npy", np.array(lens, dtype=np.int64))
            files.append({"file": f"s_{i:010d}.npy", "lens_file": f"s_{i:010d}_lens.npy"})
            c += sum(lens)
        (root / "index.json").write_text(json.dumps({"files": files}))
        seen, n_docs = [], 0
        for rank in range(world):
            ds = build_dataset({"_name": "tokenized_dataset", "data_dir": str(root),
                                "strategy": {"_name": "document", "shuffle": shuffle}}, rank=rank, world_size=world, seed=seed)
            ds.reset()
            for item in _drain(ds):
                toks = item["input_ids"].tolist()
                assert toks == list(range(toks[0], toks[0] + len(toks)))          # a document arrives whole and in order
                seen.extend(toks)
                n_docs += 1
        assert sorted(seen) == list(range(c)) and n_docs == sum(len(s) for s in shards)


values = st.lists(st.tuples(st.floats(-100, 100, allow_nan=False), st.floats(0.1, 50)), min_size=1, max_size=30)


@FAST
@given(data=values, cut=st.integers(0, 30))
def test_meters_merged_over_any_split_equal_one_meter_over_everything(data, cut):
    """Aggregation across ranks (``merge`` of meter states) gives what one process that saw all the values would
    report, for every meter kind (optimus_dl/modules/metrics/common.py)."""
    cut = min(cut, len(data))
    kinds = [(mc.AverageMeter, True), (mc.SummedMeter, False), (mc.MaxMeter, False), (mc.MinMeter, False),
             (mc.AveragedExponentMeter, True)]
    for cls, weighted in kinds:
        whole, left, right = cls(), cls(), cls()
        scale = 0.01 if cls is mc.AveragedExponentMeter else 1.0       # keep exp() in range
        for i, (v, w) in enumerate(data):
            args = (v * scale, w) if weighted else (v * scale,)
            whole.log(*args)
            (left if i < cut else right).log(*args)
        left.merge(right.state_dict())
        a, b = whole.compute(), left.compute()
        assert (a is None and b is None) or math.isclose(a, b, rel_tol=1e-9, abs_tol=1e-9), (cls.__name__, a, b)
        clone = cls.from_state_dict(whole.state_dict())
        c = clone.compute()
        assert (a is None and c is None) or math.isclose(a, c, rel_tol=1e-12, abs_tol=1e-12)


leaf = st.one_of(st.integers(-5, 5), st.booleans(), st.none(), st.floats(-2, 2, allow_nan=False),
                 st.text(alphabet="abcxyz_", min_size=0, max_size=5))
keys = st.text(alphabet="abcdefg", min_size=1, max_size=3)
trees = st.recursive(leaf, lambda kids: st.one_of(st.lists(kids, max_size=3), st.dictionaries(keys, kids, max_size=3)),
                     max_leaves=12)


@FAST
@given(tree=st.dictionaries(keys, trees, max_size=4), other=st.dictionaries(keys, trees, max_size=4))
def test_config_container_round_trips_and_merges_like_nested_dicts(tree, other):
    """``create`` / ``to_container`` are inverse on plain data, YAML text round-trips, a merge is the recursive
    dictionary update with lists replaced whole, and neither input changes (the OmegaConf rules the configs rely on)."""
    cfg = conf.create(tree)
    assert conf.to_container(cfg) == tree
    assert conf.to_container(conf.create(conf.to_yaml(cfg))) == tree

    def update(a, b):
        out = dict(a)
        for k, v in b.items():
            out[k] = update(out[k], v) if isinstance(v, dict) and isinstance(out.get(k), dict) else v
        return out

    merged = conf.merge(cfg, conf.create(other))
    assert conf.to_container(merged) == update(tree, other)
    assert conf.to_container(cfg) == tree                       # merge does not touch its inputs


@FAST
@given(rows=st.lists(st.lists(st.integers(1, 9), min_size=1, max_size=5), min_size=1, max_size=3), window=st.integers(0, 6))
def test_document_ids_and_cumulative_lengths_describe_the_same_mask(rows, window):
    """The three ways a batch can mark documents agree: ``document_ids`` per row, ``cu_seqlens`` over the flat
    stream, and the predicate "same row, same document, not in the future, inside the window"
    (optimus_dl/modules/model/blocks/attention.py:44-86)."""
    T = max(sum(r) for r in rows)
    rows = [r + ([T - sum(r)] if sum(r) < T else []) for r in rows]     # pad every row to T with one more document
    B = len(rows)
    ids = torch.tensor([[d for d, n in enumerate(r) for _ in range(n)] for r in rows])
    from_ids = build_doc_start(B, T, torch.device("cpu"), document_ids=ids)
    cu = torch.tensor([0] + list(np.cumsum([n for r in rows for n in r])))
    from_cu = build_doc_start(1, B * T, torch.device("cpu"), cu_seqlens=cu)
    assert torch.equal(from_ids, from_cu)
    mask = mask_from_doc_start(from_ids, window or None)
    flat_doc = (ids + 100 * torch.arange(B)[:, None]).reshape(-1)
    i = torch.arange(B * T)
    want = (flat_doc[:, None] == flat_doc[None, :]) & (i[None, :] <= i[:, None])
    if window:
        want &= i[None, :] > i[:, None] - window
    assert torch.equal(mask, want)
    assert mask.diagonal().all()                                        # every token sees itself


@FAST
@given(iterations=st.integers(10, 400), warm=st.floats(0.0, 0.5), decay=st.floats(0.05, 0.5),
       kind=st.sampled_from(["linear", "cosine", "square", "sqrt", "exp"]), lo=st.floats(0.01, 0.9),
       base=st.floats(1e-4, 10.0), probe=st.integers(0, 500))
def test_wsd_schedule_stays_in_range_is_monotone_per_phase_and_resumes_at_any_step(iterations, warm, decay, kind, lo, base, probe):
    """Warm-up never decreases, the plateau equals the base rate, the cool-down never increases and ends at
    ``final_lr_factor * base``; a schedule restored from its state at any step continues with the same rates
    (optimus_dl/modules/lr_scheduler/wsd_scheduler.py:14-234)."""
    from optimus_dl_b200.lr_scheduler import build_lr_scheduler

    def make():
        opt = torch.optim.SGD([{"params": [torch.nn.Parameter(torch.zeros(1))], "lr": base}], lr=base)
        return build_lr_scheduler({"_name": "wsd", "warmup_steps": None, "warmup_steps_fraction": warm, "fract_decay": decay,
                                   "decay_type": kind, "final_lr_factor": lo}, optimizer=opt, iterations=iterations), opt

    sched, opt = make()
    rates = []
    for _ in range(iterations + 3):
        rates.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    w = sched.warmup_steps
    d0 = iterations - int(decay * iterations)
    tol = 1e-9 * base
    assert all(-tol <= r <= base + tol for r in rates)
    assert all(b >= a - tol for a, b in zip(rates[:w], rates[1:w + 1]))
    assert all(math.isclose(r, base, rel_tol=1e-9) for r in rates[w:max(w, d0)])
    assert all(b <= a + tol for a, b in zip(rates[max(w, d0):iterations], rates[max(w, d0) + 1:iterations + 1]))
    assert math.isclose(rates[iterations], lo * base, rel_tol=1e-6)
    cut = min(probe, iterations)
    first, opt1 = make()
    for _ in range(cut):
        opt1.step()
        first.step()
    second, opt2 = make()
    second.load_state_dict(first.state_dict())
    for i in range(cut, min(cut + 5, iterations)):
        assert math.isclose(opt2.param_groups[0]["lr"] if i > cut else rates[cut], rates[i], rel_tol=1e-9)
        opt2.step()
        second.step()


@FAST
@given(B=st.integers(1, 3), T=st.integers(2, 12), V=st.integers(3, 40), smoothing=st.sampled_from([0.0, 0.1]),
       pad=st.booleans(), seed=st.integers(0, 100))
def test_criterion_equals_torch_cross_entropy_on_the_shifted_batch(B, T, V, smoothing, pad, seed):
    """The criterion's loss is ``F.cross_entropy`` of ``logits[:, :-1]`` against ``input_ids[:, 1:]`` with padding
    ignored, its gradient too (optimus_dl/modules/criterion/cross_entropy.py:42-376)."""
    from optimus_dl_b200.criterion import build_criterion

    g = torch.Generator().manual_seed(seed)
    table = torch.randn(V, V, generator=g, requires_grad=True)

    class Bigram(torch.nn.Module):
        def forward(self, input_ids, **_):
            return {"logits": table[input_ids]}

    ids = torch.randint(1, V, (B, T), generator=g)
    if pad:
        ids[0, -1] = 0
    crit = build_criterion({"_name": "cross_entropy", "label_smoothing": smoothing, "padding_token_id": 0 if pad else -100})
    loss, _ = crit(Bigram(), {"input_ids": ids})
    if pad and bool((ids[:, 1:] == 0).all()):
        assert loss.item() == 0.0              # nothing to predict: a zero loss, where torch's mean would be NaN
        return
    (grad,) = torch.autograd.grad(loss, table)
    t2 = table.detach().clone().requires_grad_(True)
    want = torch.nn.functional.cross_entropy(t2[ids[:, :-1]].reshape(-1, V), ids[:, 1:].reshape(-1),
                                             ignore_index=0 if pad else -100, label_smoothing=smoothing)
    (wgrad,) = torch.autograd.grad(want, t2)
    assert torch.allclose(loss, want, atol=1e-5) and torch.allclose(grad, wgrad, atol=1e-5)


@FAST
@given(T=st.integers(1, 10), hd=st.sampled_from([2, 4, 8, 16]), shift=st.integers(0, 20), seed=st.integers(0, 50))
def test_rotary_embedding_keeps_lengths_and_depends_on_position_differences_only(T, hd, shift, seed):
    """RoPE rotates pairs: vector norms are unchanged, and ``<rot(q, i), rot(k, j)>`` depends on ``i - j`` alone, so
    shifting every position by a constant changes no attention score (optimus_dl/modules/model/blocks/rope.py:13-253)."""
    from optimus_dl_b200.ops import rope as rope_ops

    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(1, T, 2, hd, generator=g), torch.randn(1, T, 1, hd, generator=g)
    table = rope_ops.precompute_freqs_cis(hd, T + shift + 1)
    pos = torch.arange(T)[None]
    q0, k0 = rope_ops.apply_rotary_emb(q, k, table, pos)
    q1, k1 = rope_ops.apply_rotary_emb(q, k, table, pos + shift)
    assert torch.allclose(q0.norm(dim=-1), q.norm(dim=-1), atol=1e-4) and torch.allclose(k1.norm(dim=-1), k.norm(dim=-1), atol=1e-4)
    s0 = torch.einsum("bthd,bshd->bhts", q0, k0.expand(-1, -1, 2, -1))
    s1 = torch.einsum("bthd,bshd->bhts", q1, k1.expand(-1, -1, 2, -1))
    assert torch.allclose(s0, s1, atol=1e-3)
