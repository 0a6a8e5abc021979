"""Cross-entropy criterion: shifting, labels, padding, smoothing, soft caps, meters and exposed protocols
(behaviour of optimus_dl/modules/criterion/cross_entropy.py:103-408), checked against plain PyTorch."""

import math

import pytest
import torch
import torch.nn.functional as F

from optimus_dl_b200.criterion.cross_entropy import CrossEntropyCriterion, CrossEntropyCriterionConfig
from optimus_dl_b200.metrics import base as mb


class _Table(torch.nn.Module):
    """Logits depend only on the input token: ``logits[b, t] = table[ids[b, t]]``."""

    def __init__(self, vocab: int, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.table = torch.nn.Parameter(torch.randn(vocab, vocab, generator=g))
        self.seen: dict = {}

    def forward(self, input_ids, **kw):
        self.seen = dict(kw, input_ids=input_ids)
        return {"logits": self.table[input_ids]}


def _crit(**kw):
    return CrossEntropyCriterion(CrossEntropyCriterionConfig(**kw))


def _meters(name="train"):
    out = mb.compute_meters(name, aggregate=False)
    return out


def test_shifts_inputs_and_every_token_aligned_tensor():
    V = 11
    model = _Table(V)
    ids = torch.randint(0, V, (3, 9))
    pos = torch.arange(9)[None].expand(3, 9)
    docs = torch.zeros(3, 9, dtype=torch.long)
    seq_lens = torch.tensor([9, 5, 7])
    extra = torch.ones(3, 4)                       # not token-aligned: passed through untouched
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit()(model, {"input_ids": ids, "position_ids": pos, "document_ids": docs, "seq_lens": seq_lens,
                                  "extra": extra})
    assert model.seen["input_ids"].shape == (3, 8) and torch.equal(model.seen["input_ids"], ids[:, :-1])
    assert model.seen["position_ids"].shape == (3, 8) and model.seen["document_ids"].shape == (3, 8)
    assert torch.equal(model.seen["seq_lens"], seq_lens - 1)
    assert model.seen["extra"].shape == (3, 4)
    ref = F.cross_entropy(model.table[ids[:, :-1]].reshape(-1, V), ids[:, 1:].reshape(-1))
    assert torch.allclose(loss, ref, atol=1e-6)


def test_explicit_labels_are_used_as_is():
    V = 7
    model = _Table(V)
    ids = torch.randint(0, V, (2, 6))
    labels = torch.randint(0, V, (2, 6))
    labels[0, :2] = -100
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit()(model, {"input_ids": ids, "labels": labels})
    assert model.seen["input_ids"].shape == (2, 6)
    ref = F.cross_entropy(model.table[ids].reshape(-1, V), labels.reshape(-1), ignore_index=-100)
    assert torch.allclose(loss, ref, atol=1e-6)


def test_padding_token_is_ignored_and_tokens_are_counted():
    V, pad = 9, 8
    model = _Table(V)
    ids = torch.randint(0, pad, (2, 8))
    ids[0, 5:] = pad
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit(padding_token_id=pad)(model, {"input_ids": ids})
        m = mb.compute_meters("train", aggregate=False)
    tg = ids[:, 1:].clone()
    tg[tg == pad] = -100
    ref = F.cross_entropy(model.table[ids[:, :-1]].reshape(-1, V), tg.reshape(-1), ignore_index=-100)
    assert torch.allclose(loss, ref, atol=1e-6)
    n_valid = int((tg != -100).sum())
    assert m["batch_tokens"] == n_valid and m["total_tokens"] == n_valid
    assert m["batch_samples"] == 2 and m["input_max_seq_len"] == 7
    assert abs(m["loss"] - ref.item()) < 1e-3
    assert abs(m["perplexity"] - math.exp(ref.item())) / math.exp(ref.item()) < 1e-3
    pred = model.table[ids[:, :-1]].argmax(-1)
    acc = ((pred == tg) & (tg != -100)).sum().item() / n_valid
    assert abs(m["accuracy"] - acc) <= 5e-3                          # logged with two decimals, as the reference does


@pytest.mark.parametrize("smoothing", [0.0, 0.1])
@pytest.mark.parametrize("cap,kind", [(None, "tanh"), (5.0, "tanh"), (1.0, "sigmoid")])
def test_label_smoothing_and_soft_caps_match_reference_math(smoothing, cap, kind):
    V = 13
    model = _Table(V, seed=3)
    with torch.no_grad():
        model.table.mul_(4.0)
    ids = torch.randint(0, V, (2, 7))
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit(label_smoothing=smoothing, logit_softcap=cap, softcap_type=kind)(model, {"input_ids": ids})
    z = model.table[ids[:, :-1]].reshape(-1, V).float()
    if cap is not None:
        z = cap * torch.tanh(z / cap) if kind == "tanh" else 23.0 * torch.sigmoid((z + 5.0) / 7.5)
    ref = F.cross_entropy(z, ids[:, 1:].reshape(-1), label_smoothing=smoothing)
    assert torch.allclose(loss, ref, atol=1e-5), (loss.item(), ref.item())
    loss.backward()
    assert model.table.grad is not None and torch.isfinite(model.table.grad).all()


def test_single_token_targets_and_all_ignored():
    V = 5
    model = _Table(V)
    ids = torch.randint(0, V, (1, 2))              # one target token
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit()(model, {"input_ids": ids})
    assert torch.allclose(loss, F.cross_entropy(model.table[ids[:, :1]].reshape(-1, V), ids[:, 1:].reshape(-1)), atol=1e-6)
    labels = torch.full((1, 2), -100)
    with mb.meters_group("train", log_freq=1):
        loss, _ = _crit()(model, {"input_ids": ids, "labels": labels})
    assert torch.isfinite(loss) and loss.item() == 0.0   # nothing to predict: zero loss, no NaN


def test_exposed_protocols_and_packed_unflatten():
    V = 6
    model = _Table(V)
    ids = torch.randint(0, V, (1, 10))
    labels = torch.randint(0, V, (1, 10))
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    want = {"loss", "logits", "logits_targets", "logits_mask", "input_tokens", "classification"}
    with mb.meters_group("train", log_freq=1):
        loss, exposed = _crit()(model, {"input_ids": ids, "labels": labels, "cu_seqlens": cu, "max_seqlen": 6},
                                requested_protocols=want)
        m = mb.compute_meters("train", aggregate=False)
    assert set(exposed) == want
    assert exposed["logits"].shape == (2, 6, V) and exposed["logits_targets"].shape == (2, 6)
    assert torch.equal(exposed["logits_targets"][0, :4], labels[0, :4]) and (exposed["logits_targets"][0, 4:] == -100).all()
    assert torch.equal(exposed["logits"][1], model.table[ids[0, 4:]].detach())
    assert torch.equal(exposed["logits_mask"], exposed["logits_targets"] != -100)
    assert torch.equal(exposed["classification"]["predictions"], exposed["logits"].argmax(-1))
    assert torch.equal(exposed["input_tokens"], ids) and torch.allclose(exposed["loss"], loss)
    assert m["batch_samples"] == 2 and m["input_max_seq_len"] == 6 and m["input_mean_seq_len"] == 5


def test_total_counters_accumulate_over_steps_while_batch_counters_reset():
    V = 6
    model = _Table(V)
    crit = _crit()
    seen = []
    for step in range(3):
        ids = torch.randint(0, V, (2, 5))
        with mb.meters_group("train", log_freq=1) as should_log:
            crit(model, {"input_ids": ids})
            assert should_log
            seen.append(mb.compute_meters("train", aggregate=False))
        mb.step_meters("train")
        mb.reset_meters("train")               # what the train loop does after a logging step
    assert [m["batch_tokens"] for m in seen] == [8, 8, 8]
    assert [m["total_tokens"] for m in seen] == [8, 16, 24]
    assert [m["total_samples"] for m in seen] == [2, 4, 6]
