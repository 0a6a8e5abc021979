"""Model families on CPU: packed-vs-padded consistency, document isolation, sliding windows, GQA,
QK-norm, parameter groups, criterion bookkeeping."""

import pytest
import torch

from optimus_dl_b200.criterion import build_criterion
from optimus_dl_b200.metrics import compute_meters, meters_group
from optimus_dl_b200.models import build_model
from optimus_dl_b200.ops.attention import attention_ref, build_doc_start, mask_from_doc_start

MODELS = {
    "gpt2": dict(_name="gpt2", n_layer=2, n_head=4, n_embd=64, vocab_size=101, block_size=64),
    "llama2": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=101, sequence_length=64, multiple_of=8),
    "qwen3": dict(_name="qwen3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, head_dim=32, vocab_size=101, sequence_length=64, intermediate_size=96),
    "olmo3": dict(_name="olmo3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=101, sequence_length=64, intermediate_size=96,
                  layer_types=["sliding_attention", "full_attention"], sliding_window=8),
}


@pytest.mark.parametrize("name", ["llama2", "qwen3", "olmo3"])
def test_packed_batch_equals_separate_documents(name):
    torch.manual_seed(0)
    m = build_model(MODELS[name]).eval()
    a, b = torch.randint(0, 101, (1, 11)), torch.randint(0, 101, (1, 17))
    la, lb = m(a)["logits"], m(b)["logits"]
    packed = torch.cat([a, b], 1)
    pos = torch.cat([torch.arange(11), torch.arange(17)])[None]
    doc = torch.cat([torch.zeros(11), torch.ones(17)])[None].long()
    lp = m(packed, document_ids=doc, position_ids=pos)["logits"]
    assert torch.allclose(lp[:, :11], la, atol=1e-4) and torch.allclose(lp[:, 11:], lb, atol=1e-4)
    lc = m(packed, cu_seqlens=torch.tensor([0, 11, 28], dtype=torch.int32), position_ids=pos, max_seqlen=17)["logits"]
    assert torch.allclose(lc, lp, atol=1e-5)
    leak = m(packed, position_ids=pos)["logits"]
    assert not torch.allclose(leak[:, 11:], lb, atol=1e-3)       # without the mask the documents mix


def test_padded_batch_matches_unpadded_prefix():
    torch.manual_seed(0)
    m = build_model(MODELS["llama2"]).eval()
    x = torch.randint(0, 101, (1, 9))
    padded = torch.cat([x, torch.zeros(1, 5, dtype=torch.long)], 1)
    assert torch.allclose(m(padded, seq_lens=torch.tensor([9]))["logits"][:, :9], m(x)["logits"], atol=1e-5)


def test_mask_rule_windows_and_reference_attention():
    ds = build_doc_start(2, 6, torch.device("cpu"), document_ids=torch.tensor([[0, 0, 1, 1, 1, 2], [5, 5, 5, 5, 5, 5]]))
    assert ds.tolist() == [0, 0, 2, 2, 2, 5, 6, 6, 6, 6, 6, 6]
    m = mask_from_doc_start(ds, window=2)
    assert m[4].nonzero().flatten().tolist() == [3, 4] and m[6].nonzero().flatten().tolist() == [6] and m[11].nonzero().flatten().tolist() == [10, 11]
    q, k, v = torch.randn(12, 4, 8), torch.randn(12, 2, 8), torch.randn(12, 2, 8)
    out = attention_ref(q, k, v, ds)
    assert torch.allclose(out[0], v[0].repeat_interleave(2, 0), atol=1e-6)      # first token only sees itself


@pytest.mark.parametrize("name", list(MODELS))
def test_parameter_groups_and_tied_embeddings(name):
    m = build_model(MODELS[name])
    groups = m.make_parameter_groups()
    decay = {n for n, _ in groups[0]["params"]}
    no_decay = {n for n, _ in groups[1]["params"]}
    assert groups[1]["weight_decay"] == 0.0 and not (decay & no_decay)
    assert decay | no_decay == {n for n, _ in m.named_parameters()}
    assert all(n.endswith("weight") and "ln" not in n and "norm" not in n for n in decay)
    if m.config.tie_word_embeddings:
        assert m.lm_head.weight is m.transformer.wte.weight and "transformer.wte.weight" in no_decay
    torch.manual_seed(0)
    out = m.generate(torch.randint(0, 101, (2, 3)), max_new_tokens=4, temperature=0.8, top_k=5)
    assert out.shape == (2, 7)


def test_cross_entropy_shift_smoothing_padding_and_meters():
    torch.manual_seed(0)
    m = build_model(MODELS["llama2"])
    ids = torch.randint(0, 101, (3, 13))
    crit = build_criterion({"_name": "cross_entropy"})
    with meters_group("train", log_freq=1):
        loss, exposed = crit(m, {"input_ids": ids}, requested_protocols={"logits", "logits_targets", "classification", "loss"})
    logits = m(ids[:, :-1])["logits"]
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 101), ids[:, 1:].reshape(-1))
    assert torch.allclose(loss, ref, atol=1e-5) and exposed["logits"].shape == (3, 12, 101)
    meters = compute_meters("train")
    assert meters["batch_tokens"] == 36 and meters["batch_samples"] == 3 and abs(meters["loss"] - ref.item()) < 1e-3
    labels = ids[:, 1:].clone()
    labels[:, -4:] = 0
    l_pad, _ = build_criterion({"_name": "cross_entropy", "padding_token_id": 0, "label_smoothing": 0.1})(m, {"input_ids": ids[:, :-1], "labels": labels})
    tgt = torch.where(labels == 0, torch.full_like(labels, -100), labels)
    ref2 = torch.nn.functional.cross_entropy(logits.reshape(-1, 101), tgt.reshape(-1), ignore_index=-100, label_smoothing=0.1)
    assert torch.allclose(l_pad, ref2, atol=1e-5)
    cap, _ = build_criterion({"_name": "cross_entropy", "logit_softcap": 5.0})(m, {"input_ids": ids})
    ref3 = torch.nn.functional.cross_entropy((5.0 * torch.tanh(logits / 5.0)).reshape(-1, 101), ids[:, 1:].reshape(-1))
    assert torch.allclose(cap, ref3, atol=1e-5)
    one, _ = crit(m, {"input_ids": ids[:, :2]})
    assert torch.isfinite(one)


def test_rope_table_and_broadcast_helper():
    """``precompute_freqs_cis`` / ``apply_rotary_emb`` / ``_reshape_for_broadcast`` (optimus_dl/modules/model/blocks/rope.py)."""
    import pytest
    import torch

    from optimus_dl_b200.models.blocks.rope import _reshape_for_broadcast, apply_rotary_emb, precompute_freqs_cis

    table = precompute_freqs_cis(64, 100)
    assert table.shape == (100, 32, 2) and table.dtype == torch.float32
    assert torch.allclose(table.norm(dim=-1), torch.ones(100, 32), atol=1e-6)        # unit (cos, sin) pairs
    assert precompute_freqs_cis(32, 50, 1000.0).shape == (50, 16, 2)
    q, k = torch.randn(2, 10, 8, 64), torch.randn(2, 10, 8, 64)
    q_rot, k_rot = apply_rotary_emb(q, k, precompute_freqs_cis(64, 10))
    assert q_rot.shape == q.shape and k_rot.dtype == k.dtype and not torch.allclose(q_rot, q)
    assert torch.allclose(q_rot.norm(dim=-1), q.norm(dim=-1), atol=1e-4)             # a rotation keeps lengths
    flat = torch.randn(10, 32, dtype=torch.complex64)
    with pytest.raises(AssertionError):
        _reshape_for_broadcast(flat, torch.randn(32, dtype=torch.complex64))
    with pytest.raises(AssertionError):
        _reshape_for_broadcast(flat, torch.randn(2, 5, 16, dtype=torch.complex64))
    assert _reshape_for_broadcast(torch.randn(2, 10, 32, 2), torch.randn(2, 10, 8, 32, 2)).shape == (2, 10, 1, 32, 2)
    assert _reshape_for_broadcast(precompute_freqs_cis(64, 10), torch.randn(2, 10, 8, 32, 2)).shape == (1, 10, 1, 32, 2)
