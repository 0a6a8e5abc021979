"""Metrics and eval recipes end to end on CPU with random weights and synthetic data."""

import types

from optimus_dl_b200.core import conf
from optimus_dl_b200.core.config_utils import non_resolving_instantiate
from optimus_dl_b200.core.registry import build

MODEL = {"_name": "llama2", "n_layer": 2, "n_head": 2, "n_embd": 32, "vocab_size": 258, "sequence_length": 64,
         "intermediate_size": 64}


def test_metrics_recipe(tmp_path):
    cfg = conf.create({
        "_name": "base",
        "common": {"use_gpu": False, "max_iterations": 3, "output_path": str(tmp_path), "tokenizer": None},
        "model": MODEL,
        "criterion": {"_name": "cross_entropy"},
        "data": {"eval_datasets": {"synth": {
            "source": {"_name": "synthetic_tokens", "vocab_size": 258, "length": 33, "num_documents": 20},
            "transform": {"_name": "basic_batcher", "batch_size": 4, "pad_token_id": 0}}}},
        "metrics": {"synth": [{"_name": "source_group", "prefix": "lm", "sources": {"lm": {"_name": "causal_lm"}},
                               "metrics": [{"_name": "accuracy"}, {"_name": "perplexity"}, {"_name": "loss"}]}]},
        "loggers": [{"_name": "jsonl", "output_dir": str(tmp_path / "logs")}],
    })
    recipe = build("metrics_recipe", non_resolving_instantiate(cfg))
    results = recipe.run()
    assert list(results) == ["metrics/synth"]
    vals = results["metrics/synth"]
    # metric names as the reference forms them: <prefix>/<name>_metric/<sub-metric>
    assert 4.0 < vals["loss"] < 7.0 and "lm/accuracy_metric/accuracy" in vals and "lm/perplexity_metric/perplexity" in vals
    assert any((tmp_path / "logs").rglob("*.jsonl"))


def test_eval_adapter_scores_and_generates():
    from optimus_dl_b200.recipe.eval import EvalConfig, EvalRecipe

    cfg = conf.merge(conf.create(EvalConfig()), conf.create({
        "common": {"checkpoint_path": None, "use_gpu": False, "tokenizer": {"_name": "char_tokenize"}, "model": MODEL},
        "lm_eval": {"batch_size": 3}}))
    lm = EvalRecipe(cfg).build_eval_model()
    req = lambda *a: types.SimpleNamespace(args=a)  # noqa: E731
    reqs = [req("hello ", "world"), req("", "abc"), req("the quick brown", " fox"), req("a", "b")]
    batched = lm.loglikelihood(reqs)
    lm.batch_size = 1
    single = lm.loglikelihood(reqs)
    assert all(abs(a[0] - b[0]) < 1e-4 and a[1] == b[1] for a, b in zip(batched, single))
    assert all(ll < 0 for ll, _ in batched)
    (rolling,) = lm.loglikelihood_rolling([req("x" * 150)])
    assert rolling < 0
    (text,) = lm.generate_until([req("hello", {"until": ["\n"], "max_gen_toks": 6})])
    assert isinstance(text, str) and "\n" not in text


def _write_corpus(root):
    import json

    import pyarrow as pa
    import pyarrow.parquet as pq

    (root / "data").mkdir(parents=True)
    docs = [f"document number {i} " + "lorem ipsum " * (i % 7 + 1) for i in range(300)]
    with open(root / "data" / "train-00000.jsonl", "w") as f:
        for d in docs[:100]:
            f.write(json.dumps({"text": d}) + "\n")
    pq.write_table(pa.table({"text": docs[100:200]}), root / "data" / "train-00001.parquet")
    pq.write_table(pa.table({"text": docs[200:]}), root / "data" / "train-00002.parquet")
    with open(root / "data" / "validation-00000.jsonl", "w") as f:
        f.write(json.dumps({"text": "held out"}) + "\n")
    return docs


def _prep_cfg(src, out, num_proc=1):
    from optimus_dl_b200.recipe.pretokenize import DataPrepConfig

    return conf.merge(conf.create(DataPrepConfig()), conf.create({
        "dataset": {"repo_id": str(src), "split": "train"},
        "processing": {"shard_size_mb": 1, "shuffle_buffer_size": 16, "num_proc": num_proc, "dtype": "uint16"},
        "output": {"dir": str(out), "name": "shard"},
        "tokenizer": {"_name": "char_tokenize"}}))


def test_pretokenize_roundtrip_and_resume(tmp_path):
    import json

    import numpy as np

    from optimus_dl_b200.recipe.pretokenize import DataPrepRecipe
    from optimus_dl_b200.recipe.pretokenize.checkpoint import CheckpointManager
    from optimus_dl_b200.recipe.pretokenize.processor import TokenProcessor
    from optimus_dl_b200.recipe.pretokenize.source import FileFinder
    from optimus_dl_b200.tokenizer import build_tokenizer

    docs = _write_corpus(tmp_path / "src")
    cfg = _prep_cfg(tmp_path / "src", tmp_path / "out")
    DataPrepRecipe(cfg).run()
    index = json.loads((tmp_path / "out" / "index.json").read_text())
    assert index["config"]["tokenizer"]["_name"] == "char_tokenize"
    toks = np.concatenate([np.load(tmp_path / "out" / f["file"]) for f in index["files"]])
    lens = np.concatenate([np.load(tmp_path / "out" / f["lens_file"]) for f in index["files"]])
    assert index["total_tokens"] == len(toks) == int(lens.sum()) and len(lens) == 300  # validation file excluded
    tok = build_tokenizer(cfg.tokenizer)
    decoded, o = set(), 0
    for n in lens:
        decoded.add(tok.decode([t for t in toks[o:o + n].tolist() if t < 256]))
        o += int(n)
    assert decoded == set(docs)
    assert not (tmp_path / "out" / "checkpoint.pkl").exists()

    # same order with worker processes, and an interrupted run resumes to the identical stream
    files = FileFinder(cfg.dataset, 42).get_files()
    full = [tuple(d) for d in TokenProcessor(files, cfg)]
    par = [tuple(d) for d in TokenProcessor(files, _prep_cfg(tmp_path / "src", tmp_path / "out2", num_proc=2))]
    assert par == full
    p1 = TokenProcessor(files, cfg)
    head = []
    for d in p1:
        head.append(tuple(d))
        if len(head) == 137:
            break
    state = p1.get_state()
    p1.close()
    p2 = TokenProcessor(files, cfg)
    p2.load_state(state)
    assert head + [tuple(d) for d in p2] == full
    assert CheckpointManager(tmp_path / "out").load() is None


def test_pretokenize_rejects_small_dtype(tmp_path):
    import pytest

    from optimus_dl_b200.recipe.pretokenize import DataPrepRecipe

    _write_corpus(tmp_path / "src")
    cfg = _prep_cfg(tmp_path / "src", tmp_path / "out")
    cfg.tokenizer = conf.create({"_name": "inline_tokens_tokenizer", "tokens": [f"t{i}" for i in range(70000)]})
    with pytest.raises(ValueError, match="exceeds the maximum value"):
        DataPrepRecipe(cfg)
