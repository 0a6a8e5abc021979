"""Worker of tests/test_reference_differential.py: imports the UNMODIFIED reference (baseline/_ref, with the stand-in
third-party modules of baseline/ref_deps) next to this package in one CPU process and compares the two on the same
inputs. ``python tests/_ref_diff_worker.py <check>`` prints ``DIFF_OK <check>`` or raises."""

import importlib
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [os.path.join(ROOT, "baseline", "ref_deps"), os.path.join(ROOT, "baseline", "_ref"), ROOT]

import logging  # noqa: E402

logging.disable(logging.INFO)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import optimus_dl  # noqa: E402,F401
from omegaconf import OmegaConf  # noqa: E402


def R(mod: str):
    return importlib.import_module("optimus_dl.modules." + mod)


MODELS = {
    "gpt2": dict(_name="gpt2", n_layer=2, n_head=4, n_embd=64, vocab_size=97, block_size=64, bias=True),
    "llama2": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=97, sequence_length=64, multiple_of=8),
    "llama2_qknorm": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=97, sequence_length=64,
                          multiple_of=8, use_qk_norm=True),
    "qwen3": dict(_name="qwen3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, head_dim=32, vocab_size=97, sequence_length=64,
                  intermediate_size=96),
    "llama2_rope_llama3": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=97, sequence_length=64,
                               multiple_of=8, tie_word_embeddings=True,
                               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                             "high_freq_factor": 4.0, "original_max_position_embeddings": 16}),
    "llama2_rope_yarn": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=97, sequence_length=64,
                             multiple_of=8, bias=True, rope_theta=500000.0,
                             rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16}),
    "qwen3_bias": dict(_name="qwen3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, head_dim=32, vocab_size=97,
                       sequence_length=64, intermediate_size=96, attention_bias=True),
    "olmo3": dict(_name="olmo3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=97, sequence_length=64,
                  intermediate_size=96, layer_types=["sliding_attention", "full_attention"], sliding_window=8),
}


def _pair(cfg):
    import optimus_dl_b200.models as om

    torch.manual_seed(0)
    ref = R("model").build_model(OmegaConf.create(cfg))
    ours = om.build_model(dict(cfg))
    assert set(ref.state_dict()) == set(ours.state_dict()), sorted(set(ref.state_dict()) ^ set(ours.state_dict()))[:5]
    ours.load_state_dict(ref.state_dict())
    return ref, ours


def check_models() -> None:
    """Same weights -> same logits (plain and packed batches), same parameter groups, for every model family."""
    for name, cfg in MODELS.items():
        ref, ours = _pair(cfg)
        ref.eval(), ours.eval()
        x = torch.randint(0, 97, (2, 24))
        docs = torch.tensor([[0] * 10 + [1] * 14, [0] * 24])
        pos = torch.stack([torch.cat([torch.arange(10), torch.arange(14)]), torch.arange(24)])
        with torch.no_grad():
            assert torch.allclose(ref(x)["logits"], ours(x)["logits"], atol=2e-6), name
            if name != "gpt2":       # the reference's GPT-2 ignores document and position ids
                a = ref(x, document_ids=docs, position_ids=pos)["logits"]
                b = ours(x, document_ids=docs, position_ids=pos)["logits"]
                assert torch.allclose(a, b, atol=2e-6), name
                # a flat (packed) batch described by cumulative lengths, and per-row valid lengths (positions past
                # them are padding and not compared)
                cu = torch.tensor([0, 7, 15, 24], dtype=torch.int32)
                fpos = torch.cat([torch.arange(7), torch.arange(8), torch.arange(9)])[None]
                a = ref(x[:1], cu_seqlens=cu, max_seqlen=9, position_ids=fpos)["logits"]
                b = ours(x[:1], cu_seqlens=cu, max_seqlen=9, position_ids=fpos)["logits"]
                assert torch.allclose(a, b, atol=2e-6), name
            lens = torch.tensor([24, 13])
            a, b = ref(x, seq_lens=lens)["logits"], ours(x, seq_lens=lens)["logits"]
            assert torch.allclose(a[0], b[0], atol=2e-6) and torch.allclose(a[1, :13], b[1, :13], atol=2e-6), name

        def sig(groups):
            return [(tuple(sorted(k for k in g if k != "params")), len(g["params"]), g.get("weight_decay")) for g in groups]

        assert sig(ref.make_parameter_groups()) == sig(ours.make_parameter_groups()), name


def check_train_parts() -> None:
    """Criterion loss and meters; AdamW / SOAP with every schedule, step by step, from the same gradients."""
    import optimus_dl_b200.criterion as oc
    import optimus_dl_b200.lr_scheduler as ol
    import optimus_dl_b200.optim as oo
    from optimus_dl_b200.metrics import base as omb
    from optimus_dl_b200.parallel.collective import FakeCollective

    rmb = importlib.import_module("optimus_dl.modules.metrics")
    ref, ours = _pair(MODELS["llama2"])
    rfake = importlib.import_module("optimus_dl.modules.distributed.fake").FakeCollective(0, 1)
    for ccfg in (dict(_name="cross_entropy"), dict(_name="cross_entropy", label_smoothing=0.1),
                 dict(_name="cross_entropy", padding_token_id=5),
                 dict(_name="cross_entropy", logit_softcap=5.0, softcap_type="tanh"),
                 dict(_name="cross_entropy", label_smoothing=0.2, logit_softcap=1.0, softcap_type="sigmoid")):
        rc = R("criterion").build_criterion(OmegaConf.create(ccfg), collective=rfake)
        c = oc.build_criterion(dict(ccfg), collective=FakeCollective(0, 1, torch.device("cpu")))
        x = torch.randint(0, 97, (3, 20))
        with rmb.meters_group("g", log_freq=1):
            rl, _ = rc(ref, {"input_ids": x.clone()})
        with omb.meters_group("g", log_freq=1):
            l, _ = c(ours, {"input_ids": x.clone()})
        assert abs(rl.item() - l.item()) < 1e-6, ccfg
        gr, g = torch.autograd.grad(rl, ref.lm_head.weight)[0], torch.autograd.grad(l, ours.lm_head.weight)[0]
        assert torch.allclose(gr, g, atol=1e-7), ccfg
        a, b = rmb.compute_meters("g"), omb.compute_meters("g")
        a.pop("ms_spent_logging", None), b.pop("ms_spent_logging", None)
        assert set(a) == set(b), (sorted(a), sorted(b))
        assert all(abs(float(a[k]) - float(b[k])) <= 1e-6 * max(1.0, abs(float(a[k]))) for k in a), (ccfg, a, b)
        rmb.reset_meters("g"), omb.reset_meters("g")
    for ocfg in (dict(_name="adamw", lr=1e-2, weight_decay=0.1), dict(_name="soap", lr=1e-2, weight_decay=0.01, precondition_frequency=2)):
        for scfg in (None, dict(_name="wsd", warmup_steps=2, fract_decay=0.5), dict(_name="cosine_annealing"),
                     dict(_name="linear_warmup", warmup_steps=3)):
            ref, ours = _pair(MODELS["llama2"])
            ro = R("optim").build_optimizer(OmegaConf.create(ocfg), params=ref.make_parameter_groups())
            o = oo.build_optimizer(dict(ocfg), params=ours.make_parameter_groups())
            rs = R("lr_scheduler").build_lr_scheduler(OmegaConf.create(scfg), optimizer=ro, iterations=4) if scfg else None
            s = ol.build_lr_scheduler(dict(scfg), optimizer=o, iterations=4) if scfg else None
            g = torch.Generator().manual_seed(1)
            for _ in range(4):
                x = torch.randint(0, 97, (8, 32), generator=g)
                ref(x)["logits"].float().logsumexp(-1).mean().backward()
                for p, q in zip(ref.parameters(), ours.parameters()):     # the same gradients for both optimizers
                    q.grad = p.grad.clone()
                ro.step(), o.step(), ro.zero_grad(), o.zero_grad()
                if rs is not None:
                    rs.step(), s.step()
                assert [gr["lr"] for gr in ro.param_groups] == [gr["lr"] for gr in o.param_groups]
            worst = max((p - q).abs().max().item() for p, q in zip(ref.parameters(), ours.parameters()))
            assert worst < (1e-7 if ocfg["_name"] == "adamw" else 1e-4), (ocfg["_name"], scfg, worst)


def _corpus(tmp: str) -> tuple[str, str]:
    txt = os.path.join(tmp, "t.txt")
    with open(txt, "w") as f:
        for i in range(400):
            f.write(("line %d " % i) + "abcdefghij" * (i % 7 + 1) + "\n")
    tok = os.path.join(tmp, "tok")
    os.makedirs(tok)
    rng, c, files = np.random.default_rng(0), 0, []
    for s in range(3):
        lens = rng.integers(5, 60, size=20)
        np.save(os.path.join(tok, f"s_{s:010d}.npy"), np.arange(c, c + lens.sum(), dtype=np.uint16))
        np.save(os.path.join(tok, f"s_{s:010d}_lens.npy"), lens.astype(np.uint32))
        files.append({"file": f"s_{s:010d}.npy", "lens_file": f"s_{s:010d}_lens.npy", "num_tokens": int(lens.sum()),
                      "num_docs": len(lens), "shard_idx": s})
        c += int(lens.sum())
    json.dump({"files": files, "total_tokens": c, "config": {"dtype": "np.uint16"}}, open(os.path.join(tok, "index.json"), "w"))
    return txt, tok


def _same(a, b) -> bool:
    if isinstance(a, dict):
        return isinstance(b, dict) and a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, (np.ndarray, torch.Tensor)) or isinstance(b, (np.ndarray, torch.Tensor)):
        return np.array_equal(np.asarray(a), np.asarray(b))
    return a == b


def check_data() -> None:
    """Pipelines built from one config hand out identical batches, and each resumes from the other's state."""
    import optimus_dl_b200.data as od

    rd = R("data")
    txt, tok = _corpus(tempfile.mkdtemp())

    def chain(bs):
        return {"_name": "compose", "transforms": [
            {"_name": "tokenize", "tokenizer_config": {"_name": "char_tokenize"}, "worker_cfg": {"num_workers": 0}},
            {"_name": "chunk_tokens", "max_seq_len": 32}, {"_name": "shuffle", "buffer_size": 16},
            {"_name": "flat_batcher", "batch_size": bs, "seq_len": 32, "mask_documents": True}]}

    pipes = {
        "txt+loop": {"source": {"_name": "loop", "inner": {"_name": "txt_lines", "file_link": txt}}, "transform": chain(2)},
        "documents shuffled, flat": {
            "source": {"_name": "tokenized_dataset", "data_dir": tok, "strategy": {"_name": "document", "shuffle": True}},
            "transform": {"_name": "compose", "transforms": [
                {"_name": "shuffle", "buffer_size": 8},
                {"_name": "flat_batcher", "batch_size": 2, "seq_len": 16, "mask_documents": True, "flatten": True}]}},
        "skips + padded batches": {
            "source": {"_name": "tokenized_dataset", "data_dir": tok, "strategy": {"_name": "document"}},
            "transform": {"_name": "compose", "transforms": [
                {"_name": "skip_random", "probability": 0.3}, {"_name": "skip_interleaved", "skip_count": 1},
                {"_name": "basic_batcher", "batch_size": 3, "pad_token_id": 0}]}},
        "composite": {"source": {"_name": "composite", "stop_criteria": "CYCLE_FOREVER", "datasets": {
            "a": {"dataset": {"_name": "txt_lines", "file_link": txt}, "weight": 1.0, "cycle": True},
            "b": {"dataset": {"_name": "loop", "inner": {"_name": "txt_lines", "file_link": txt}}, "weight": 3.0, "cycle": True}}},
            "transform": chain(1)},
    }
    for name, cfg in pipes.items():
        for rank, world in ((0, 1), (1, 3)):
            def build(ref: bool):
                if ref:
                    return rd.build_data_pipeline(OmegaConf.create({**cfg, "profile": False, "report_freq": 100}), rank=rank,
                                                  world_size=world, seed=13).dataloader
                return od.build_data_pipeline(dict(cfg), rank=rank, world_size=world, seed=13).dataloader

            r, o = build(True), build(False)
            r.reset(), o.reset()
            n = 0
            for _ in range(12):
                try:
                    a = next(r)
                except StopIteration:
                    a = None
                try:
                    b = next(o)
                except StopIteration:
                    b = None
                assert (a is None) == (b is None) and (a is None or _same(a, b)), (name, rank, world, n)
                if a is None:
                    break
                n += 1
            if a is None:
                continue
            r2, o2 = build(True), build(False)
            r2.reset(o.state_dict()), o2.reset(r.state_dict())
            want = next(r)
            assert _same(next(r2), want) and _same(next(o2), want), (name, rank, world, "resume from the other's state")


def check_checkpoints() -> None:
    """A checkpoint written by either manager loads in the other; both then continue bit-identically."""
    import optimus_dl_b200.lr_scheduler as ol
    import optimus_dl_b200.models as om
    import optimus_dl_b200.optim as oo
    from optimus_dl_b200.checkpoint import CheckpointManager as OurCM
    from optimus_dl_b200.parallel.collective import FakeCollective as OurFake

    ck = R("checkpoint")
    rfake = importlib.import_module("optimus_dl.modules.distributed.fake").FakeCollective
    cfg, ocfg, scfg = MODELS["llama2"], dict(_name="adamw", lr=1e-2, weight_decay=0.1), dict(_name="wsd", warmup_steps=2, fract_decay=0.5)

    def make(ref: bool):
        torch.manual_seed(0)
        if ref:
            m = R("model").build_model(OmegaConf.create(cfg))
            o = R("optim").build_optimizer(OmegaConf.create(ocfg), params=m.make_parameter_groups())
            return m, o, R("lr_scheduler").build_lr_scheduler(OmegaConf.create(scfg), optimizer=o, iterations=10)
        m = om.build_model(dict(cfg))
        m.load_state_dict(make(True)[0].state_dict())
        o = oo.build_optimizer(dict(ocfg), params=m.make_parameter_groups())
        return m, o, ol.build_lr_scheduler(dict(scfg), optimizer=o, iterations=10)

    def train(m, o, s, n, seed):
        g = torch.Generator().manual_seed(seed)
        for _ in range(n):
            x = torch.randint(0, 97, (4, 16), generator=g)
            loss = m(x)["logits"].float().logsumexp(-1).mean()
            o.zero_grad(), loss.backward(), o.step(), s.step()

    for from_ref in (True, False):
        d = tempfile.mkdtemp()
        m, o, s = make(from_ref)
        train(m, o, s, 3, seed=1)
        if from_ref:
            ck.CheckpointManager(ck.CheckpointManagerConfig(_name="base")).save_checkpoint(
                checkpoint_path=d, model=m, optimizer=o, lr_scheduler=s, collective=rfake(0, 1), full_config={"model": cfg},
                iteration=3, is_save_persistent=True, is_save_last=True)
            m2, o2, s2 = make(False)
            OurCM(output_path=d).load_checkpoint(d, model=m2, optimizer=o2, lr_scheduler=s2,
                                                 collective=OurFake(0, 1, torch.device("cpu")))
        else:
            OurCM(output_path=d).save_checkpoint(iteration=3, model=m, optimizer=o, lr_scheduler=s,
                                                 collective=OurFake(0, 1, torch.device("cpu")), full_config={"model": cfg})
            m2, o2, s2 = make(True)
            ck.CheckpointManager(ck.CheckpointManagerConfig(_name="base")).load_checkpoint(
                checkpoint_path=d, model=m2, optimizer=o2, lr_scheduler=s2, collective=rfake(0, 1))
        train(m, o, s, 2, seed=5), train(m2, o2, s2, 2, seed=5)
        assert all(torch.equal(p, q) for p, q in zip(m.parameters(), m2.parameters())), from_ref
        assert o.param_groups[0]["lr"] == o2.param_groups[0]["lr"]


def check_recipe_accumulation() -> None:
    """The recipe with two accumulation steps, gradient clipping and bf16 autocast."""
    check_recipe(extra=["optimization.acc_steps=2", "optimization.clip_grad_norm=0.5", "optimization.amp.enabled=true"], tol=1e-3)


def check_recipe_resume() -> None:
    """Four iterations, then a second run on the same output directory that resumes from the checkpoint (model,
    optimizer, schedule, data position, meters) and continues to eight."""
    check_recipe(phases=[["optimization.iterations=4"], ["optimization.iterations=8"]])


def _recipe_overrides(tmp: str, which: str, data: str, extra: list[str] | None) -> list[str]:
    return [f"common.output_path={tmp}/{which}", "optimization.iterations=8", "common.save_freq=4", "common.log_freq=1",
            "common.eval_freq=4", "++common.eval_iterations=2", "++common.use_gpu=false", "~model_transforms",
            "optimization.amp.enabled=false", "data.train_datasets.source.inner._name=txt_lines",
            f"+data.train_datasets.source.inner.file_link={data}", "data.eval_datasets.tinyshakespeare.source._name=txt_lines",
            f"+data.eval_datasets.tinyshakespeare.source.file_link={data}", "++common.seed=42", "++common.data_seed=42",
            "++common.deterministic=true", "++model.n_layer=1", "++model.n_head=2", "++model.n_embd=32",
            "++model.intermediate_size=64", "lr_scheduler.warmup_steps=0", "args.batch_size=4", "args.seq_len=64",
            "loggers.1.enabled=false", f"loggers.0.output_dir={tmp}/{which}/logs"] + list(extra or [])


def _recipe_corpus(tmp: str) -> str:
    data = os.path.join(tmp, "data.txt")
    if not os.path.exists(data):
        with open(data + f".{os.getpid()}", "w") as f:
            for i in range(600):
                f.write(f"Line {i}: This is some dummy text for training Llama, number {i * i}.\n")
        os.replace(data + f".{os.getpid()}", data)
    return data


def _run_reference_recipe(tmp: str, extra: list[str] | None, phases: list[list[str]], transforms: list[dict]) -> None:
    """The reference's recipe on the fully resolved config (its own instantiate step needs OmegaConf internals); the
    weights it starts from are kept in ``init.pt`` for the other side."""
    import optimus_dl.recipe.train.base  # noqa: F401
    from optimus_dl.core.registry import build as ref_build
    from optimus_dl_b200.core import compose, conf
    import optimus_dl_b200.core.config_utils  # noqa: F401  (registers the resolvers the config uses)

    data, init_file = _recipe_corpus(tmp), os.path.join(tmp, "init.pt")
    for i, phase in enumerate(phases):
        cfg = compose.compose(os.path.join(ROOT, "configs", "train"), "train_llama_shakespeare",
                              _recipe_overrides(tmp, "ref", data, extra) + phase)
        plain = conf.to_container(cfg, resolve=True)
        for k in ("model_builder", "optimizer_builder", "criterion_builder", "data_builder", "scheduler_builder",
                  "logger_manager", "checkpoint_manager", "evaluator"):
            plain[k] = {**(plain.get(k) or {})}
            if plain[k].get("_name") is None:
                plain[k]["_name"] = "base"
        plain["model_transforms"] = list(transforms)
        recipe = ref_build("train_recipe", OmegaConf.create(plain))
        if i == 0:
            orig = recipe.build_model

            def keep_initial_weights(*a, _orig=orig, **k):
                m = _orig(*a, **k)
                if int(os.environ.get("RANK", 0)) == 0:
                    inner = getattr(m, "module", m)
                    torch.save({n: v.detach().clone() for n, v in inner.state_dict().items()}, init_file)
                return m

            recipe.build_model = keep_initial_weights
        recipe.run()


def _run_our_recipe(tmp: str, extra: list[str] | None, phases: list[list[str]], transforms: list[dict]) -> None:
    from optimus_dl_b200.core import compose
    from optimus_dl_b200.core.config_utils import non_resolving_instantiate
    from optimus_dl_b200.core.registry import build
    import optimus_dl_b200.recipe.train  # noqa: F401

    data, init_file = _recipe_corpus(tmp), os.path.join(tmp, "init.pt")
    for phase in phases:
        cfg = compose.compose(os.path.join(ROOT, "configs", "train"), "train_llama_shakespeare",
                              _recipe_overrides(tmp, "ours", data, extra) + phase)
        cfg.model_transforms = [{"_name": "load_weights", "checkpoint_path": init_file}] + list(transforms)
        build("train_recipe", non_resolving_instantiate(cfg)).run()


def _compare_recipe_logs(tmp: str, tol: float) -> None:
    import glob

    def logs(which):
        out = {}
        for f in sorted(glob.glob(f"{tmp}/{which}/logs/**/*.jsonl", recursive=True)):
            for line in open(f):
                r = json.loads(line)
                out.setdefault((r["group"], r["step"]), {}).update({k: v for k, v in r.items() if k != "timestamp"})
        return out

    r, o = logs("ref"), logs("ours")
    assert set(r) == set(o), (sorted(r, key=str), sorted(o, key=str))
    assert ("train", 8) in r and ("eval/tinyshakespeare", 8) in r and ("init", 1) in r
    ours_only = {"optimizer_step_skipped", "model/num_params_total", "model/num_params_trainable"}
    for key in r:
        a, b = r[key], o[key]
        assert set(a) <= set(b) and set(b) - set(a) <= ours_only, (key, sorted(set(a) ^ set(b)))
        for k, v in a.items():
            if k.startswith("perf/") or k == "ms_spent_logging" or not isinstance(v, (int, float)):
                continue
            assert abs(v - b[k]) <= tol * max(1.0, abs(v)), (key, k, v, b[k])


def check_recipe(extra: list[str] | None = None, tol: float = 1e-5, phases: list[list[str]] | None = None) -> None:
    """The whole training recipe (8 iterations, evaluation every 4, checkpoints) from one composed config and the
    same initial weights: every number either side logs (loss, perplexity, accuracy, gradient norm, learning rate,
    token counts, metric-engine values; train and eval groups) agrees."""
    tmp = tempfile.mkdtemp()
    _run_reference_recipe(tmp, extra, phases or [[]], [])
    _run_our_recipe(tmp, extra, phases or [[]], [])
    _compare_recipe_logs(tmp, tol)


def check_recipe_ddp_side() -> None:
    """One side (``ref`` / ``ours`` / ``compare``) of the two-rank variant: each recipe runs under its own ``torchrun``
    with the ``ddp`` transform, in the directory named on the command line."""
    side, tmp = sys.argv[2], sys.argv[3]
    if side == "ref":
        _run_reference_recipe(tmp, None, [[]], [{"_name": "ddp"}])
    elif side == "ours":
        _run_our_recipe(tmp, None, [[]], [{"_name": "ddp"}])
    else:
        _compare_recipe_logs(tmp, 1e-5)


def check_generation() -> None:
    """The ``generation`` metric source: greedy, with an end-of-sequence token, and sampled (temperature, top-k,
    top-p) under the same torch seed give the same tokens, for a rotary, a learned-position and a sliding-window
    model (this package decodes with a key/value cache, the reference re-runs the prefix)."""
    from optimus_dl_b200.metrics.source import build_metric_source

    ref_build = importlib.import_module("optimus_dl.modules.metrics.source").build_metric_source
    for name in ("llama2", "gpt2", "olmo3"):
        ref, ours = _pair(MODELS[name])
        ref.eval(), ours.eval()
        for scfg in (dict(_name="generation", max_new_tokens=12), dict(_name="generation", max_new_tokens=12, eos_token_id=3),
                     dict(_name="generation", max_new_tokens=8, do_sample=True, temperature=0.8, top_k=5),
                     dict(_name="generation", max_new_tokens=8, do_sample=True, temperature=1.3, top_p=0.7)):
            x = torch.randint(0, 97, (3, 9))
            torch.manual_seed(1)
            a = ref_build(OmegaConf.create(scfg))({}, model=ref, batch={"input_ids": x.clone()})
            torch.manual_seed(1)
            b = build_metric_source(dict(scfg))({}, model=ours, batch={"input_ids": x.clone()})
            assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a), (name, scfg)


def check_metrics_recipe() -> None:
    """The metrics recipe (model from a config, criterion, one evaluation dataset, a source group and a bare metric)
    from the same weights: the same result keys and values, and the same logger group / file / step."""
    import glob

    import optimus_dl.recipe.metrics.base  # noqa: F401
    from optimus_dl.core.registry import build as ref_build
    from optimus_dl_b200.core import conf
    from optimus_dl_b200.core.config_utils import non_resolving_instantiate
    from optimus_dl_b200.core.registry import build
    import optimus_dl_b200.recipe.metrics  # noqa: F401

    tmp = tempfile.mkdtemp()
    data, init_file = os.path.join(tmp, "d.txt"), os.path.join(tmp, "init.pt")
    with open(data, "w") as f:
        f.write("".join(f"Line {i}: some text to score, number {i * i}.\n" for i in range(300)))

    def cfg(which):
        return {"_name": "base", "args": {},
                "common": {"name": "m", "seed": 42, "data_seed": 42, "output_path": f"{tmp}/{which}", "checkpoint_path": None,
                           "use_gpu": False, "max_iterations": 3, "distributed": {"tp_size": 1, "sharding_world_size": 1}},
                "model": {"_name": "llama2", "n_layer": 1, "n_head": 2, "n_embd": 32, "vocab_size": 264, "sequence_length": 64,
                          "multiple_of": 8},
                "criterion": {"_name": "cross_entropy"},
                "data": {"eval_datasets": {"txt": {"source": {"_name": "txt_lines", "file_link": data},
                                                   "transform": {"_name": "compose", "transforms": [
                                                       {"_name": "tokenize", "tokenizer_config": {"_name": "char_tokenize"},
                                                        "worker_cfg": {"num_workers": 0}},
                                                       {"_name": "chunk_tokens", "max_seq_len": 32},
                                                       {"_name": "flat_batcher", "batch_size": 4, "seq_len": 32},
                                                       {"_name": "to_device"}]}}}},
                "metrics": {"txt": [{"_name": "source_group", "prefix": "lm", "sources": {"lm": {"_name": "causal_lm"}},
                                     "metrics": [{"_name": "accuracy"}, {"_name": "perplexity"}, {"_name": "loss"}]},
                                    {"_name": "accuracy"}]},
                "model_transforms": [], "loggers": [{"_name": "jsonl", "output_dir": f"{tmp}/{which}/logs"}]}

    c = cfg("ref")
    for k in ("model_builder", "criterion_builder", "data_builder", "logger_manager", "checkpoint_manager", "evaluator"):
        c[k] = {"_name": "base"}
    rec = ref_build("metrics_recipe", OmegaConf.create(c))
    orig = rec.model_builder.build_model

    def keep(*a, **k):
        m = orig(*a, **k)
        torch.save(m.state_dict(), init_file)
        return m

    rec.model_builder.build_model = keep
    r = rec.run()
    c = cfg("ours")
    c["model_transforms"] = [{"_name": "load_weights", "checkpoint_path": init_file}]
    o = build("metrics_recipe", non_resolving_instantiate(conf.create(c))).run()
    assert sorted(r) == sorted(o) == ["metrics/txt"]
    a, b = r["metrics/txt"], o["metrics/txt"]
    assert set(a) == set(b) and "lm/perplexity_metric/perplexity" in a and "accuracy_metric/total" in a, sorted(set(a) ^ set(b))
    for k, v in a.items():
        if not k.startswith("perf/") and k != "ms_spent_logging" and isinstance(v, (int, float)):
            assert abs(v - b[k]) <= 1e-6 * max(1.0, abs(v)), (k, v, b[k])

    def logged(which):
        out = set()
        for f in glob.glob(f"{tmp}/{which}/logs/**/*.jsonl", recursive=True):
            out |= {(os.path.basename(f), json.loads(line)["group"], json.loads(line)["step"]) for line in open(f)}
        return out

    assert logged("ref") == logged("ours") == {("metrics_eval_metrics_txt.jsonl", "eval/metrics/txt", 0)}


def check_eval_adapter() -> None:
    """The lm_eval adapter in ``reference_scoring`` mode returns the reference adapter's numbers (log-likelihood of a
    continuation, greedy flag, rolling log-likelihood); the default mode follows the harness's conventions instead."""
    from types import SimpleNamespace

    import optimus_dl_b200.tokenizer as ot
    from optimus_dl_b200.eval.model import LLMBaselinesModel

    cfg = dict(MODELS["llama2"], vocab_size=264, sequence_length=128)
    ref_model, our_model = _pair(cfg)
    tcfg = {"_name": "char_tokenize"}
    r = R("eval.model").LLMBaselinesModel(ref_model.eval(), R("tokenizer").build_tokenizer(OmegaConf.create(tcfg)),
                                          OmegaConf.create(tcfg), device="cpu")
    o = LLMBaselinesModel(our_model.eval(), ot.build_tokenizer(dict(tcfg)), dict(tcfg), device="cpu", reference_scoring=True)
    reqs = [SimpleNamespace(args=("The quick brown", " fox jumps")), SimpleNamespace(args=("", "hello")),
            SimpleNamespace(args=("abc" * 30, "def" * 10))]
    for (a, ga), (b, gb) in zip(r.loglikelihood(reqs), o.loglikelihood(reqs)):
        assert abs(a - b) < 1e-3 and ga == gb, (a, b)
    rolling = [SimpleNamespace(args=("some longer text to roll over " * 3,)), SimpleNamespace(args=("x",))]
    assert all(abs(a - b) < 1e-3 for a, b in zip(r.loglikelihood_rolling(rolling), o.loglikelihood_rolling(rolling)))
    plain = LLMBaselinesModel(our_model.eval(), ot.build_tokenizer(dict(tcfg)), dict(tcfg), device="cpu")
    assert abs(plain.loglikelihood(reqs[:1])[0][0] - o.loglikelihood(reqs[:1])[0][0]) > 1e-3      # a different convention


def check_optimizer_routing() -> None:
    """Which parameters each sub-optimizer of ``muon`` and of a ``composite`` configuration receives, with which
    group settings; the composite then takes the same steps from the same gradients and exports the same state keys."""
    import optimus_dl_b200.optim as oo

    def routing(opt, model):
        names = {id(p): n for n, p in model.named_parameters()}
        return {f"{k}:{type(o).__name__}": [(sorted(names[id(p)] for p in g["params"]),
                                             {a: b for a, b in g.items() if a in ("lr", "weight_decay")}) for g in o.param_groups]
                for k, o in opt.optimizers.items()}

    composite = dict(_name="composite", optimizers={
        "a_attn": {"params_regexp": ".*attn.*", "optimizer_config": {"_name": "adamw", "lr": 1e-3}},
        "b_mlp": {"params_regexp": ".*mlp\\.w.*", "optimizer_config": {"_name": "soap", "lr": 3e-3}},
        "z_rest": {"params_regexp": None, "optimizer_config": {"_name": "adamw", "lr": 2e-3, "weight_decay": 0.0}}})
    for ocfg in (dict(_name="muon", lr=1e-2, weight_decay=0.1), composite):
        ref, ours = _pair(MODELS["llama2"])
        ro = R("optim").build_optimizer(OmegaConf.create(ocfg), params=ref.make_parameter_groups())
        o = oo.build_optimizer(dict(ocfg), params=ours.make_parameter_groups())
        assert routing(ro, ref) == routing(o, ours), ocfg["_name"]
        if ocfg["_name"] != "composite":
            continue
        g = torch.Generator().manual_seed(1)
        for _ in range(3):
            x = torch.randint(0, 97, (8, 32), generator=g)
            ref(x)["logits"].float().logsumexp(-1).mean().backward()
            for p, q in zip(ref.parameters(), ours.parameters()):
                q.grad = p.grad.clone()
            ro.step(), o.step(), ro.zero_grad(), o.zero_grad()
        assert max((p - q).abs().max().item() for p, q in zip(ref.parameters(), ours.parameters())) < 1e-4
        assert sorted(ro.state_dict()) == sorted(o.state_dict())


def check_schedules() -> None:
    """Every learning-rate schedule over its whole length, two parameter groups, two run lengths: the same rate at
    every step (about 200 configurations: all WSD decay shapes, warm-up lengths, final factors, piecewise-linear
    waypoints, a lowered cool-down start, cosine annealing, linear warm-up)."""
    import itertools

    import optimus_dl_b200.lr_scheduler as ol

    def opt():
        return torch.optim.SGD([{"params": [torch.nn.Parameter(torch.zeros(1))], "lr": 0.3},
                                {"params": [torch.nn.Parameter(torch.zeros(1))], "lr": 0.01}], lr=0.1)

    cfgs = [dict(_name="wsd", warmup_steps=w, fract_decay=fd, decay_type=dt, final_lr_factor=f, init_div_factor=idv, **extra)
            for w, fd, dt, f, idv in itertools.product((0, 7), (0.1, 0.5), ("linear", "cosine", "exp", "miror_cosine", "square", "sqrt"),
                                                       (0.0, 0.1), (25, 100))
            for extra in ({}, {"sqrt_power": 0.3} if dt == "sqrt" else {})]
    cfgs += [dict(_name="wsd", warmup_steps=5, fract_decay=0.4, decay_type="linear_pw", linear_pw_subdivisions=[0.5, 0.2], final_lr_factor=0.05),
             dict(_name="wsd", warmup_steps=None, warmup_steps_fraction=0.1, fract_decay=0.3, cooldown_start_lr_factor=0.7),
             dict(_name="cosine_annealing", eta_min=0.01), dict(_name="cosine_annealing", T_max=13),
             dict(_name="linear_warmup", warmup_steps=9, start_lr=0.001), dict(_name="linear_warmup", warmup_steps=0)]
    for c in cfgs:
        for iters in (40, 101):
            a, b = opt(), opt()
            ra = R("lr_scheduler").build_lr_scheduler(OmegaConf.create(c), optimizer=a, iterations=iters)
            rb = ol.build_lr_scheduler(dict(c), optimizer=b, iterations=iters)
            for step in range(iters + 5):
                la, lb = [g["lr"] for g in a.param_groups], [g["lr"] for g in b.param_groups]
                assert all(abs(x - y) <= 1e-12 * max(1.0, abs(x)) for x, y in zip(la, lb)), (c, iters, step, la, lb)
                a.step(), b.step(), ra.step(), rb.step()
            assert ra.state_dict().keys() == rb.state_dict().keys(), c


def check_pretokenize() -> None:
    """Both data-preparation recipes on one local corpus (parquet and JSON-lines files, several output shards, two
    tokenizer processes): the same shard files, byte for byte, and the same index. The reference lists and fetches
    files through the hub client; here those two calls are pointed at the local directory, and its worker processes
    are forked instead of spawned so that they see the same substitution."""
    import hashlib
    import multiprocessing as mp
    from unittest.mock import patch

    import pyarrow as pa
    import pyarrow.parquet as pq

    from optimus_dl_b200.core import conf
    from optimus_dl_b200.recipe.pretokenize import DataPrepConfig, DataPrepRecipe

    tmp = tempfile.mkdtemp()
    src = os.path.join(tmp, "repo")
    os.makedirs(os.path.join(src, "data"))
    rng = np.random.default_rng(0)
    for f in range(3):
        texts = ["doc %d-%d " % (f, i) + "lorem ipsum " * int(rng.integers(1, 40)) for i in range(1500)]
        pq.write_table(pa.table({"text": texts}), os.path.join(src, "data", f"train-{f:05d}-of-00003.parquet"))
    with open(os.path.join(src, "data", "train_extra.jsonl"), "w") as fh:
        for i in range(50):
            fh.write(json.dumps({"text": f"json line {i} " + "x y z " * (i % 9)}) + "\n")

    def cfg(out):
        return {"dataset": {"repo_id": src, "split": "train", "config_name": None, "cache_dir": None, "file_pattern": None},
                "processing": {"shard_size_mb": 1, "shuffle_buffer_size": 500, "text_column": "text", "seed": 42,
                               "dtype": "uint16", "num_proc": 2},
                "output": {"dir": out, "name": "shard"}, "tokenizer": {"_name": "char_tokenize"}}

    def digest(d):
        out = {}
        for f in sorted(os.listdir(d)):
            if f.endswith(".npy"):
                a = np.load(os.path.join(d, f))
                out[f] = (a.dtype.str, a.shape, hashlib.sha1(a.tobytes()).hexdigest())
            elif f == "index.json":
                j = json.load(open(os.path.join(d, f)))
                out[f] = (j["files"], j["total_tokens"])
        return out

    DataPrepRecipe(conf.merge(conf.create(DataPrepConfig()), conf.create(cfg(os.path.join(tmp, "ours"))))).run()
    rr = importlib.import_module("optimus_dl.recipe.pretokenize.recipe")
    rs = importlib.import_module("optimus_dl.recipe.pretokenize.source")
    rp = importlib.import_module("optimus_dl.recipe.pretokenize.processor")
    rc = importlib.import_module("optimus_dl.recipe.pretokenize.config")

    def list_files(repo_id, repo_type=None, **_):
        return sorted(os.path.relpath(os.path.join(r, f), repo_id) for r, _d, fs in os.walk(repo_id) for f in fs)

    def download(repo_id, filename, repo_type=None, cache_dir=None, **_):
        return os.path.join(repo_id, filename)

    get_context = mp.get_context
    with patch.object(rs, "list_repo_files", list_files), patch.object(rs, "hf_hub_download", download), \
            patch.object(rp, "hf_hub_download", download), patch.object(mp, "get_context", lambda method=None: get_context("fork")):
        rr.DataPrepRecipe(OmegaConf.merge(OmegaConf.structured(rc.DataPrepConfig), OmegaConf.create(cfg(os.path.join(tmp, "ref"))))).run()
    a, b = digest(os.path.join(tmp, "ref")), digest(os.path.join(tmp, "ours"))
    assert len(a) >= 5 and a == b, [k for k in set(a) | set(b) if a.get(k) != b.get(k)]


if __name__ == "__main__":
    name = sys.argv[1]
    globals()["check_" + name]()
    print("DIFF_OK", name, flush=True)
