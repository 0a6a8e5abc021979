"""Composite, Muon and SOAP optimizers (CPU)."""

import copy

import pytest
import torch
import torch.nn as nn

from optimus_dl_b200.core import conf
from optimus_dl_b200.optim import build_optimizer
from optimus_dl_b200.optim.composite import CompositeOptimizer, get_subgroup
from optimus_dl_b200.optim.muon import Muon, newton_schulz
from optimus_dl_b200.optim.soap import SOAP, merged_shape


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 8))


def _named(m):
    return [(n, p) for n, p in m.named_parameters()]


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in [(32, 64), (64, 32), (48, 48)]:
        g = torch.randn(*shape)
        o = newton_schulz(g, steps=10).float()
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.3 and s.min() > 0.5, (shape, s.min(), s.max())
        u, _, vh = torch.linalg.svd(g, full_matrices=False)
        assert torch.nn.functional.cosine_similarity((u @ vh).flatten(), o.flatten(), dim=0) > 0.9


def test_muon_matches_torch_muon():
    if not hasattr(torch.optim, "Muon"):
        pytest.skip("torch.optim.Muon not available")
    torch.manual_seed(0)
    w1 = nn.Parameter(torch.randn(24, 40))
    w2 = nn.Parameter(w1.detach().clone())
    ours, ref = Muon([w1], lr=0.02), torch.optim.Muon([w2], lr=0.02)
    for i in range(3):
        g = torch.randn(24, 40, generator=torch.Generator().manual_seed(i))
        w1.grad, w2.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    assert torch.allclose(w1, w2, atol=2e-2), (w1 - w2).abs().max()


def test_muon_factory_builds_composite_and_trains():
    net = _net()
    cfg = conf.create({"_name": "muon", "lr": 0.02, "weight_decay": 0.0})
    opt = build_optimizer(cfg, params=_named(net))
    assert isinstance(opt, CompositeOptimizer) and set(opt.optimizers) == {"muon", "support"}
    names = {g["composite_optimizer_name"] for g in opt.param_groups}
    assert names == {"muon", "support"}
    x, y = torch.randn(64, 16), torch.randn(64, 8)
    first = None
    for _ in range(40):
        opt.zero_grad()
        loss = (net(x) - y).pow(2).mean()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.7 * first


def test_composite_routing_state_roundtrip_and_lr_alias():
    net = _net()
    cfg = conf.create({"_name": "composite", "optimizers": {
        "a": {"params_regexp": r"0\..*", "optimizer_config": {"_name": "adamw", "lr": 1e-2, "fused": False}},
        "rest": {"params_regexp": None, "optimizer_config": {"_name": "soap", "lr": 1e-2}}}})
    opt = build_optimizer(cfg, params=_named(net))
    assert [g["composite_optimizer_path"] for g in opt.param_groups] == [["a"], ["rest"]]
    x, y = torch.randn(32, 16), torch.randn(32, 8)
    for _ in range(3):
        opt.zero_grad()
        (net(x) - y).pow(2).mean().backward()
        opt.step()
    # a scheduler writing into the composite's groups must reach the children
    opt.param_groups[0]["lr"] = 5e-3
    assert opt.optimizers["a"].param_groups[0]["lr"] == 5e-3
    sd = copy.deepcopy(opt.state_dict())
    net2 = _net()
    opt2 = build_optimizer(cfg, params=_named(net2))
    opt2.load_state_dict(sd)
    net2.load_state_dict(net.state_dict())
    assert opt2.optimizers["a"].param_groups[0] is opt2.param_groups[0]
    assert opt2.optimizers["a"].state is opt2.state
    for o, n in ((opt, net), (opt2, net2)):
        o.zero_grad()
        (n(x) - y).pow(2).mean().backward()
        o.step()
    for p, q in zip(net.parameters(), net2.parameters()):
        assert torch.allclose(p, q, atol=1e-6)


def test_composite_errors():
    net = _net()
    with pytest.raises(ValueError, match="did not match"):
        build_optimizer(conf.create({"_name": "composite", "optimizers": {
            "a": {"params_regexp": "nothing", "optimizer_config": {"_name": "adamw"}}}}), params=_named(net))
    with pytest.raises(ValueError, match="not matched by any"):
        build_optimizer(conf.create({"_name": "composite", "optimizers": {
            "a": {"params_regexp": r"0\..*", "optimizer_config": {"_name": "adamw", "fused": False}}}}), params=_named(net))
    with pytest.raises(ValueError):
        get_subgroup(list(net.parameters()), lambda n, p: True)


def test_soap_descends_and_merges_dims():
    assert merged_shape((4, 8, 3, 3), 100) == [96, 3]
    assert merged_shape((50000, 64), 10000) == [50000, 64]
    torch.manual_seed(0)
    w = nn.Parameter(torch.randn(20, 12))
    b = nn.Parameter(torch.zeros(20))
    x = torch.randn(256, 12)
    target = x @ torch.randn(12, 20)
    opt = SOAP([w, b], lr=0.05, weight_decay=0.0, precondition_frequency=5)
    losses = []
    for _ in range(200):
        opt.zero_grad()
        loss = ((x @ w.t() + b) - target).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.05 * losses[0]
    q = opt.state[w]["Q"]
    assert torch.allclose(q[0].t() @ q[0], torch.eye(20), atol=1e-4)
    assert opt.state[b]["GG"] == [None]


def test_soap_is_adam_in_the_eigenbasis_of_the_gradient_statistics():
    """The update written out for a matrix (optimus_dl/modules/optim/soap.py:157-279): statistics ``L = EMA(G G^T)``,
    ``R = EMA(G^T G)`` with eigenvectors in the COLUMNS of ``Q_L``, ``Q_R``; Adam runs on ``Q_L^T G Q_R`` and its
    direction returns as ``Q_L (.) Q_R^T``; the first call only seeds the statistics; they are updated after each
    step and their bases refreshed by one QR power iteration every ``precondition_frequency`` steps."""
    torch.manual_seed(3)
    lr, b1, b2, eps, wd, freq = 0.02, 0.9, 0.95, 1e-8, 0.1, 3
    # square, so that both statistics have full rank from the first gradient on (in a null space the eigenvectors
    # are arbitrary and Adam's m / sqrt(v) turns rounding noise into visible steps)
    w = nn.Parameter(torch.randn(6, 6))
    opt = SOAP([w], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd, precondition_frequency=freq)
    p = w.detach().clone()
    grads = [torch.randn(6, 6) for _ in range(6)]

    def eig(m):
        return torch.linalg.eigh(m + 1e-30 * torch.eye(m.shape[0]))[1].flip(1)

    L = (1 - b2) * grads[0] @ grads[0].t()
    Rm = (1 - b2) * grads[0].t() @ grads[0]
    QL, QR = eig(L), eig(Rm)
    m, v = torch.zeros(6, 6), torch.zeros(6, 6)
    w.grad = grads[0]
    opt.step()
    assert torch.equal(w.detach(), p)                            # the first call moves nothing
    for t, g in enumerate(grads[1:], start=1):
        g_rot = QL.t() @ g @ QR
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g_rot * g_rot
        direction = QL @ ((QL.t() @ m @ QR) / (v.sqrt() + eps)) @ QR.t()
        p = p - lr * ((1 - b2 ** t) ** 0.5) / (1 - b1 ** t) * direction
        p = p - lr * wd * p
        L = b2 * L + (1 - b2) * g @ g.t()
        Rm = b2 * Rm + (1 - b2) * g.t() @ g
        if t % freq == 0:
            for axis, (stat, q) in enumerate(((L, QL), (Rm, QR))):
                order = torch.argsort(torch.diag(q.t() @ stat @ q), descending=True)
                v = v.index_select(axis, order)
                qn = torch.linalg.qr(stat @ q[:, order])[0]
                if axis == 0:
                    QL = qn
                else:
                    QR = qn
        w.grad = g
        opt.step()
        assert torch.allclose(w.detach(), p, atol=1e-4), (t, (w.detach() - p).abs().max().item())
    # a rotation by Q instead of Q^T is also orthogonal and also descends, but it is a different optimizer
    assert not torch.allclose(QL, QL.t(), atol=1e-2)


# ---------------------------------------------------------------------- adamw factory and the optimizer builder
def test_adamw_factory_accepts_named_groups_and_matches_torch_on_cpu():
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.optim import build_optimizer

    torch.manual_seed(0)
    cfg = dict(_name="llama2", n_layer=1, n_head=2, n_kv_head=1, n_embd=32, vocab_size=53, sequence_length=16, multiple_of=8)
    a, b = build_model(cfg), build_model(cfg)
    b.load_state_dict(a.state_dict())
    groups = a.make_parameter_groups()
    assert all(isinstance(p, tuple) and isinstance(p[0], str) for g in groups for p in g["params"])   # named parameters
    decay = {n for n, _ in groups[0]["params"]}
    assert "transformer.h.0.attn.wq.weight" in decay and not any("ln_" in n for n in decay)
    opt = build_optimizer({"_name": "adamw", "lr": 1e-2, "betas": [0.9, 0.95], "weight_decay": 0.1}, params=groups)
    wd = sorted(g["weight_decay"] for g in opt.param_groups)
    assert wd == [0.0, 0.1] and all(g["lr"] == 1e-2 and tuple(g["betas"]) == (0.9, 0.95) for g in opt.param_groups)
    names = dict(b.named_parameters())
    ref = torch.optim.AdamW([{"params": [names[n] for n, _ in g["params"]], "weight_decay": g.get("weight_decay", 0.1)}
                             for g in b.make_parameter_groups()], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for step in range(3):
        x = torch.randint(0, 53, (2, 8), generator=torch.Generator().manual_seed(step))
        for model, o in ((a, opt), (b, ref)):
            o.zero_grad()
            model(x)["logits"].float().logsumexp(-1).mean().backward()
            o.step()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-6), n
    with pytest.raises(Exception):
        build_optimizer({"_name": "adamw", "learning_rate": 1.0}, params=groups)      # strict config: unknown key


def test_optimizer_builder_counts_parameters_and_passes_the_clip_value():
    from optimus_dl_b200.core import conf
    from optimus_dl_b200.metrics import base as mb
    from optimus_dl_b200.recipe.train.builders.optimizer_builder import OptimizerBuilder

    lin = torch.nn.Linear(4, 3)
    cfg = conf.create({"optimizer": {"_name": "adamw", "lr": 0.5}, "clip_grad_norm": 2.0})
    with mb.meters_group("init", log_freq=1):
        opt = OptimizerBuilder(optimization_config=cfg).build_optimizer(list(lin.named_parameters()))
        assert mb.compute_meters("init")["optimized_params"] == 15
    assert opt.param_groups[0]["lr"] == 0.5 and len(opt.param_groups[0]["params"]) == 2


def test_composite_accepts_config_dataclasses_and_a_catch_all_entry():
    """``CompositeOptimizerConfigEntry`` instances as entries (optimus_dl/modules/optim/composite.py), ``params_regexp:
    None`` as "everything that is left", and live ``param_groups`` of the sub-optimizers."""
    import torch.nn as nn

    from optimus_dl_b200.optim.composite import (CompositeOptimizer, CompositeOptimizerConfig, CompositeOptimizerConfigEntry,
                                                 make_composite_optimizer)

    for weight_cfg in ({"_name": "adamw", "lr": 1e-2}, {"_name": "muon", "lr": 1e-2}):
        model = nn.Linear(10, 5)
        cfg = CompositeOptimizerConfig(optimizers={
            "weight_opt": CompositeOptimizerConfigEntry(params_regexp=".*weight", optimizer_config=weight_cfg),
            "bias_opt": CompositeOptimizerConfigEntry(params_regexp=".*bias", optimizer_config={"_name": "adamw", "lr": 1e-3})})
        opt = make_composite_optimizer(cfg, params=model.named_parameters())
        assert isinstance(opt, CompositeOptimizer) and set(opt.optimizers) == {"weight_opt", "bias_opt"}
        assert opt.optimizers["weight_opt"].param_groups[0]["lr"] == 1e-2 and opt.optimizers["bias_opt"].param_groups[0]["lr"] == 1e-3
        for group in opt.param_groups:
            if group["composite_optimizer_name"] == "weight_opt":
                group["lr"] = 5e-2
        assert opt.optimizers["weight_opt"].param_groups[0]["lr"] == 5e-2      # the same dict, not a copy
        model(torch.randn(3, 10)).sum().backward()
        before = model.weight.detach().clone()
        opt.step()
        assert not torch.equal(before, model.weight)
    model = nn.Linear(10, 5)
    rest = make_composite_optimizer(CompositeOptimizerConfig(optimizers={
        "w": CompositeOptimizerConfigEntry(params_regexp=".*weight", optimizer_config={"_name": "adamw", "lr": 1e-2}),
        "rest": CompositeOptimizerConfigEntry(params_regexp=None, optimizer_config={"_name": "adamw", "lr": 1e-3})}),
        params=model.named_parameters())
    assert len(rest.optimizers["rest"].param_groups[0]["params"]) == 1


def test_muon_and_soap_refuse_parameters_of_the_sharding_engine():
    import pytest
    import torch

    from optimus_dl_b200.optim.muon import Muon
    from optimus_dl_b200.optim.soap import SOAP

    p = torch.nn.Parameter(torch.zeros(4, 4))
    p._shard_group = object()       # what the fully_shard transform leaves on a parameter
    with pytest.raises(ValueError, match="fully_shard"):
        Muon([p])
    with pytest.raises(ValueError, match="fully_shard"):
        SOAP([p])
