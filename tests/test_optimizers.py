"""Optimizer classes: parity with the reference package on CPU, behaviour checks, and CUDA runs
compared with the CPU runs of the same code."""
import copy

import pytest
import torch

import dion_b200

SHAPES = ((64, 128), (64, 128), (128, 64), (4, 32, 48))


def _run(cls, kw, device="cpu", steps=3, shapes=SHAPES, scalar="adamw", pre=None):
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(*s).to(device)) for s in shapes]
    v = torch.nn.Parameter(torch.randn(128).to(device))
    opt = cls([dict(params=ps), dict(params=[v], algorithm=scalar)], lr=0.02, **kw)
    if pre is not None:
        pre(opt, ps)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        for p in ps + [v]:
            p.grad = torch.randn(p.shape, generator=g).to(device)
        opt.step()
    return [p.detach().float().cpu() for p in ps + [v]], opt


MEGABATCH = [
    ("Muon", dict(nesterov=True)),
    ("Muon", dict(use_polar_express=False, cautious_wd=True, adjust_lr="rms_norm")),
    ("NorMuon", dict()),
    ("NorMuon", dict(nesterov=True, cautious_wd=True)),
    ("Dion2", dict()),
    ("Dion2", dict(fraction=0.5, ef_decay=0.9)),
    ("NorDion2", dict()),
    ("NorDion2", dict(fraction=0.5)),
    ("Muon", dict(mu=0.8, betas=(0.8, 0.9), epsilon=1e-6)),
    ("NorMuon", dict(muon_beta2=0.9, use_polar_express=False)),
    ("Dion2", dict(selection_scope="global", fraction=0.25)),
    ("NorDion2", dict(fraction=0.25, use_polar_express=False)),
]


@pytest.mark.parametrize("name,kw", MEGABATCH)
def test_megabatch_parity_with_reference(ref_dion, name, kw):
    a, oa = _run(getattr(ref_dion, name), kw)
    b, ob = _run(getattr(dion_b200, name), kw)
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 2e-4
    sa, sb = oa.state_dict(), ob.state_dict()
    assert sa["param_groups"] == sb["param_groups"]
    for k in sa["state"]:
        assert set(sa["state"][k]) == set(sb["state"][k])
        for kk, val in sa["state"][k].items():
            assert val.shape == sb["state"][k][kk].shape and val.dtype == sb["state"][k][kk].dtype


def test_flatten_parity_with_reference_single_parameters(ref_dion):
    """``flatten=True`` folds a >2-D parameter to [shape[0], rest]; 2-D parameters are unchanged.
    Compared one parameter per shape, where the reference applies exactly this meaning."""
    kw = dict(flatten=True, adjust_lr="spectral_norm", weight_decay=0.0, use_polar_express=False)
    shapes = ((64, 128), (128, 64), (4, 32, 48), (8, 6, 3, 3))
    a, _ = _run(ref_dion.Muon, kw, shapes=shapes)
    b, _ = _run(dion_b200.Muon, kw, shapes=shapes)
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 2e-4


def _same_q_init(opt, ps):
    torch.manual_seed(5)
    for p in ps:
        if hasattr(opt, "_get_or_initialize_state"):
            try:
                opt._get_or_initialize_state(p, opt.param_groups[0])
                continue
            except TypeError:
                pass
        g = opt.param_groups[0]
        opt._init_opt_state_dion(p, opt.state[p], g["rank_fraction"], g["rank_multiple_of"])


@pytest.mark.parametrize("name,kw", [
    ("Dion", dict()), ("Dion", dict(rank_fraction=0.25)),
    ("Dion", dict(rank_fraction=0.5, rank_multiple_of=8)),
    ("DionReference", dict()), ("DionReference", dict(rank_fraction=0.25, qr_method="qr")),
    ("DionReference", dict(rank_fraction=0.5, qr_method="cqr", cqr_warmup_steps=2, power_iters=2)),
])
def test_dion_parity_with_reference(ref_dion, name, kw):
    shapes = ((64, 128), (64, 128), (128, 64), (96, 96))
    a, _ = _run(getattr(ref_dion, name), kw, shapes=shapes, steps=4, scalar="lion", pre=_same_q_init)
    b, _ = _run(getattr(dion_b200, name), kw, shapes=shapes, steps=4, scalar="lion", pre=_same_q_init)
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 1e-5


def test_dion_mixed_precision_states_and_parity(ref_dion):
    """``DionMixedPrecisionConfig``: bf16 momentum and Q, fp32 AdamW variance on fp32 weights -
    the state tensors take the configured types and the run follows the reference's with the
    same configuration (reference README: "Mixed Precision Dion")."""
    shapes = ((64, 128), (128, 64), (96, 96))

    def run(pkg, scalar):
        mp = pkg.DionMixedPrecisionConfig(momentum_dtype=torch.bfloat16, Q_dtype=torch.bfloat16,
                                          variance_dtype=torch.float32)
        return _run(pkg.Dion, dict(rank_fraction=0.25, mixed_precision_config=mp), shapes=shapes,
                    steps=4, scalar=scalar, pre=_same_q_init)

    # The reference's AdamW path rejects momentum and variance of different types, so the
    # side-by-side run uses Lion for the vector; AdamW with mixed types is checked on ours alone.
    ours, opt = run(dion_b200, "lion")
    theirs, _ = run(ref_dion, "lion")
    matrix, vector = opt.param_groups[0]["params"][0], opt.param_groups[1]["params"][0]
    assert opt.state[matrix]["momentum"].dtype == torch.bfloat16
    assert opt.state[matrix]["Q"].dtype == torch.bfloat16
    assert opt.state[vector]["momentum"].dtype == torch.bfloat16
    for x, y in zip(ours, theirs):
        assert (x - y).abs().max().item() < 2e-3     # bf16 state: rounding order differs slightly
    full, _ = _run(dion_b200.Dion, dict(rank_fraction=0.25), shapes=shapes, steps=4,
                   scalar="lion", pre=_same_q_init)
    for x, y in zip(ours, full):
        assert (x - y).abs().max().item() < 5e-2     # and stays close to the fp32-state run
    adam, opt = run(dion_b200, "adamw")
    vector = opt.param_groups[1]["params"][0]
    assert opt.state[vector]["variance"].dtype == torch.float32
    assert opt.state[vector]["momentum"].dtype == torch.bfloat16
    assert all(torch.isfinite(t).all() for t in adam)


def test_simple_and_muon_reference_parity(ref_dion):
    shapes = ((64, 128), (128, 64))
    for name, kw in (("DionSimple", dict(rank=16)), ("MuonReference", dict())):
        torch.manual_seed(3)
        a, _ = _run(getattr(ref_dion, name), kw, shapes=shapes)
        torch.manual_seed(3)
        b, _ = _run(getattr(dion_b200, name), kw, shapes=shapes)
        for x, y in zip(a, b):
            assert (x - y).abs().max().item() < 1e-5


def test_dion3_is_nordion2():
    assert dion_b200.Dion3 is dion_b200.NorDion2
    p = torch.nn.Parameter(torch.randn(8, 8))
    assert dion_b200.Dion3([p]).param_groups[0]["algorithm"] == "nordion2"


@pytest.mark.parametrize("name", ["Muon", "NorMuon", "Dion2", "NorDion2"])
def test_state_prepopulated_and_resumable(name):
    cls = getattr(dion_b200, name)
    ps = [torch.nn.Parameter(torch.randn(16, 32)) for _ in range(2)]
    v = torch.nn.Parameter(torch.randn(7))
    frozen = torch.nn.Parameter(torch.randn(16, 32))  # never gets a gradient
    opt = cls([dict(params=ps + [frozen]), dict(params=[v], algorithm="adamw")], lr=0.01)
    sd = opt.state_dict()
    assert len(sd["state"]) == 4
    assert "momentum" in sd["state"][0] and "step_dev" in sd["state"][3]
    assert isinstance(sd["param_groups"][0]["lr"], float)
    before = frozen.detach().clone()
    for p in ps + [v]:
        p.grad = torch.randn_like(p)
    opt.step()
    assert torch.equal(frozen, before)
    opt2 = cls([dict(params=ps + [frozen]), dict(params=[v], algorithm="adamw")], lr=0.5)
    opt2.load_state_dict(copy.deepcopy(opt.state_dict()))
    assert float(opt2.param_groups[0]["lr"]) == pytest.approx(0.01)
    assert isinstance(opt2.param_groups[0]["lr"], torch.Tensor)
    assert opt2.state[v]["step_dev"].dtype == torch.float32
    assert float(opt2.state[v]["step_dev"]) == 1.0
    late = torch.nn.Parameter(torch.randn(4, 4))
    opt2.add_param_group(dict(params=[late]))
    assert "momentum" in opt2.state[late]


def test_lr_tensor_identity_and_scheduler():
    p = torch.nn.Parameter(torch.randn(8, 8))
    opt = dion_b200.Muon([p], lr=0.1)
    lr_t = opt.param_groups[0]["lr"]
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 0.5 ** s)
    p.grad = torch.randn_like(p)
    opt.step()
    sched.step()
    assert opt.param_groups[0]["lr"] is lr_t and float(lr_t) == pytest.approx(0.05)
    opt.param_groups[0]["lr"] = 0.3  # hand-rolled schedule assigns a float
    opt.step()
    assert opt.param_groups[0]["lr"] is lr_t and float(lr_t) == pytest.approx(0.3)


def test_validation_errors():
    p = torch.nn.Parameter(torch.randn(8, 8))
    with pytest.raises(ValueError):
        dion_b200.Muon([p], lr=-1)
    with pytest.raises(ValueError):
        dion_b200.Dion2([p], fraction=0.0)
    with pytest.raises(ValueError):
        dion_b200.Dion2([p], selection_scope="x")
    with pytest.raises(ValueError):
        dion_b200.Muon([p], adjust_lr="bad")
    with pytest.raises(TypeError):
        dion_b200.Muon([p], distributed_mesh="mesh")
    with pytest.raises(ValueError):
        dion_b200.Dion([p], power_iters=2)
    opt = dion_b200.Muon([dict(params=[p], algorithm="sgd")])
    p.grad = torch.randn_like(p)
    with pytest.raises(ValueError):
        opt.step()


def test_num_heads_matches_3d_parameter():
    torch.manual_seed(0)
    w = torch.randn(4 * 16, 32)
    g = torch.randn(4 * 16, 32)
    for name in ("Muon", "NorMuon", "Dion2", "NorDion2"):
        cls = getattr(dion_b200, name)
        a = torch.nn.Parameter(w.clone())
        b = torch.nn.Parameter(w.clone().view(4, 16, 32))
        oa = cls([dict(params=[a], num_heads=4)], lr=0.02)
        ob = cls([dict(params=[b])], lr=0.02)
        for _ in range(2):
            a.grad, b.grad = g.clone(), g.clone().view(4, 16, 32)
            oa.step()
            ob.step()
        assert (a.view(4, 16, 32) - b).abs().max().item() < 1e-6, name


def test_split_sizes_matches_separate_parameters():
    torch.manual_seed(0)
    sizes = (32, 16, 16)
    w = torch.randn(sum(sizes), 48)
    g = torch.randn(sum(sizes), 48)
    for name in ("Muon", "NorMuon"):
        cls = getattr(dion_b200, name)
        fused = torch.nn.Parameter(w.clone())
        parts = [torch.nn.Parameter(t.clone()) for t in w.split(list(sizes))]
        of = cls([dict(params=[fused], split_sizes=sizes)], lr=0.02)
        op = cls([dict(params=parts)], lr=0.02)
        for _ in range(2):
            fused.grad = g.clone()
            for p, gp in zip(parts, g.split(list(sizes))):
                p.grad = gp.clone()
            of.step()
            op.step()
        assert (fused - torch.cat([p.detach() for p in parts])).abs().max().item() < 2e-2, name
    with pytest.raises(NotImplementedError):
        p = torch.nn.Parameter(w.clone())
        p.grad = g.clone()
        dion_b200.Dion2([dict(params=[p], split_sizes=sizes)]).step()


def test_global_scope_k_uses_true_size():
    from dion_b200.optim.dion2 import make_select_and_orthogonalize
    ident = lambda X, epsilon=None: X  # noqa: E731
    f = make_select_and_orthogonalize(ident, 0.25, -2, global_select_size=18)
    X = torch.zeros(1, 24, 8)
    X[0, :18] = torch.arange(1, 19).float()[:, None]
    out = f(X)
    assert (out.abs().sum(-1) > 0).sum().item() == 5  # ceil(0.25 * 18), not ceil(0.25 * 24)


@pytest.mark.gpu
@pytest.mark.parametrize("name,kw", MEGABATCH + [("Dion", dict(rank_fraction=0.25))])
def test_cuda_matches_cpu(name, kw):
    from dion_b200.ops.gemm import check_status
    shapes = ((64, 128), (64, 128), (128, 64), (4, 32, 48)) if name != "Dion" else \
        ((64, 128), (64, 128), (128, 64))
    pre = _same_q_init if name == "Dion" else None
    a, _ = _run(getattr(dion_b200, name), kw, "cpu", shapes=shapes, pre=pre)
    if name == "Dion":
        def pre(opt, ps):  # identical Q on both devices
            gen = torch.Generator().manual_seed(5)
            for p in ps:
                st = opt._get_or_initialize_state(p, opt.param_groups[0])
                st["Q"].copy_(torch.randn(st["Q"].shape, generator=gen).to(st["Q"].device))
        a, _ = _run(getattr(dion_b200, name), kw, "cpu", shapes=shapes, pre=pre)
    b, _ = _run(getattr(dion_b200, name), kw, "cuda", shapes=shapes, pre=pre)
    torch.cuda.synchronize()
    check_status()
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 5e-3  # lr * bf16 Newton-Schulz differences


@pytest.mark.parametrize("name", ["Muon", "NorMuon", "Dion2", "NorDion2", "Dion3", "Dion",
                                  "DionReference", "DionSimple", "MuonReference",
                                  "CudaGraphOptimizer"])
def test_constructor_signatures_match_the_reference(ref_dion, name):
    """Same argument names, order and default values, so call sites written for the reference
    construct these classes unchanged."""
    import inspect
    if name == "CudaGraphOptimizer":
        from dion.cuda_graph import CudaGraphOptimizer as theirs
    else:
        theirs = getattr(ref_dion, name)
    ours = getattr(dion_b200, name)
    a = inspect.signature(theirs.__init__).parameters
    b = inspect.signature(ours.__init__).parameters
    assert list(a) == list(b)
    for key in a:
        if not callable(a[key].default):
            assert a[key].default == b[key].default, key
        assert a[key].kind == b[key].kind, key
