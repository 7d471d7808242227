"""Behaviour every optimizer class must show on any device (run here on CPU): parameters move,
identical runs agree bit for bit, mixed parameter groups and missing gradients are handled,
bad arguments are rejected."""
import pytest
import torch

import dion_b200


def _make(seed=0):
    torch.manual_seed(seed)
    mats = [torch.nn.Parameter(torch.randn(32, 48) * 0.1), torch.nn.Parameter(torch.randn(48, 32) * 0.1),
            torch.nn.Parameter(torch.randn(32, 32) * 0.1)]
    vecs = [torch.nn.Parameter(torch.randn(48)), torch.nn.Parameter(torch.randn(32))]
    return mats, vecs


FACTORIES = {
    "muon": lambda g: dion_b200.Muon(g, lr=0.02, mu=0.9, weight_decay=0.01),
    "muon_nesterov_pe": lambda g: dion_b200.Muon(g, lr=0.02, nesterov=True, use_polar_express=True),
    "normuon": lambda g: dion_b200.NorMuon(g, lr=0.02),
    "dion2": lambda g: dion_b200.Dion2(g, lr=0.02, fraction=0.25),
    "dion2_global": lambda g: dion_b200.Dion2(g, lr=0.02, fraction=0.5, selection_scope="global"),
    "nordion2": lambda g: dion_b200.NorDion2(g, lr=0.02, fraction=0.5),
    "dion": lambda g: dion_b200.Dion(g, lr=0.02, rank_fraction=0.5),
    "dion_reference": lambda g: dion_b200.DionReference(g, lr=0.02, rank_fraction=0.5),
    "dion_simple": lambda g: dion_b200.DionSimple(g, lr=0.02, rank=8),
    "muon_reference": lambda g: dion_b200.MuonReference(g, lr=0.02),
}


def _run(name, steps=3, seed=0, scalar_algo="adamw"):
    mats, vecs = _make(seed)
    groups = [dict(params=mats), dict(params=vecs, algorithm=scalar_algo, lr=0.01)]
    opt = FACTORIES[name](groups)
    g = torch.Generator().manual_seed(3)
    for _ in range(steps):
        for p in mats + vecs:
            p.grad = torch.randn(p.shape, generator=g)
        opt.step()
    return [p.detach().clone() for p in mats + vecs], opt


@pytest.mark.parametrize("name", list(FACTORIES))
def test_parameters_move_and_stay_finite(name):
    before = [p.detach().clone() for p in sum(_make(), [])]
    after, _ = _run(name)
    for b, a in zip(before, after):
        assert torch.isfinite(a).all()
        assert not torch.equal(a, b)


@pytest.mark.parametrize("name", list(FACTORIES))
def test_two_identical_runs_agree_exactly(name):
    a, _ = _run(name)
    b, _ = _run(name)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("name", ["muon", "dion2", "normuon", "dion"])
def test_lion_group_works_beside_the_matrix_algorithm(name):
    after, opt = _run(name, scalar_algo="lion")
    assert all(torch.isfinite(a).all() for a in after)
    algos = {g["algorithm"] for g in opt.param_groups}
    assert "lion" in algos and len(algos) == 2


@pytest.mark.parametrize("name", ["muon", "normuon", "dion2", "nordion2", "dion"])
def test_parameters_without_gradient_are_left_alone(name):
    mats, vecs = _make()
    opt = FACTORIES[name]([dict(params=mats), dict(params=vecs, algorithm="adamw", lr=0.01)])
    frozen = mats[1].detach().clone()
    for p in mats + vecs:
        p.grad = torch.randn_like(p)
    mats[1].grad = None
    opt.step()
    assert torch.equal(mats[1], frozen)
    assert not torch.equal(mats[0], _make()[0][0])


def test_vector_in_matrix_group_is_rejected():
    _, vecs = _make()
    opt = dion_b200.Muon([dict(params=vecs)], lr=0.02)
    for p in vecs:
        p.grad = torch.randn_like(p)
    with pytest.raises((AssertionError, ValueError, RuntimeError)):
        opt.step()


@pytest.mark.parametrize("kw", [dict(lr=-1.0), dict(mu=-0.1), dict(adjust_lr="bogus")])
def test_bad_hyperparameters_are_rejected(kw):
    mats, _ = _make()
    with pytest.raises(ValueError):
        dion_b200.Muon([dict(params=mats)], **kw)


def test_dion2_scope_default_is_local_and_full_fraction_makes_scopes_equal():
    mats, _ = _make()
    opt = dion_b200.Dion2([dict(params=mats)], lr=0.02, fraction=0.25)
    assert opt.param_groups[0].get("selection_scope", "local") == "local"

    def run(scope):
        ms, _ = _make()
        o = dion_b200.Dion2([dict(params=ms)], lr=0.02, fraction=1.0, selection_scope=scope)
        g = torch.Generator().manual_seed(9)
        for _ in range(2):
            for p in ms:
                p.grad = torch.randn(p.shape, generator=g)
            o.step()
        return [p.detach().clone() for p in ms]

    for a, b in zip(run("local"), run("global")):
        assert torch.allclose(a, b, atol=1e-6)


class _DeviceLookalike(torch.Tensor):
    """A wrapper-subclass tensor that reports a CUDA device while its data lives elsewhere - what
    DTensor-like wrappers look like to code that is about to hand a raw address to a kernel (the
    reference tests the same guard with a mock ``__torch_dispatch__`` tensor,
    tests/test_dion2_post_ortho_triton.py:95-159)."""

    @staticmethod
    def __new__(cls, inner):
        return torch.Tensor._make_wrapper_subclass(
            cls, inner.shape, dtype=inner.dtype, device="cuda", strides=inner.stride())

    def __init__(self, inner):
        self.inner = inner

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        from torch.utils._pytree import tree_map
        strip = lambda t: t.inner if isinstance(t, _DeviceLookalike) else t  # noqa: E731
        out = func(*tree_map(strip, args), **tree_map(strip, kwargs or {}))
        return tree_map(lambda t: _DeviceLookalike(t) if isinstance(t, torch.Tensor) else t, out)


def test_wrapper_subclass_tensors_never_reach_a_raw_pointer_kernel():
    from dion_b200.ops import foreach as F
    from dion_b200.utils.tensors import is_plain_tensor
    torch.manual_seed(0)
    x0 = torch.randn(6, 8)
    u = torch.randn(3, 8).bfloat16()
    idx = torch.tensor([4, 0, 2])
    wrapped = _DeviceLookalike(x0.clone())
    assert wrapped.is_cuda and not is_plain_tensor(wrapped)
    assert not F._kernel_ok([wrapped], [u])
    # The update goes through tensor arithmetic (dispatched to the wrapper) and matches the
    # plain-tensor result exactly.
    plain = x0.clone()
    maps = [torch.full((6,), -1, dtype=torch.int32)]
    maps[0][idx] = torch.arange(3, dtype=torch.int32)
    F.dion2_post([plain], [u], [idx], maps, 0.1, 0.01, 1.5, -2)
    F.dion2_post([wrapped], [u], [idx], maps, 0.1, 0.01, 1.5, -2)
    assert torch.equal(wrapped.inner, plain)
    untouched = [r for r in range(6) if r not in idx.tolist()]
    assert torch.equal(plain[untouched], x0[untouched] * (1 - 0.1 * 0.01))


def _public_overrides(cls):
    return sorted(n for n, a in vars(cls).items()
                  if callable(a) and not n.startswith("_") and hasattr(torch.optim.Optimizer, n))


def test_graph_wrapper_is_call_compatible_with_torch_optimizer():
    """The CUDA-graph wrapper stands in for a ``torch.optim.Optimizer``: every method it
    overrides keeps torch's parameter names and kinds (distributed checkpointing calls
    ``load_state_dict(state_dict=...)`` by keyword), found by reflection so that a method
    overridden later is checked too (reference: tests/test_cuda_graph.py:818-872)."""
    import inspect
    from dion_b200 import CudaGraphOptimizer, Dion2
    names = _public_overrides(CudaGraphOptimizer)
    assert {"load_state_dict", "state_dict", "zero_grad", "step", "add_param_group"} <= set(names)
    for name in names:
        ours = inspect.signature(getattr(CudaGraphOptimizer, name))
        base = inspect.signature(getattr(torch.optim.Optimizer, name))
        assert [(p.name, p.kind) for p in ours.parameters.values()] == \
            [(p.name, p.kind) for p in base.parameters.values()], name
    # and the keyword call really loads: the step counter of a saved run arrives
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(8, 16)) for _ in range(2)]
    src = Dion2([dict(params=ps)], lr=0.01)
    for _ in range(2):
        for p in ps:
            p.grad = torch.randn_like(p)
        src.step()
    saved = src.state_dict()
    qs = [torch.nn.Parameter(torch.randn(8, 16)) for _ in range(2)]
    wrap = CudaGraphOptimizer(Dion2([dict(params=qs)], lr=0.01), warmup_steps=1)
    before = wrap.param_groups[0]["step"]
    wrap.load_state_dict(state_dict=saved)
    assert wrap.param_groups[0]["step"] == src.param_groups[0]["step"] != before


def test_graph_wrapper_steps_eagerly_for_host_parameters():
    """With parameters on the CPU there is nothing to record: every step is an ordinary step and
    matches the unwrapped optimizer."""
    from dion_b200 import CudaGraphOptimizer, Muon
    torch.manual_seed(0)
    w0 = torch.randn(8, 16)
    grads = [torch.randn(8, 16) for _ in range(4)]
    out = []
    for wrap in (False, True):
        p = torch.nn.Parameter(w0.clone())
        opt = Muon([dict(params=[p])], lr=0.01)
        opt = CudaGraphOptimizer(opt, warmup_steps=1) if wrap else opt
        for g in grads:
            p.grad = g.clone()
            opt.step()
            opt.zero_grad()
        out.append(p.detach().clone())
    assert torch.equal(out[0], out[1])
