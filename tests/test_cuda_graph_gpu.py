"""CudaGraphOptimizer: replay must follow schedules that are applied between steps, refuse
captures that would silently drop parameters, and survive release / resume.  (The behaviours
are those the reference checks in tests/test_cuda_graph.py; the scenarios are built here.)"""
import io

import pytest
import torch

pytestmark = pytest.mark.gpu

WARMUP, STEPS, TOL = 2, 7, 2e-3   # TOL: one bf16 rounding of an orthogonalized update * lr


def _opt_classes():
    import dion_b200
    return [dion_b200.Muon, dion_b200.NorMuon, dion_b200.Dion2, dion_b200.NorDion2]


def _build(cls, weight_decay=0.01, **kw):
    torch.manual_seed(11)
    mats = [torch.nn.Parameter(torch.randn(64, 128, device="cuda")),
            torch.nn.Parameter(torch.randn(128, 64, device="cuda"))]
    vecs = [torch.nn.Parameter(torch.randn(64, device="cuda")),
            torch.nn.Parameter(torch.randn(128, device="cuda"))]
    opt = cls([dict(params=mats), dict(params=vecs, algorithm="adamw")], lr=0.02,
              weight_decay=weight_decay, **kw)
    return mats + vecs, opt


def _grads(params, steps=STEPS):
    g = torch.Generator(device="cuda").manual_seed(5)
    return [[torch.randn(p.shape, device="cuda", generator=g) for p in params]
            for _ in range(steps)]


def _drive(params, opt, stepper, grads, before_step=None):
    for p in params:
        p.grad = torch.zeros_like(p)
    for t, gs in enumerate(grads):
        if before_step is not None:
            before_step(t)
        for p, g in zip(params, gs):
            p.grad.copy_(g)
        stepper.step()
    torch.cuda.synchronize()
    return [p.detach().clone() for p in params]


def _maxdiff(a, b):
    return max((x - y).abs().max().item() for x, y in zip(a, b))


@pytest.mark.parametrize("idx", range(4))
def test_replay_follows_learning_rate_assigned_as_float(idx):
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    cls = _opt_classes()[idx]
    lrs = [0.03 - 0.003 * t for t in range(STEPS)]

    def run(graphed, schedule):
        params, opt = _build(cls)
        stepper = CudaGraphOptimizer(opt, warmup_steps=WARMUP) if graphed else opt

        def set_lr(t):
            for group in opt.param_groups:
                group["lr"] = schedule[t]      # plain float assignment, as a user script does
        out = _drive(params, opt, stepper, _grads(params), set_lr)
        if graphed:
            stepper.release()
        return out

    eager, graph = run(False, lrs), run(True, lrs)
    frozen = run(True, [lrs[WARMUP]] * STEPS)
    assert _maxdiff(eager, graph) < TOL
    assert _maxdiff(graph, frozen) > 5 * TOL    # the schedule really mattered


def test_replay_follows_cosine_scheduler_and_lr_tensor_is_stable():
    import dion_b200
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer

    def run(graphed):
        params, opt = _build(dion_b200.Muon)
        stepper = CudaGraphOptimizer(opt, warmup_steps=WARMUP) if graphed else opt
        sched = torch.optim.lr_scheduler.CosineAnnealingLR(stepper, T_max=STEPS)
        ids = []
        for p in params:
            p.grad = torch.zeros_like(p)
        for gs in _grads(params):
            for p, g in zip(params, gs):
                p.grad.copy_(g)
            stepper.step()
            sched.step()
            ids.append(tuple(id(g["lr"]) for g in opt.param_groups))
        torch.cuda.synchronize()
        assert len(set(ids)) == 1, "the lr tensors must keep their identity across steps"
        if graphed:
            stepper.release()
        return [p.detach().clone() for p in params]

    assert _maxdiff(run(False), run(True)) < TOL


@pytest.mark.parametrize("idx", range(4))
def test_tensor_weight_decay_is_live_under_replay(idx):
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    cls = _opt_classes()[idx]
    wds = [0.3 - 0.03 * t for t in range(STEPS)]

    def run(graphed, schedule):
        params, opt = _build(cls, weight_decay=torch.tensor(0.03))
        for group in opt.param_groups:
            assert isinstance(group["weight_decay"], torch.Tensor)
            assert group["weight_decay"].is_cuda
        stepper = CudaGraphOptimizer(opt, warmup_steps=WARMUP) if graphed else opt

        def set_wd(t):
            for group in opt.param_groups:
                group["weight_decay"].fill_(schedule[t])
        out = _drive(params, opt, stepper, _grads(params), set_wd)
        if graphed:
            stepper.release()
        return out

    eager, graph = run(False, wds), run(True, wds)
    frozen = run(True, [wds[WARMUP]] * STEPS)
    assert _maxdiff(eager, graph) < TOL
    assert _maxdiff(graph, frozen) > 1e-3


def test_float_weight_decay_stays_a_float_and_tensor_opt_in_latches():
    import dion_b200
    _, opt = _build(dion_b200.Dion2)
    opt._sync_hyperparam_tensors()
    assert all(not isinstance(g["weight_decay"], torch.Tensor) for g in opt.param_groups)
    assert all(name != "weight_decay" for _, name in opt._hyperparam_tensors)
    # Assigning a tensor later opts the group in ...
    for group in opt.param_groups:
        group["weight_decay"] = torch.tensor(0.03, device="cuda")
    opt._sync_hyperparam_tensors()
    held = [g["weight_decay"] for g in opt.param_groups]
    for i, group in enumerate(opt.param_groups):
        assert group["weight_decay"] is opt._hyperparam_tensors[(i, "weight_decay")]
    # ... for good: a float assigned afterwards refills the same tensor.
    for group in opt.param_groups:
        group["weight_decay"] = 0.01
    opt._sync_hyperparam_tensors()
    for group, t in zip(opt.param_groups, held):
        assert group["weight_decay"] is t and t.item() == pytest.approx(0.01)


def test_live_weight_decay_and_state_survive_save_and_load():
    import dion_b200
    params, opt = _build(dion_b200.NorMuon, weight_decay=torch.tensor(0.05))
    grads = _grads(params, 3)
    _drive(params, opt, opt, grads)
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    sd = torch.load(buf, map_location="cpu")
    assert all(isinstance(g["weight_decay"], float) for g in sd["param_groups"])
    params2, opt2 = _build(dion_b200.NorMuon, weight_decay=torch.tensor(0.05))
    with torch.no_grad():
        for a, b in zip(params2, params):
            a.copy_(b)
    opt2.load_state_dict(sd)
    for i, group in enumerate(opt2.param_groups):
        assert isinstance(group["weight_decay"], torch.Tensor)
        assert group["weight_decay"].item() == pytest.approx(0.05)
    more = _grads(params, 2)
    a = _drive(params, opt, opt, more)
    b = _drive(params2, opt2, opt2, more)
    assert _maxdiff(a, b) < TOL


def test_capture_refuses_parameters_without_gradients_and_leaves_no_graph():
    import dion_b200
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    params, opt = _build(dion_b200.Muon)
    stepper = CudaGraphOptimizer(opt, warmup_steps=1)
    for p in params:
        p.grad = torch.randn_like(p)
    stepper.step()                      # warm-up
    params[1].grad = None
    with pytest.raises(RuntimeError, match="grad"):
        stepper.step()
    assert stepper._graph is None
    params[1].grad = torch.randn_like(params[1])
    stepper.step()                      # captures now
    assert stepper._graph is not None
    stepper.release()


def test_release_recaptures_and_host_step_counters_advance():
    import dion_b200
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    params, opt = _build(dion_b200.Dion2)
    stepper = CudaGraphOptimizer(opt, warmup_steps=1)
    for p in params:
        p.grad = torch.randn_like(p)
    for _ in range(4):
        stepper.step()
    assert all(g["step"] == 4 for g in opt.param_groups)
    first = stepper._graph
    assert first is not None
    stepper.release()
    assert stepper._graph is None
    for _ in range(3):
        stepper.step()
    assert stepper._graph is not None and stepper._graph is not first
    assert all(g["step"] == 7 for g in opt.param_groups)
    stepper.release()


def test_tensor_hyperparameter_introduced_after_capture_is_an_error():
    import dion_b200
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    params, opt = _build(dion_b200.Muon)
    stepper = CudaGraphOptimizer(opt, warmup_steps=1)
    for p in params:
        p.grad = torch.randn_like(p)
    for _ in range(3):
        stepper.step()
    for group in opt.param_groups:
        group["weight_decay"] = torch.tensor(0.2, device="cuda")
    with pytest.raises(RuntimeError, match="after"):
        stepper.step()
    stepper.release()
    stepper.step()                      # warm-up again, then it may be captured with the tensor
    stepper.step()
    stepper.release()
