"""Whole-step CUDA graph runtime and the bucketed gradient all-reduce."""
import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_ranks


def _mlp(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 8),
                               torch.nn.Tanh(), torch.nn.Linear(8, 1))


def _sync_worker(rank, world):
    from dion_b200.parallel.graph_step import BucketedGradSync, GraphedTrainStep
    model = _mlp()
    params = list(model.parameters())
    # ~1 KB buckets: several buckets, each launched from a hook.
    sync = BucketedGradSync(params, None, bucket_mb=0.001)
    assert len(sync.buckets) > 1
    torch.manual_seed(100 + rank)
    x = torch.randn(4, 16)
    model(x).sum().backward()
    local = [p.grad.clone() for p in params]
    sync.finish()
    for p, g in zip(params, local):
        ref = g.clone()
        dist.all_reduce(ref)
        assert torch.allclose(p.grad, ref / world, atol=1e-6)
    # A second round re-arms the hooks.
    model.zero_grad(set_to_none=True)
    model(x).sum().backward()
    sync.finish()
    for p, g in zip(params, local):
        ref = g.clone()
        dist.all_reduce(ref)
        assert torch.allclose(p.grad, ref / world, atol=1e-6)
    sync.remove()

    # The eager form of the step object keeps replicas identical.
    model = _mlp()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    step = GraphedTrainStep(lambda a: model(a).pow(2).mean(), list(model.parameters()), opt, [x],
                            device=torch.device("cpu"), autocast_dtype=None, use_graph=False)
    for i in range(3):
        torch.manual_seed(7 * rank + i)
        step(torch.randn(4, 16))
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    for other in gathered:
        assert torch.equal(other, flat)
    return True


def test_bucketed_grad_sync_gloo():
    run_ranks(_sync_worker, 2)


def _tiny_gpt():
    from dion_b200.models.gpt import GPT, GPTConfig
    torch.manual_seed(0)
    m = GPT(GPTConfig(n_layer=2, n_embd=128, n_head=2, vocab_size=512, sequence_len=64)).cuda()
    m.init_weights()
    return m


def _make_opt(model, name):
    import dion_b200
    groups = [dict(params=list(model.transformer.h.parameters())),
              dict(params=list(model.transformer.wte.parameters()), algorithm="adamw", lr=0.01,
                   weight_decay=0),
              dict(params=list(model.lm_head.parameters()), algorithm="adamw", lr=0.01,
                   weight_decay=0)]
    if name == "dion2":
        return dion_b200.Dion2(groups, lr=0.02, fraction=0.25, ef_decay=0.95, weight_decay=0.01,
                               use_polar_express=False)
    return dion_b200.Muon(groups, lr=0.02, mu=0.95, weight_decay=0.01, nesterov=True)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["dion2", "muon"])
def test_graphed_step_matches_eager(name):
    from dion_b200.parallel.graph_step import GraphedTrainStep
    from dion_b200.ops.gemm import check_status
    g = torch.Generator().manual_seed(1)
    batches = [torch.randint(0, 512, (2, 4, 64), generator=g).cuda() for _ in range(8)]
    losses = {}
    for use_graph in (False, True):
        model = _tiny_gpt()
        opt = _make_opt(model, name)
        step = GraphedTrainStep(lambda x, y: model(x, y), list(model.parameters()), opt,
                                [batches[0][0], batches[0][1]], device=torch.device("cuda"),
                                warmup=2, use_graph=use_graph)
        out = []
        for xy in batches:
            out.append(float(step(xy[0], xy[1]).item()))
        torch.cuda.synchronize()
        check_status()
        if use_graph:
            assert step.graph is not None
        assert all(g["step"] == len(batches) for g in opt.param_groups)
        losses[use_graph] = out
        step.release()
    assert losses[True][0] == pytest.approx(losses[False][0], rel=1e-5)
    for a, b in zip(losses[True], losses[False]):
        assert a == pytest.approx(b, rel=2e-2, abs=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["muon", "dion2"])
def test_cuda_graph_optimizer_matches_eager(name):
    """Captured ``optimizer.step()`` (warm-up, capture, replay) against the eager optimizer."""
    import dion_b200
    from dion_b200.optim.cuda_graph import CudaGraphOptimizer
    from dion_b200.ops.gemm import check_status

    def run(graphed):
        torch.manual_seed(0)
        mats = [torch.nn.Parameter(torch.randn(256, 128, device="cuda") * 0.1) for _ in range(4)]
        vecs = [torch.nn.Parameter(torch.randn(128, device="cuda"))]
        groups = [dict(params=mats), dict(params=vecs, algorithm="adamw", lr=0.01)]
        if name == "muon":
            opt = dion_b200.Muon(groups, lr=0.02, mu=0.9, weight_decay=0.01)
        else:
            opt = dion_b200.Dion2(groups, lr=0.02, fraction=0.5, ef_decay=0.9, weight_decay=0.01)
        stepper = CudaGraphOptimizer(opt, warmup_steps=2) if graphed else opt
        sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0 / (1 + s))
        g = torch.Generator(device="cuda").manual_seed(1)
        for p in mats + vecs:
            p.grad = torch.zeros_like(p)
        for _ in range(6):
            for p in mats + vecs:
                p.grad.copy_(torch.randn(p.shape, device="cuda", generator=g))
            stepper.step()
            sched.step()
        torch.cuda.synchronize()
        check_status()
        if graphed:
            assert stepper._graph is not None
            stepper.release()
        return [p.detach().clone() for p in mats + vecs]

    eager, graphed = run(False), run(True)
    # The Frobenius norms are accumulated with floating-point atomics, so two runs can differ by
    # a bf16 rounding of the orthogonalized update (about lr * 2^-8 per step).
    for a, b in zip(eager, graphed):
        assert torch.allclose(a, b, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_trainer_with_graph_step_runs_and_loss_falls():
    """`train.py --graph_step` on one GPU: the captured step trains (repeated synthetic data)."""
    import os
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr",
           "127.0.0.1", "--nproc-per-node", "1", os.path.join(root, "train.py"),
           "--synthetic", "--no_wandb", "--debug", "--model_dim", "128", "--n_layer", "2",
           "--n_head", "2", "--sequence_length", "64", "--batch_size", "16",   # 2 micro-batches
           "--device_batch_size", "8", "--val_loss_every", "0", "--scalar_opt", "adamw",
           "--optimizer", "muon", "--num_iterations", "12", "--graph_step"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    losses = [float(m) for m in re.findall(r"train_loss=([0-9.]+)", res.stdout)]
    assert len(losses) == 12
    assert all(l == l and l < 20 for l in losses)


def _accum_worker(rank, world):
    """k micro-batches through the step object == one batch of k times the size."""
    from dion_b200.parallel.graph_step import GraphedTrainStep

    def run(k):
        model = _mlp()
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        ex = torch.zeros(4 // k, 16)
        step = GraphedTrainStep(lambda a: model(a).pow(2).mean(), list(model.parameters()), opt,
                                [ex], device=torch.device("cpu"), autocast_dtype=None,
                                use_graph=False, accumulation_steps=k)
        losses = []
        for i in range(3):
            torch.manual_seed(11 * rank + i)
            data = torch.randn(4, 16)
            losses.append(float(step(data if k == 1 else data.view(k, 4 // k, 16))))
        return losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()])

    l1, p1 = run(1)
    l2, p2 = run(2)
    assert torch.allclose(p1, p2, atol=1e-6)
    assert all(abs(a - b) < 1e-6 for a, b in zip(l1, l2))
    gathered = [torch.empty_like(p2) for _ in range(world)]
    dist.all_gather(gathered, p2)
    assert all(torch.equal(g, p2) for g in gathered)
    return True


def test_gradient_accumulation_in_step_object_gloo():
    run_ranks(_accum_worker, 2)
