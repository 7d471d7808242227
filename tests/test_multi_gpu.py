"""Multi-GPU (NCCL, one process per GPU) tests: the fused peer-memory exchange against the
collective path and a single-GPU run, replicated (DDP) work splitting, and the bounded wait."""
import os

import pytest
import torch
import torch.distributed as dist

import dion_b200
from tests.dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


SHAPES = ((256, 512),) * 5 + ((512, 256),) * 3 + ((256, 256),) * 4


def _weights(shapes, seed=7):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*s, generator=g) for s in shapes]


def _single_gpu(name, kw, steps):
    ps = [torch.nn.Parameter(w.cuda()) for w in _weights(SHAPES)]
    opt = getattr(dion_b200, name)([dict(params=ps)], lr=0.05, **kw)
    for s in range(steps):
        for p, g in zip(ps, _weights(SHAPES, 100 + s)):
            p.grad = g.cuda()
        opt.step()
    torch.cuda.synchronize()
    return [p.detach().cpu() for p in ps]


def _sharded(rank, world, name, kw, steps, fused, shard=0):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    from dion_b200.ops.gemm import check_status
    os.environ["DION_B200_FUSED_EXCHANGE"] = "1" if fused else "0"
    mesh = init_device_mesh("cuda", (world,))
    ps = [torch.nn.Parameter(distribute_tensor(w.cuda(), mesh, [Shard(shard)]))
          for w in _weights(SHAPES)]
    opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=mesh, lr=0.05, **kw)
    for s in range(steps):
        for p, g in zip(ps, _weights(SHAPES, 100 + s)):
            p.grad = distribute_tensor(g.cuda(), mesh, [Shard(shard)])
        opt.step()
    torch.cuda.synchronize()
    check_status()
    used = len(getattr(opt, "_fused_exchanges", {}))
    full = [p.detach().full_tensor().cpu() for p in ps]
    return (full, used) if rank == 0 else None


def _replicated(rank, world, name, kw, steps):
    ps = [torch.nn.Parameter(w.cuda()) for w in _weights(SHAPES)]
    opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=dist.group.WORLD, lr=0.05, **kw)
    for s in range(steps):
        for p, g in zip(ps, _weights(SHAPES, 100 + s)):
            p.grad = g.cuda()
        opt.step()
    torch.cuda.synchronize()
    return [p.detach().cpu() for p in ps] if rank == 0 else None


@pytest.mark.parametrize("world", [2, 4, 8])
def test_muon_fused_exchange_matches_collective_and_single(tmp_path, world):
    _need(world)
    kw = dict(nesterov=True, use_polar_express=False)
    ref = _single_gpu("Muon", kw, 3)
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    coll, used0 = run_ranks(_sharded, world, "nccl", ("Muon", kw, 3, False), str(tmp_path / "a"))[0]
    fused, used1 = run_ranks(_sharded, world, "nccl", ("Muon", kw, 3, True), str(tmp_path / "b"))[0]
    assert used0 == 0 and used1 > 0  # the fused path really ran
    for r, c, f in zip(ref, coll, fused):
        assert (r - c).abs().max().item() < 2e-3
        assert (r - f).abs().max().item() < 2e-3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchange_of_column_shards_matches_collective_and_single(tmp_path, world):
    """``Shard(1)`` parameters: the momentum kernel's strided store into the owner's matrix, the
    Gram GEMM gated by K-slabs (wide) or tile rows (tall), the update GEMM's column-split remote
    store - against the collective path and an unsharded run."""
    _need(world)
    name, kw = "Muon", dict(nesterov=True, use_polar_express=False)
    ref = _single_gpu(name, kw, 3)
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    coll, used0 = run_ranks(_sharded, world, "nccl", (name, kw, 3, False, 1), str(tmp_path / "a"))[0]
    fused, used1 = run_ranks(_sharded, world, "nccl", (name, kw, 3, True, 1), str(tmp_path / "b"))[0]
    assert used0 == 0 and used1 > 0
    for r, c, f in zip(ref, coll, fused):
        assert (c - f).abs().max().item() < 2e-3
        assert (r - f).abs().max().item() < 2e-3


def test_replicated_work_split_matches_single(tmp_path):
    _need(2)
    for name, kw in (("Muon", dict()), ("Dion2", dict()), ("NorMuon", dict())):
        ref = _single_gpu(name, kw, 2)
        d = tmp_path / name
        d.mkdir()
        out = run_ranks(_replicated, 2, "nccl", (name, kw, 2), str(d))[0]
        for r, o in zip(ref, out):
            assert (r - o).abs().max().item() < 2e-3, name


def test_wait_on_flag_nobody_sets_times_out_cleanly():
    """A bounded device-side wait returns an error status instead of hanging, and the context
    stays usable."""
    from dion_b200.ops import gemm
    from dion_b200.parallel import symm
    dev = torch.device("cuda")
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    seq = torch.ones((), dtype=torch.int32, device=dev)
    status = gemm.status_tensor(dev)
    status.zero_()
    symm.wait_flags(flags, seq, 0, status)   # nothing ever raises these flags
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer") as err:
        gemm.check_status()
    assert "waited for sequence 1, found 0" in str(err.value)   # who / what is reported
    x = torch.ones(8, device=dev)
    assert float((x * 2).sum()) == 16.0      # context still alive
    gemm.check_status()                       # status was cleared


def test_update_is_refused_after_a_timeout_and_the_next_step_raises():
    """The apply kernel waits for a producer that never signals: the wait runs out, the weights
    stay bit-identical, the status names the silent rank, and the optimizer's next step raises
    without anybody having synchronized on its behalf."""
    from dion_b200.ops import _backend, foreach, gemm
    dev = torch.device("cuda")
    _backend.lib("foreach_ops")
    _backend.set_wait_budget_ms(50)
    try:
        gemm.status_tensor(dev).zero_()
        g = torch.Generator(device=dev).manual_seed(0)
        X = [torch.randn(64, 128, device=dev, generator=g) for _ in range(4)]
        U = [torch.randn(64, 128, device=dev, generator=g).bfloat16() for _ in range(4)]
        before = [x.clone() for x in X]
        flags = torch.zeros(2, dtype=torch.int32, device=dev)   # producers 0 and 1: never raised
        seq = torch.ones((), dtype=torch.int32, device=dev)
        wait = (flags, seq, 2, gemm.status_tensor(dev))
        foreach.muon_post(X, U, 0.1, 0.01, 1.0, wait=wait)
        torch.cuda.synchronize()
        for x, b in zip(X, before):
            assert torch.equal(x, b)
        # Once the status word is set, later kernels of the same kind refuse as well, even if
        # their own producer has signalled.
        flags.fill_(1)
        foreach.muon_post(X, U, 0.1, 0.01, 1.0, wait=wait)
        V = [torch.ones(64, 1, device=dev) for _ in range(4)]
        foreach.normuon_rowstats(torch.stack(U), V, 0.95, guard=gemm.status_tensor(dev))
        torch.cuda.synchronize()
        for x, b in zip(X, before):
            assert torch.equal(x, b)
        assert all(bool((v == 1).all()) for v in V)
        # An optimizer notices at its next step (snapshot taken after a step, read before one).
        p = torch.nn.Parameter(torch.randn(64, 128, device=dev))
        opt = dion_b200.Muon([dict(params=[p])], lr=0.01)
        opt._snapshot_device_status()
        torch.cuda.synchronize()
        p.grad = torch.randn_like(p)
        with pytest.raises(RuntimeError, match="flag of source rank") as err:
            opt.step()
        assert "waited for sequence 1, found 0" in str(err.value)
        opt.step()                       # status cleared: the run can go on
        gemm.check_status()
    finally:
        _backend.set_wait_budget_ms(2000)
        gemm.status_tensor(dev).zero_()


@pytest.mark.parametrize("name,kw", [("NorMuon", dict(use_polar_express=False)),
                                     ("Dion2", dict(fraction=0.25)),
                                     ("NorDion2", dict(fraction=0.5))])
def test_fused_exchange_matches_collective_other_optimizers(tmp_path, name, kw):
    _need(2)
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    coll, used0 = run_ranks(_sharded, 2, "nccl", (name, kw, 3, False), str(tmp_path / "a"))[0]
    fused, used1 = run_ranks(_sharded, 2, "nccl", (name, kw, 3, True), str(tmp_path / "b"))[0]
    assert used0 == 0 and used1 > 0
    for c, f in zip(coll, fused):
        assert (c - f).abs().max().item() < 2e-3, name


def _symm_allreduce_worker(rank, world, use_nvls):
    import os
    os.environ["DION_B200_NVLS"] = "1" if use_nvls else "0"
    from dion_b200.ops.gemm import check_status
    from dion_b200.parallel import symm
    dev = torch.device("cuda", rank)
    pg = dist.group.WORLD
    red = symm.SymmetricAllReduce(pg, 8 << 20, dev)
    out = {"multimem": red.uses_multimem}
    for dtype, n in ((torch.float32, 1000003), (torch.bfloat16, 65536 + 8), (torch.float32, 5)):
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        t = torch.randn(n, device=dev, generator=g).to(dtype)
        ref = t.clone().float()
        dist.all_reduce(ref)
        for op in ("sum", "avg"):
            x = t.clone()
            red.all_reduce_tensor_(x, op)
            torch.cuda.synchronize()
            check_status()
            want = ref / world if op == "avg" else ref
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert (x.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    # Zero-copy form and the cached helper.
    v = red.view((4096,), torch.float32)
    v.fill_(float(rank + 1))
    red.all_reduce_(4096, torch.float32, "sum")
    torch.cuda.synchronize()
    assert torch.all(v == world * (world + 1) / 2)
    y = torch.full((3, 7), float(rank), device=dev)
    symm.symmetric_all_reduce_(y, pg, "avg")
    torch.cuda.synchronize()
    assert torch.allclose(y, torch.full_like(y, (world - 1) / 2))
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("use_nvls", [True, False])
def test_symmetric_all_reduce_matches_nccl(tmp_path, use_nvls):
    _need(2)
    world = 4 if torch.cuda.device_count() >= 4 else 2
    res = run_ranks(_symm_allreduce_worker, world, backend="nccl", args=(use_nvls,),
                    result_dir=str(tmp_path))
    assert len(res) == world
    if not use_nvls:
        assert not any(r["multimem"] for r in res)


def _dion_ddp_worker(rank, world, mode):
    import os
    os.environ["DION_B200_SYMM_ALLREDUCE"] = "1" if mode == "symmetric" else "0"
    os.environ["DION_B200_FUSED_LOWRANK"] = "1" if mode == "fused" else "0"
    from dion_b200.ops.gemm import check_status
    dev = torch.device("cuda", rank)
    torch.manual_seed(3)
    params = [torch.nn.Parameter(torch.randn(256, 128, device=dev) * 0.1) for _ in range(3)]
    params += [torch.nn.Parameter(torch.randn(128, 256, device=dev) * 0.1) for _ in range(2)]
    opt = dion_b200.Dion([dict(params=params)], replicate_mesh=dist.group.WORLD,
                         replicate_mesh_grad_sync=True, rank_fraction=0.25, lr=0.02)
    g = torch.Generator(device=dev).manual_seed(50 + rank)   # different gradients per rank
    for _ in range(3):
        for p in params:
            p.grad = torch.randn(p.shape, device=dev, generator=g)
        opt.step()
    opt.synchronize_for_checkpoint()
    torch.cuda.synchronize()
    check_status()
    out = [p.detach().cpu() for p in params]
    out.append(torch.tensor(float(len(opt._lowrank_sync))))
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_dion_compressed_sync_paths_agree(tmp_path, world):
    """Legacy Dion under DDP with compressed P/R synchronization, three ways: NCCL collectives,
    the symmetric-memory all-reduce kernel, and the reduce-scatter carried by the GEMM epilogue
    (with the all-gather kernel).  All give the same weights, and replicas stay identical."""
    _need(world)
    out = {}
    for mode in ("nccl", "symmetric", "fused"):
        d = tmp_path / mode
        d.mkdir()
        out[mode] = run_ranks(_dion_ddp_worker, world, backend="nccl", args=(mode,),
                              result_dir=str(d))
    assert out["fused"][0][-1].item() > 0 and out["nccl"][0][-1].item() == 0  # the path really ran
    for res in out.values():
        for other in res[1:]:
            for a, b in zip(res[0][:-1], other[:-1]):
                assert torch.allclose(a, b, atol=1e-5)
    for mode in ("symmetric", "fused"):
        for a, b in zip(out["nccl"][0][:-1], out[mode][0][:-1]):
            assert torch.allclose(a, b, atol=2e-3, rtol=1e-2), mode


def _dion_fsdp_worker(rank, world, fused):
    import os
    os.environ["DION_B200_FUSED_LOWRANK"] = "1" if fused else "0"
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    from dion_b200.ops.gemm import check_status
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("fs",))
    torch.manual_seed(5)      # the optimizer derives the seeds of Q and of the sketches from it
    g = torch.Generator().manual_seed(11)
    shapes = ((256, 128),) * 3 + ((128, 512),) * 2
    ws = [torch.randn(*s, generator=g) * 0.1 for s in shapes]
    ps = [torch.nn.Parameter(distribute_tensor(w.cuda(), mesh, [Shard(0)])) for w in ws]
    opt = dion_b200.Dion([dict(params=ps)], outer_shard_mesh=mesh, rank_fraction=0.25, lr=0.02)
    for s in range(3):
        for p, shape in zip(ps, shapes):
            grad = torch.randn(*shape, generator=g)
            p.grad = distribute_tensor(grad.cuda(), mesh, [Shard(0)])
        opt.step()
    torch.cuda.synchronize()
    check_status()
    full = [p.detach().full_tensor().cpu() for p in ps]
    return (full, len(opt._lowrank_sync)) if rank == 0 else None


def test_dion_fsdp_reduce_scatter_in_the_gemm_epilogue_matches_nccl(tmp_path):
    """Row-sharded (FSDP) legacy Dion: the partial sums of P are reduce-scattered by the GEMM
    epilogue over peer memory instead of by NCCL; same weights."""
    _need(2)
    res = {}
    for fused in (False, True):
        d = tmp_path / str(fused)
        d.mkdir()
        res[fused] = run_ranks(_dion_fsdp_worker, 2, backend="nccl", args=(fused,),
                               result_dir=str(d))[0]
    assert res[False][1] == 0 and res[True][1] > 0
    for a, b in zip(res[False][0], res[True][0]):
        assert torch.allclose(a, b, atol=2e-3, rtol=1e-2)


def test_trainer_dion_with_fsdp_and_tensor_parallel_on_gpus():
    """`train.py` with fs=2 x tp=2 on four GPUs: tensor-parallel layers hand the model kernels
    lazy collective results, which have to be completed before a kernel reads them."""
    _need(4)
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4",
           "--master-addr", "127.0.0.1", "--master-port", "29733", os.path.join(root, "train.py"),
           "--synthetic", "--no_wandb", "--debug", "--model_dim", "256", "--n_layer", "2",
           "--n_head", "4", "--sequence_length", "128", "--batch_size", "16",
           "--device_batch_size", "4", "--val_loss_every", "0", "--scalar_opt", "adamw",
           "--num_iterations", "3", "--optimizer", "dion", "--dp_size", "1", "--fs_size", "2",
           "--tp_size", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    losses = [float(m) for m in re.findall(r"train_loss=([0-9.]+)", res.stdout)]
    assert len(losses) == 3 and all(l == l and l < 20 for l in losses)


def _graphed_ddp_worker(rank, world, use_graph):
    from dion_b200.models.gpt import GPT, GPTConfig
    from dion_b200.ops.gemm import check_status
    from dion_b200.parallel.graph_step import GraphedTrainStep
    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=2, n_embd=128, n_head=2, vocab_size=512, sequence_len=64)).to(dev)
    model.init_weights()
    groups = [dict(params=list(model.transformer.h.parameters())),
              dict(params=list(model.transformer.wte.parameters()) + list(model.lm_head.parameters()),
                   algorithm="adamw", lr=0.01, weight_decay=0)]
    opt = dion_b200.Dion2(groups, distributed_mesh=dist.group.WORLD, lr=0.02, fraction=0.25,
                          use_polar_express=False)
    g = torch.Generator().manual_seed(10 + rank)          # different data on every rank
    batches = [torch.randint(0, 512, (2, 4, 64), generator=g).to(dev) for _ in range(6)]
    step = GraphedTrainStep(lambda x, y: model(x, y), list(model.parameters()), opt,
                            [batches[0][0], batches[0][1]], device=dev,
                            process_group=dist.group.WORLD, warmup=2, use_graph=use_graph,
                            bucket_mb=0.05)               # several buckets
    losses = [float(step(b[0], b[1]).item()) for b in batches]
    torch.cuda.synchronize()
    check_status()
    flat = torch.cat([p.detach().reshape(-1).float() for p in model.parameters()])
    step.release()
    return {"losses": losses, "params": flat.cpu()}


def test_graphed_data_parallel_step_keeps_replicas_identical_and_matches_eager(tmp_path):
    _need(2)
    out = {}
    for use_graph in (False, True):
        d = tmp_path / str(use_graph)
        d.mkdir()
        out[use_graph] = run_ranks(_graphed_ddp_worker, 2, backend="nccl", args=(use_graph,),
                                   result_dir=str(d))
    for res in out.values():
        assert torch.equal(res[0]["params"], res[1]["params"])
        assert all(l == l for l in res[0]["losses"])
    a, b = out[False][0]["params"], out[True][0]["params"]
    assert (a - b).abs().max().item() < 5e-3


def _fsdp_symm_ag_worker(rank, world, symmetric):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from dion_b200.models.gpt import GPT, GPTConfig
    from dion_b200.ops.gemm import check_status
    from dion_b200.parallel.fsdp_comm import use_symmetric_all_gather
    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=3, n_embd=128, n_head=2, vocab_size=512, sequence_len=64)).to(dev)
    model.init_weights()
    mesh = init_device_mesh("cuda", (world,))
    for block in model.transformer.h:
        fully_shard(block, mesh=mesh)
    fully_shard(model, mesh=mesh)
    comm = use_symmetric_all_gather(model, mesh.get_group(), dev) if symmetric else None
    opt = dion_b200.Muon(
        [dict(params=list(model.transformer.h.parameters())),
         dict(params=list(model.transformer.wte.parameters()) + list(model.lm_head.parameters()),
              algorithm="adamw", lr=0.01, weight_decay=0)],
        distributed_mesh=mesh, lr=0.02, use_polar_express=False)
    g = torch.Generator().manual_seed(20 + rank)
    losses = []
    for _ in range(4):
        xy = torch.randint(0, 512, (2, 4, 64), generator=g).to(dev)
        loss = model(xy[0], xy[1])
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        losses.append(float(loss.item()))
    torch.cuda.synchronize()
    check_status()
    flat = torch.cat([p.detach().to_local().reshape(-1).float() for p in model.parameters()])
    return {"losses": losses, "params": flat.cpu(),
            "kernel_calls": comm.calls if comm is not None else 0,
            "fallbacks": comm.fallbacks if comm is not None else 0}


def test_fsdp_all_gather_through_symmetric_memory_matches_nccl(tmp_path):
    _need(2)
    out = {}
    for symmetric in (False, True):
        d = tmp_path / str(symmetric)
        d.mkdir()
        out[symmetric] = run_ranks(_fsdp_symm_ag_worker, 2, backend="nccl", args=(symmetric,),
                                   result_dir=str(d))
    assert out[True][0]["kernel_calls"] > 0
    # The gather itself is an exact copy (first loss identical); later steps differ only by the
    # floating-point atomics in the optimizer's norm accumulation.
    for r in range(2):
        assert out[True][r]["losses"][0] == out[False][r]["losses"][0]
        for a, b in zip(out[True][r]["losses"], out[False][r]["losses"]):
            assert abs(a - b) < 1e-3
        # (Adam amplifies noise-level gradient differences on near-zero entries, so compare on
        # average rather than element by element.)
        diff = (out[True][r]["params"] - out[False][r]["params"]).abs()
        assert diff.mean().item() < 1e-4 and (diff > 5e-3).float().mean().item() < 1e-3


def _sharded_graph_worker(rank, world, name, mode):
    """Sharded optimizer step, eager or replayed by CudaGraphOptimizer, with an LR that a
    scheduler would change in place between steps."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    from dion_b200 import CudaGraphOptimizer
    from dion_b200.ops.gemm import check_status
    dev = torch.device("cuda", rank)
    mesh = init_device_mesh("cuda", (world,))
    gen = torch.Generator(device=dev).manual_seed(1234)
    shapes = ((128, 256),) * 3 + ((256, 128),) * 2
    ps = [torch.nn.Parameter(distribute_tensor(torch.randn(*s, generator=gen, device=dev), mesh,
                                               [Shard(0)])) for s in shapes]
    for p, s in zip(ps, shapes):
        p.grad = distribute_tensor(torch.zeros(*s, device=dev), mesh, [Shard(0)])
    opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=mesh, lr=0.1)
    wrap = None if mode == "eager" else CudaGraphOptimizer(opt, warmup_steps=2)
    step = opt.step if wrap is None else wrap.step
    steps = 6
    grads = [[distribute_tensor(torch.randn(*s, generator=gen, device=dev), mesh, [Shard(0)])
              for s in shapes] for _ in range(steps)]
    try:
        for t in range(steps):
            for p, g in zip(ps, grads[t]):
                p.grad.copy_(g)
            for group in opt.param_groups:
                group["lr"].fill_(0.1 * (0.25 + t / steps))
            step()
        torch.cuda.synchronize()
        check_status()
        full = [p.detach().full_tensor().cpu() for p in ps]
        used = len(opt._fused_exchanges)
    finally:
        if wrap is not None:
            wrap.release()
    return (full, used) if rank == 0 else None


@pytest.mark.parametrize("name", ["NorDion2", "Muon"])
def test_captured_sharded_step_matches_eager_with_the_fused_exchange(tmp_path, name):
    """Two ranks, row-sharded parameters: the step replayed from a CUDA graph (which then holds
    the peer-memory exchange: flag waits, remote stores, sequence numbers kept on the device)
    gives the weights of the eager run while the learning rate changes between replays."""
    _need(2)
    out = {}
    for mode in ("eager", "graph"):
        d = tmp_path / mode
        d.mkdir()
        out[mode] = run_ranks(_sharded_graph_worker, 2, "nccl", (name, mode), str(d))[0]
    assert out["graph"][1] > 0      # the fused exchange was part of the recording
    # Not bit-identical: the Frobenius norm travels as partial sums that blocks add with
    # floating-point atomics, whose order varies from run to run; the last-bit difference in
    # the scale occasionally flips a bf16 rounding inside the iteration (two eager runs differ
    # in the same way).  A stale learning rate or a missed exchange would be off by >1e-2.
    for a, b in zip(out["eager"][0], out["graph"][0]):
        assert (a - b).abs().max().item() <= 1e-3


def _dion2_empty_shard_worker(rank, world, global_rows, cols):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    from dion_b200.ops.gemm import check_status
    dev = torch.device("cuda", rank)
    mesh = init_device_mesh("cuda", (world,))
    torch.manual_seed(0)
    full = torch.randn(global_rows, cols, device=dev)
    param = torch.nn.Parameter(distribute_tensor(full, mesh, [Shard(0)]))
    before = param.to_local().clone()
    opt = dion_b200.Dion2([param], distributed_mesh=mesh, lr=0.01)
    for step in range(3):
        torch.manual_seed(step + 1)
        g = torch.randn(global_rows, cols, device=dev)
        param.grad = distribute_tensor(g, mesh, [Shard(0)])
        opt.step()
    torch.cuda.synchronize()
    check_status()
    after = param.to_local()
    if after.shape[0] > 0:
        assert not torch.equal(after, before), f"rank {rank}: weights did not update"
    else:
        assert torch.equal(after, before), f"rank {rank}: empty shard mutated"
    return None


@pytest.mark.parametrize("world,global_rows", [(2, 1), (4, 2), (4, 5)])
def test_dion2_step_with_empty_shards_over_nccl(world, global_rows):
    """Fewer rows than ranks (or a ragged split): ranks with an empty local shard take part in
    the exchange and leave their (empty) weights alone; the others update."""
    _need(world)
    run_ranks(_dion2_empty_shard_worker, world, "nccl", (global_rows, 16))


def _ragged_worker(rank, world, shapes, fused):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    from dion_b200.ops.gemm import check_status
    os.environ["DION_B200_FUSED_EXCHANGE"] = "1" if fused else "0"
    mesh = init_device_mesh("cuda", (world,))
    ps = [torch.nn.Parameter(distribute_tensor(w.cuda(), mesh, [Shard(0)]))
          for w in _weights(shapes)]
    opt = dion_b200.Muon([dict(params=ps)], distributed_mesh=mesh, lr=0.05, nesterov=True,
                         use_polar_express=False)
    for s in range(3):
        for p, g in zip(ps, _weights(shapes, 100 + s)):
            p.grad = distribute_tensor(g.cuda(), mesh, [Shard(0)])
        opt.step()
    torch.cuda.synchronize()
    check_status()
    full = [p.detach().full_tensor().cpu() for p in ps]
    return (full, len(opt._fused_exchanges)) if rank == 0 else None


@pytest.mark.parametrize("world,shapes", [
    (2, ((255, 128),) * 3),                            # 128 + 127 rows
    (4, ((125, 256),) * 5 + ((5, 64),) * 3),           # 32,32,32,29 rows; 2,2,1,0 rows
])
def test_fused_exchange_with_ragged_and_empty_shards(tmp_path, world, shapes):
    """Rows that do not divide by the number of ranks, and fewer rows than ranks: the fused
    exchange pads every rank's slice to the same height (as the collective path does) and gives
    the collective path's weights."""
    _need(world)
    res = {}
    for fused in (False, True):
        d = tmp_path / str(fused)
        d.mkdir()
        res[fused] = run_ranks(_ragged_worker, world, "nccl", (shapes, fused), str(d))[0]
    assert res[False][1] == 0 and res[True][1] > 0
    for a, b in zip(res[False][0], res[True][0]):
        assert (a - b).abs().max().item() < 2e-3
