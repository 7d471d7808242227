"""Multi-process CPU (gloo) runs of the distributed code paths, compared with single-process
runs of the same optimizers."""
import pytest
import torch
import torch.distributed as dist

import dion_b200
from tests.dist_utils import run_ranks

SHAPES = ((16, 32), (16, 32), (16, 32), (32, 16), (32, 16))


def _grads(step, shapes):
    g = torch.Generator().manual_seed(100 + step)
    return [torch.randn(*s, generator=g) for s in shapes]


def _weights(shapes):
    g = torch.Generator().manual_seed(7)
    return [torch.randn(*s, generator=g) for s in shapes]


def _single(name, kw, shapes=SHAPES, steps=2):
    ps = [torch.nn.Parameter(w) for w in _weights(shapes)]
    opt = getattr(dion_b200, name)([dict(params=ps)], lr=0.1, **kw)
    for s in range(steps):
        for p, g in zip(ps, _grads(s, shapes)):
            p.grad = g
        opt.step()
    return [p.detach().clone() for p in ps]


def _sharded_worker(rank, world, name, kw, shapes, steps, shard_dim):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (world,))
    ps = [torch.nn.Parameter(distribute_tensor(w, mesh, [Shard(shard_dim)])) for w in _weights(shapes)]
    opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=mesh, lr=0.1, **kw)
    for s in range(steps):
        for p, g in zip(ps, _grads(s, shapes)):
            p.grad = distribute_tensor(g, mesh, [Shard(shard_dim)])
        opt.step()
    full = [p.detach().full_tensor().clone() for p in ps]
    return full if rank == 0 else None


def _replicated_worker(rank, world, name, kw, shapes, steps):
    ps = [torch.nn.Parameter(w) for w in _weights(shapes)]
    opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=dist.group.WORLD, lr=0.1, **kw)
    for s in range(steps):
        for p, g in zip(ps, _grads(s, shapes)):
            p.grad = g
        opt.step()
    return [p.detach().clone() for p in ps] if rank == 0 else None


SHARDED_CASES = [
    ("Muon", dict(nesterov=True), 0, 1e-6),               # layout-invariant
    ("Muon", dict(nesterov=True), 1, 1e-6),
    ("NorMuon", dict(), 0, 2e-2),                          # per-shard Frobenius norms
    ("Dion2", dict(selection_scope="global"), 0, 5e-4),    # exact whole-matrix top-k
    ("Dion2", dict(selection_scope="global"), 1, 5e-4),
    ("NorDion2", dict(selection_scope="global", fraction=1.0), 0, 2e-2),
    ("Dion2", dict(fraction=1.0), 0, 5e-4),              # local scope, everything selected
    ("Dion2", dict(fraction=1.0), 1, 5e-4),
]


WIDE, TALL = ((16, 32),) * 3, ((32, 16),) * 3


def _case_shapes(name, sd):
    # Dion2 selects along the sharded dim when sharded and along the shorter dim otherwise; the
    # two agree for wide matrices sharded by rows and tall matrices sharded by columns.
    if name == "Dion2":
        return WIDE if sd == 0 else TALL
    return SHAPES


def _many_sharded(rank, world, cases, shapes, steps):
    return [_sharded_worker(rank, world, n, kw, _case_shapes(n, sd), steps, sd)
            for n, kw, sd, _ in cases]


def _many_replicated(rank, world, names, shapes, steps):
    return [_replicated_worker(rank, world, n, {}, shapes, steps) for n in names]


def test_sharded_matches_single_process(tmp_path):
    outs = run_ranks(_many_sharded, 2, "gloo", (SHARDED_CASES, SHAPES, 2), str(tmp_path))[0]
    for (name, kw, sd, tol), out in zip(SHARDED_CASES, outs):
        for a, b in zip(_single(name, kw, _case_shapes(name, sd)), out):
            assert (a - b).abs().max().item() <= tol, (name, sd)


def test_replicated_matches_single_process(tmp_path):
    names = ["Muon", "NorMuon", "Dion2", "NorDion2"]
    outs = run_ranks(_many_replicated, 2, "gloo", (names, SHAPES, 2), str(tmp_path))[0]
    for name, out in zip(names, outs):
        for a, b in zip(_single(name, {}), out):
            assert (a - b).abs().max().item() <= 1e-6, name


def _eight_rank_worker(rank, world):
    shapes = ((24, 16),) * 3 + ((16, 40),) * 11      # fewer and more matrices than ranks
    a = _sharded_worker(rank, world, "Muon", dict(nesterov=True), shapes, 2, 0)
    b = _sharded_worker(rank, world, "Muon", dict(nesterov=True), shapes, 2, 1)
    wide = ((8, 24),) * 3 + ((16, 40),) * 11      # Dion2 by rows: sharded and single agree if wide
    c = _sharded_worker(rank, world, "Dion2", dict(selection_scope="global"), wide, 2, 0)
    d = _replicated_worker(rank, world, "Dion2", {}, shapes, 2)
    return (a, b, c, d) if rank == 0 else None


def test_eight_ranks_match_single_process(tmp_path):
    """World size 8 (one node of B200s): buckets with fewer and with more matrices than ranks,
    rows (24, 16) and columns (16, 40) that leave 3-, 2- or 5-wide shards, sharded by either
    dimension or replicated with the work dealt out."""
    shapes = ((24, 16),) * 3 + ((16, 40),) * 11
    wide = ((8, 24),) * 3 + ((16, 40),) * 11
    a, b, c, d = run_ranks(_eight_rank_worker, 8, "gloo", (), str(tmp_path))[0]
    for ref, out, tol in ((_single("Muon", dict(nesterov=True), shapes), a, 1e-6),
                          (_single("Muon", dict(nesterov=True), shapes), b, 1e-6),
                          (_single("Dion2", dict(selection_scope="global"), wide), c, 5e-4),
                          (_single("Dion2", {}, shapes), d, 1e-6)):
        for x, y in zip(ref, out):
            assert x.shape == y.shape and (x - y).abs().max().item() <= tol


def _uneven_worker(rank, world):
    shapes = ((3, 8), (3, 8), (3, 8))  # 3 rows over 4 ranks: one rank holds nothing
    a = _sharded_worker(rank, world, "Muon", {}, shapes, 2, 0)
    b = _sharded_worker(rank, world, "Dion2", dict(selection_scope="global"), shapes, 2, 0)
    c = _sharded_worker(rank, world, "Dion2", dict(fraction=0.5), ((6, 8), (6, 8)), 2, 0)
    return (a, b, c) if rank == 0 else None


def test_uneven_and_empty_shards_do_not_hang(tmp_path):
    shapes = ((3, 8), (3, 8), (3, 8))
    a, b, c = run_ranks(_uneven_worker, 4, "gloo", (), str(tmp_path))[0]
    for ref, out in ((_single("Muon", {}, shapes), a),
                     (_single("Dion2", dict(selection_scope="global"), shapes), b)):
        for x, y in zip(ref, out):
            assert x.shape == y.shape and (x - y).abs().max().item() <= 5e-4
    assert all(torch.isfinite(t).all() for t in c)  # local scope with short shards


def _dion_worker(rank, world, mode, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    shapes = ((32, 64), (32, 64), (64, 32), (64, 32))
    torch.manual_seed(0)
    if mode == "ddp":
        ps = [torch.nn.Parameter(w) for w in _weights(shapes)]
        opt = dion_b200.Dion([dict(params=ps)], replicate_mesh=dist.group.WORLD,
                             replicate_mesh_grad_sync=True, rank_fraction=0.25, lr=0.1)
        mk = lambda g: g  # noqa: E731
    else:
        if mode == "fsdp":
            mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fs",))
            opt_kw = dict(outer_shard_mesh=mesh["fs"])
            place = lambda i: [Shard(0)]  # noqa: E731
        elif mode == "tp":
            mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
            opt_kw = dict(inner_shard_mesh=mesh["tp"])
            place = lambda i: [Shard(0)] if i < 2 else [Shard(1)]  # noqa: E731
        else:  # fsdp x tp on a 2x2 mesh
            mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("fs", "tp"))
            opt_kw = dict(outer_shard_mesh=mesh["fs"], inner_shard_mesh=mesh["tp"])
            place = lambda i: [Shard(1), Shard(0)] if i < 2 else [Shard(0), Shard(1)]  # noqa: E731
        ps = [torch.nn.Parameter(distribute_tensor(w, mesh, place(i)))
              for i, w in enumerate(_weights(shapes))]
        opt = dion_b200.Dion([dict(params=ps)], rank_fraction=0.25, lr=0.1, **opt_kw)
        mk = lambda g, i=None: g  # noqa: E731
    for s in range(steps):
        for i, (p, g) in enumerate(zip(ps, _grads(s, shapes))):
            p.grad = g if mode == "ddp" else distribute_tensor(g, p.device_mesh, p.placements)
        opt.step()
    if hasattr(opt, "synchronize_for_checkpoint"):
        opt.synchronize_for_checkpoint()
    out = [p.detach().full_tensor().clone() if mode != "ddp" else p.detach().clone() for p in ps]
    qs = [tuple(opt.state[p]["Q"].shape) for p in ps]
    return (out, qs) if rank == 0 else None


def _dion_modes_worker(rank, world, modes):
    return [_dion_worker(rank, world, m, 3) for m in modes]


@pytest.mark.parametrize("modes,world", [(("ddp", "fsdp", "tp"), 2), (("fsdp_tp",), 4)])
def test_dion_distributed_modes_run_and_descend(tmp_path, modes, world):
    results = run_ranks(_dion_modes_worker, world, "gloo", (modes,), str(tmp_path))[0]
    start = _weights(((32, 64), (32, 64), (64, 32), (64, 32)))
    for mode, (out, qs) in zip(modes, results):
        for a, b in zip(start, out):
            assert a.shape == b.shape and torch.isfinite(b).all(), mode
            assert (a - b).abs().max().item() > 0, mode
        assert qs[0][1] == 8, mode  # r = ceil(0.25 * 32)


def _wrapper_tensor_worker(rank, world):
    """Results of functional collectives are lazy wrapper tensors; code that hands addresses to
    kernels has to complete and unwrap them first, without cutting the autograd graph."""
    import torch.distributed._functional_collectives as fc
    from dion_b200.models import functional as Fn
    from dion_b200.utils.tensors import is_plain_tensor, materialize, to_local, unwrap

    x = torch.full((4, 8), float(rank + 1), requires_grad=True)
    y = fc.all_reduce(x * 2.0, "sum", dist.group.WORLD)
    assert isinstance(y, fc.AsyncCollectiveTensor) and not is_plain_tensor(y)
    z = materialize(y)
    assert is_plain_tensor(z)
    assert torch.equal(z.detach(), torch.full((4, 8), 2.0 * sum(range(1, world + 1))))
    z.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all() and x.grad.abs().sum() > 0
    w = fc.all_reduce(torch.ones(3), "sum", dist.group.WORLD)
    assert is_plain_tensor(unwrap(w)) and is_plain_tensor(to_local([w])[0])
    # The model functions accept the wrapper (fallback arithmetic on CPU) and differentiate.
    h = fc.all_reduce(torch.randn(2, 4, 16), "sum", dist.group.WORLD)
    out = Fn.rms_norm(h)
    assert is_plain_tensor(out) and out.shape == (2, 4, 16)
    return True


def test_functional_collective_results_are_unwrapped(tmp_path):
    run_ranks(_wrapper_tensor_worker, 2)


def _hsdp_worker(rank, world, cases):
    """Hybrid sharding: parameters replicated over ``dp`` and row-sharded over ``fs``; the
    optimizer is given the ``fs`` sub-mesh (as the trainer does), replicas compute redundantly."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Replicate, Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp", "fs"))
    placements = [Replicate(), Shard(0)]
    outs = []
    for name, kw, _ in cases:
        shapes = _case_shapes(name, 0)
        ps = [torch.nn.Parameter(distribute_tensor(w, mesh, placements)) for w in _weights(shapes)]
        opt = getattr(dion_b200, name)([dict(params=ps)], distributed_mesh=mesh["fs"], lr=0.1, **kw)
        for s in range(2):
            for p, g in zip(ps, _grads(s, shapes)):
                p.grad = distribute_tensor(g, mesh, placements)
            opt.step()
        outs.append([p.detach().full_tensor().clone() for p in ps])  # collective: on every rank
    return outs if rank == 0 else None


HSDP_CASES = [("Muon", {}, 1e-6), ("NorMuon", {}, 2e-2),
              ("Dion2", dict(selection_scope="global"), 5e-4)]


def test_hybrid_sharded_mesh_matches_single_process(tmp_path):
    outs = run_ranks(_hsdp_worker, 4, "gloo", (HSDP_CASES,), str(tmp_path))[0]
    for (name, kw, tol), out in zip(HSDP_CASES, outs):
        for a, b in zip(_single(name, kw, _case_shapes(name, 0)), out):
            assert (a - b).abs().max().item() <= tol, name


def _flattened_mesh_worker(rank, world):
    """Several mesh dimensions (data x context parallel) flattened into the one sharding mesh
    that the optimizer is given (the reference documents this use, README.md:317-337)."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp", "cp"))
    flat = mesh["dp", "cp"]._flatten("dp_cp")
    ps = [torch.nn.Parameter(distribute_tensor(w, flat, [Shard(0)])) for w in _weights(SHAPES)]
    opt = dion_b200.Muon([dict(params=ps)], distributed_mesh=flat, lr=0.1)
    for s in range(2):
        for p, g in zip(ps, _grads(s, SHAPES)):
            p.grad = distribute_tensor(g, flat, [Shard(0)])
        opt.step()
    full = [p.detach().full_tensor().clone() for p in ps]
    return full if rank == 0 else None


def test_flattened_mesh_matches_single_process(tmp_path):
    out = run_ranks(_flattened_mesh_worker, 4, "gloo", (), str(tmp_path))[0]
    for a, b in zip(_single("Muon", {}), out):
        assert (a - b).abs().max().item() <= 1e-6


def _compressed_sync_worker(rank, world, steps):
    """Data-parallel ranks with different gradients: (a) Dion synchronizes only the low-rank
    factors (decoupled momentum), (b) gradients are averaged first and Dion synchronizes nothing.
    The weights agree up to rounding; (a)'s momenta differ between ranks until
    ``synchronize_for_checkpoint`` averages them (reference README, "Compressed Data-Parallel
    Gradient Sync for Dion")."""
    shapes = ((32, 64), (64, 32), (48, 48))   # rank 24 of 48 x 48 saves nothing: not compressed
    outs = {}
    for mode in ("compressed", "averaged"):
        ps = [torch.nn.Parameter(w) for w in _weights(shapes)]
        torch.manual_seed(0)   # same random Q on every rank and in both runs
        opt = dion_b200.Dion([dict(params=ps)], replicate_mesh=dist.group.WORLD,
                             replicate_mesh_grad_sync=(mode == "compressed"),
                             rank_fraction=0.5, lr=0.05)
        for s in range(steps):
            g = torch.Generator().manual_seed(1000 * s + rank)
            for p in ps:
                p.grad = torch.randn(p.shape, generator=g)
                if mode == "averaged":
                    dist.all_reduce(p.grad)
                    p.grad /= world
            opt.step()
        moms = [opt.state[p]["momentum"].clone() for p in ps]
        spread = []
        for m in moms:
            lo, hi = m.clone(), m.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            spread.append((hi - lo).abs().max().item())
        opt.synchronize_for_checkpoint()
        after = []
        for p in ps:
            m = opt.state[p]["momentum"]
            lo, hi = m.clone(), m.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            after.append((hi - lo).abs().max().item())
        outs[mode] = ([p.detach().clone() for p in ps], spread, after,
                      [opt.state[p]["momentum"].clone() for p in ps])
    return outs if rank == 0 else None


def test_compressed_data_parallel_sync_equals_gradient_averaging(tmp_path):
    outs = run_ranks(_compressed_sync_worker, 2, "gloo", (3,), str(tmp_path))[0]
    wa, spread_a, after_a, mom_a = outs["compressed"]
    wb, spread_b, after_b, mom_b = outs["averaged"]
    for a, b in zip(wa, wb):
        assert (a - b).abs().max().item() < 1e-5
    assert min(spread_a[:2]) > 1e-3      # decoupled momentum really differs between ranks
    assert spread_a[2] == 0.0            # (m + n) r >= m n: that gradient is all-reduced in full
    assert max(spread_b) == 0.0          # with averaged gradients it never does
    assert max(after_a) < 1e-6           # and the checkpoint synchronization removes the spread
    for a, b in zip(mom_a, mom_b):       # the averaged decoupled momentum is the coupled one
        assert (a - b).abs().max().item() < 1e-5


def _bad_sharding_worker(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("fs", "tp"))
    w = torch.randn(32, 64)
    seen = []
    # Dion: FSDP and TP must shard different matrix dimensions.
    p = torch.nn.Parameter(distribute_tensor(w, mesh, [Shard(0), Shard(0)]))
    try:
        opt = dion_b200.Dion([dict(params=[p])], outer_shard_mesh=mesh["fs"],
                             inner_shard_mesh=mesh["tp"], lr=0.1)
        p.grad = distribute_tensor(torch.randn(32, 64), mesh, [Shard(0), Shard(0)])
        opt.step()
        seen.append("accepted")
    except RuntimeError as exc:
        seen.append(str(exc))
    # Megabatch optimizers: one sharded matrix dimension at most.
    q = torch.nn.Parameter(distribute_tensor(w, mesh, [Shard(0), Shard(1)]))
    try:
        opt = dion_b200.Muon([dict(params=[q])], distributed_mesh=mesh["fs"], lr=0.1)
        q.grad = distribute_tensor(torch.randn(32, 64), mesh, [Shard(0), Shard(1)])
        opt.step()
        seen.append("accepted")
    except NotImplementedError as exc:
        seen.append(str(exc))
    return seen if rank == 0 else None


def test_unsupported_shardings_are_rejected_on_every_rank(tmp_path):
    dion_msg, muon_msg = run_ranks(_bad_sharding_worker, 4, "gloo", (), str(tmp_path))[0]
    assert "double-sharded" in dion_msg
    assert "multiple sharded dimensions" in muon_msg


def _muon_reference_worker(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (world,))
    ps = [torch.nn.Parameter(distribute_tensor(w, mesh, [Shard(0)])) for w in _weights(SHAPES)]
    opt = dion_b200.MuonReference([dict(params=ps)], lr=0.1)
    for s in range(2):
        for p, g in zip(ps, _grads(s, SHAPES)):
            p.grad = distribute_tensor(g, mesh, [Shard(0)])
        opt.step()
    full = [p.detach().full_tensor().clone() for p in ps]
    return full if rank == 0 else None


def test_muon_reference_on_sharded_parameters_matches_single_process(tmp_path):
    """The all-gather variant (every rank assembles each full matrix) gives the single-process
    result on row-sharded DTensor parameters."""
    out = run_ranks(_muon_reference_worker, 2, "gloo", (), str(tmp_path))[0]
    for a, b in zip(_single("MuonReference", {}), out):
        assert (a - b).abs().max().item() <= 1e-6


DION_SHAPES = ((32, 64), (32, 64), (64, 32), (64, 32))


def _dion_common_q(opt, ps, distribute=None):
    """Create Dion's state now and replace every ``Q`` by (the shards of) one fixed full matrix,
    so that runs with different layouts start from the same point."""
    group = opt.param_groups[0]
    gen = torch.Generator().manual_seed(11)
    for p in ps:
        opt._init_opt_state_dion(p, opt.state[p], group["rank_fraction"], group["rank_multiple_of"])
        q = opt.state[p]["Q"]
        full = torch.randn(tuple(q.shape), generator=gen)
        opt.state[p]["Q"] = full if distribute is None else distribute(full, q)


def _dion_single(transposed, steps=3, cls="Dion"):
    ps = [torch.nn.Parameter(w) for w in _weights(DION_SHAPES)]
    opt = getattr(dion_b200, cls)([dict(params=ps)], rank_fraction=0.25, lr=0.1)
    for p, t in zip(ps, transposed):     # iterate on the side the sharded layout iterates on
        opt._get_dion_param_config(p).is_transposed = t
    _dion_common_q(opt, ps)
    for s in range(steps):
        for p, g in zip(ps, _grads(s, DION_SHAPES)):
            p.grad = g
        opt.step()
    return [p.detach().clone() for p in ps]


def _dion_layout_worker(rank, world, mode, steps, cls="Dion"):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    if mode == "fsdp":
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fs",))
        kw, place = dict(outer_shard_mesh=mesh["fs"]), lambda i: [Shard(0)]  # noqa: E731
    elif mode == "tp":
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
        kw = dict(inner_shard_mesh=mesh["tp"])
        place = lambda i: [Shard(0)] if i < 2 else [Shard(1)]  # noqa: E731
    elif mode == "fsdp_tp":
        mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("fs", "tp"))
        kw = dict(outer_shard_mesh=mesh["fs"], inner_shard_mesh=mesh["tp"])
        place = lambda i: [Shard(1), Shard(0)] if i < 2 else [Shard(0), Shard(1)]  # noqa: E731
    else:   # dp x fs x tp on eight ranks: replicas synchronize the low-rank factors
        full_mesh = init_device_mesh("cpu", (2, 2, 2), mesh_dim_names=("dp", "fs", "tp"))
        mesh = full_mesh["fs", "tp"]
        kw = dict(replicate_mesh=full_mesh["dp"], outer_shard_mesh=full_mesh["fs"],
                  inner_shard_mesh=full_mesh["tp"], replicate_mesh_grad_sync=True)
        place = lambda i: [Shard(1), Shard(0)] if i < 2 else [Shard(0), Shard(1)]  # noqa: E731
    ps = [torch.nn.Parameter(distribute_tensor(w, mesh, place(i)))
          for i, w in enumerate(_weights(DION_SHAPES))]
    opt = getattr(dion_b200, cls)([dict(params=ps)], rank_fraction=0.25, lr=0.1, **kw)
    _dion_common_q(opt, ps, lambda full, q: distribute_tensor(full, q.device_mesh, q.placements))
    for s in range(steps):
        for p, g in zip(ps, _grads(s, DION_SHAPES)):
            p.grad = distribute_tensor(g, p.device_mesh, p.placements)
        opt.step()
    full = [p.detach().full_tensor().clone() for p in ps]
    transposed = [opt._get_dion_param_config(p).is_transposed for p in ps]
    return (full, transposed) if rank == 0 else None


@pytest.mark.parametrize("cls", ["Dion", "DionReference"])
@pytest.mark.parametrize("mode,world", [("fsdp", 2), ("tp", 2), ("fsdp_tp", 4),
                                        ("dp_fsdp_tp", 8)])
def test_dion_sharded_layouts_equal_the_single_process_run(tmp_path, mode, world, cls):
    """Legacy Dion on FSDP, tensor-parallel and FSDP x TP shards follows the single-process
    trajectory when both start from the same ``Q`` and iterate on the same side of the matrix
    (a sharded layout fixes that side by which dimension it shards; the sketch of the randomized
    QR differs between the runs and must not matter)."""
    out, transposed = run_ranks(_dion_layout_worker, world, "gloo", (mode, 3, cls),
                                str(tmp_path))[0]
    for a, b in zip(_dion_single(transposed, cls=cls), out):
        assert (a - b).abs().max().item() < 1e-4, mode


def test_batched_and_unbatched_dion_agree_from_a_common_start():
    """The batched optimizer and the one-matrix-at-a-time variant are the same algorithm: from a
    common ``Q`` (and on the same side of each matrix) their weights agree to rounding, although
    their randomized sketches differ."""
    for sides in ([False] * 4, [True, True, False, False]):
        a = _dion_single(sides, cls="Dion")
        b = _dion_single(sides, cls="DionReference")
        for x, y in zip(a, b):
            assert (x - y).abs().max().item() < 1e-5


def _submatrix_exchange_worker(rank, world):
    """Local-scope Dion2 exchanges only the ``k`` selected rows of each shard.  Forcing the
    exchange to carry whole (zero-padded) shards instead must give the same update (the reference
    makes this comparison by patching its exchange function,
    tests/test_dion2_selection_scope.py:243-256)."""
    import dion_b200.optim.dion2 as d2
    kw = dict(fraction=0.5)
    lean = _sharded_worker(rank, world, "Dion2", kw, WIDE, 2, 0)
    real_plan = d2.MegabatchPlan
    seen = []

    def whole_shards(*args, **kwargs):
        seen.append(kwargs.get("local_comm_size"))
        kwargs["local_comm_size"] = None
        return real_plan(*args, **kwargs)

    d2.MegabatchPlan = whole_shards
    try:
        padded = _sharded_worker(rank, world, "Dion2", kw, WIDE, 2, 0)
    finally:
        d2.MegabatchPlan = real_plan
    return (lean, padded, seen) if rank == 0 else None


def test_dion2_submatrix_exchange_equals_whole_shard_exchange(tmp_path):
    lean, padded, seen = run_ranks(_submatrix_exchange_worker, 2, "gloo", (), str(tmp_path))[0]
    assert seen and all(k == 4 for k in seen)          # 8 local rows, half of them selected
    for a, b in zip(lean, padded):
        assert (a - b).abs().max().item() <= 1e-3


def _keller_jordan_worker(rank, world):
    from dion_b200 import MuonKellerJordan
    ps = [torch.nn.Parameter(w) for w in _weights(SHAPES)]
    opt = MuonKellerJordan(ps, lr=0.05)
    for s in range(2):
        for p, g in zip(ps, _grads(s, SHAPES)):
            p.grad = g
        opt.step()
    return [p.detach().clone() for p in ps] if rank == 0 else None


def test_keller_jordan_muon_by_formula_and_across_ranks(tmp_path, monkeypatch):
    """``MuonKellerJordan``: momentum, Nesterov look-ahead, five fixed-coefficient Newton-Schulz
    steps, update scaled by ``sqrt(rows / cols)``; with several ranks the parameters are dealt
    round-robin and one all-reduce shares the updates, which changes nothing in the result."""
    from dion_b200 import MuonKellerJordan
    from dion_b200.optim.muon_reference import zeropower_via_newtonschulz5
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("RANK", "0")
    ps = [torch.nn.Parameter(w) for w in _weights(SHAPES)]
    want = [w.clone() for w in _weights(SHAPES)]
    bufs = [torch.zeros_like(w) for w in want]
    opt = MuonKellerJordan(ps, lr=0.05, momentum=0.9)
    for s in range(2):
        for i, (p, g) in enumerate(zip(ps, _grads(s, SHAPES))):
            p.grad = g
            bufs[i].mul_(0.9).add_(g)
            look = g + 0.9 * bufs[i]
            u = zeropower_via_newtonschulz5(look, steps=5) * (g.size(0) / g.size(1)) ** 0.5
            want[i] -= 0.05 * u.bfloat16().float()      # updates travel as bf16
        opt.step()
    for a, b in zip(want, ps):
        assert torch.allclose(a, b.detach(), atol=1e-6)
    single = [p.detach().clone() for p in ps]
    # two ranks with default momentum against one process with the same settings
    ps1 = [torch.nn.Parameter(w) for w in _weights(SHAPES)]
    opt1 = MuonKellerJordan(ps1, lr=0.05)
    for s in range(2):
        for p, g in zip(ps1, _grads(s, SHAPES)):
            p.grad = g
        opt1.step()
    out = run_ranks(_keller_jordan_worker, 2, "gloo", (), str(tmp_path))[0]
    for a, b in zip(ps1, out):
        assert torch.equal(a.detach(), b)
    assert any(not torch.equal(a, b.detach()) for a, b in zip(single, ps1))   # momentum matters
