"""Host-side building blocks: the cooperative task runtime and the step arena."""
import pytest
import torch

from dion_b200.parallel.async_runtime import AsyncRuntime, AsyncTask, run_to_completion
from dion_b200.utils.arena import StepArena, alloc


def _task(name, legs, log):
    def gen():
        for leg in range(legs):
            log.append((name, leg))
            yield
        log.append((name, "done"))
    return gen()


def test_tasks_overlap_within_the_window_and_all_finish():
    log = []
    source = (AsyncTask(_task(n, 2, log)) for n in "abcd")
    AsyncRuntime(source, max_concurrent_tasks=2).run()
    # every task ran all its legs, in order, exactly once
    for n in "abcd":
        assert [e for e in log if e[0] == n] == [(n, 0), (n, 1), (n, "done")]
    pos = {e: i for i, e in enumerate(log)}
    # the second task starts before the first one finishes (its collective would be in flight)
    assert pos[("b", 0)] < pos[("a", "done")]
    # but the window bounds how many are alive: "c" starts only after "a" is done
    assert pos[("c", 0)] > pos[("a", "done")]
    # tasks are created lazily: with a window of one they run strictly one after the other
    log.clear()
    AsyncRuntime((AsyncTask(_task(n, 2, log)) for n in "xy"), max_concurrent_tasks=1).run()
    assert log.index(("y", 0)) > log.index(("x", "done"))


def test_runtime_rejects_an_empty_window_and_handles_trivial_tasks():
    with pytest.raises(ValueError):
        AsyncRuntime(iter(()), max_concurrent_tasks=0)
    log = []
    AsyncRuntime((AsyncTask(_task(n, 0, log)) for n in "pq"), max_concurrent_tasks=3).run()
    assert log == [("p", "done"), ("q", "done")]       # tasks that never yield complete at once
    AsyncRuntime(iter(()), max_concurrent_tasks=2).run()   # no tasks at all

    def returns_value():
        yield
        return 42
    assert run_to_completion(returns_value()) == 42


def test_arena_hands_out_the_same_addresses_every_step():
    arena = StepArena()
    dev = torch.device("cpu")

    def one_step():
        arena.reset()
        a = arena.alloc((4, 8), torch.float32, dev)
        b = arena.alloc((3,), torch.bfloat16, dev, zero=True)
        c = arena.alloc((0, 5), torch.float32, dev)
        return a, b, c

    a1, b1, c1 = one_step()
    a1.fill_(7.0)
    a2, b2, c2 = one_step()
    assert (a1.data_ptr(), b1.data_ptr()) == (a2.data_ptr(), b2.data_ptr())
    assert a2.shape == (4, 8) and c2.shape == (0, 5) and float(b2.abs().sum()) == 0.0
    assert float(a2[0, 0]) == 7.0                    # not cleared unless asked
    before = arena.bytes()
    arena.reset()
    big = arena.alloc((16, 8), torch.float32, dev)   # a slot that is too small is replaced
    assert big.numel() == 128 and arena.bytes() > before
    arena.reset()
    assert arena.alloc((4, 8), torch.float32, dev).data_ptr() == big.data_ptr()
    plain = alloc(None, (2, 2), torch.float32, dev, zero=True)
    assert plain.shape == (2, 2) and float(plain.sum()) == 0.0


def test_fused_exchange_eligibility_uses_only_rank_independent_facts(monkeypatch):
    """Which buckets take the peer-memory exchange: evenly row-sharded 2-D matrices with a column
    count the TMA rules allow, a built-in Newton-Schulz driver and 2-8 ranks on one node; anything
    else keeps the collective path.  The decision reads no local shard size, so every rank of an
    uneven layout decides alike."""
    from dion_b200.ops import newton_schulz as NS
    from dion_b200.parallel import fused_exchange as FX
    monkeypatch.setattr(FX.symm, "symmetric_memory_available", lambda pg: True)
    monkeypatch.delenv("DION_B200_FUSED_EXCHANGE", raising=False)
    pg = object()
    ok = dict(local_shape=(256, 1024), comm_dim=-2, global_rows=1024, world=4, pg=pg,
              ns_func=NS.polar_express, flatten=False, split_sizes=None)
    assert FX.eligible(**ok)
    for change in (dict(comm_dim=-1),                      # column shards
                   dict(local_shape=(3, 256, 1024)),       # batched parameter
                   dict(global_rows=1022),                 # uneven row shards
                   dict(global_rows=None),
                   dict(local_shape=(256, 1020)),          # row length not a multiple of 8
                   dict(world=1), dict(world=16),
                   dict(pg=None),
                   dict(flatten=True), dict(split_sizes=(512, 512)),
                   dict(ns_func=lambda X, epsilon: X),      # user driver: iteration unknown
                   dict(ns_func=NS.gram_newton_schulz)):
        assert not FX.eligible(**{**ok, **change}), change
    # the local shard size itself plays no part (an empty shard on one rank changes nothing)
    assert FX.eligible(**{**ok, "local_shape": (0, 1024)})
    monkeypatch.setenv("DION_B200_FUSED_EXCHANGE", "0")
    assert not FX.eligible(**ok)
    monkeypatch.delenv("DION_B200_FUSED_EXCHANGE")
    monkeypatch.setattr(FX.symm, "symmetric_memory_available", lambda pg: False)
    assert not FX.eligible(**ok)


def test_fused_exchange_eligibility_of_column_shards(monkeypatch):
    """Column shards are taken only by callers that ask (``allow_columns``), only when every
    rank holds the same whole number of 32-column chunks and nothing else shards that dimension;
    the fused low-rank synchronisation of legacy Dion is opt-in."""
    from dion_b200.ops import newton_schulz as NS
    from dion_b200.parallel import fused_exchange as FX
    from dion_b200.parallel import lowrank_sync as LS
    monkeypatch.setattr(FX.symm, "symmetric_memory_available", lambda pg: True)
    monkeypatch.delenv("DION_B200_FUSED_EXCHANGE", raising=False)
    ok = dict(local_shape=(512, 256), comm_dim=-1, global_rows=1024, world=4, pg=object(),
              ns_func=NS.newton_schulz_quintic, flatten=False, split_sizes=None)
    assert not FX.eligible(**ok)
    assert FX.eligible(**ok, allow_columns=True)
    for change in (dict(global_rows=1028, local_shape=(512, 257)),   # ragged blocks
                   dict(global_rows=960, local_shape=(512, 240)),    # 240 is no multiple of 32
                   dict(local_shape=(512, 128)),                     # also sharded elsewhere
                   dict(local_shape=(516, 256)),                     # rows: Gram is a TMA operand
                   dict(flatten=True)):
        assert not FX.eligible(**{**ok, **change}, allow_columns=True), change
    monkeypatch.delenv("DION_B200_FUSED_LOWRANK", raising=False)
    assert not LS.fused_lowrank_enabled()
    monkeypatch.setenv("DION_B200_FUSED_LOWRANK", "1")
    assert LS.fused_lowrank_enabled()


def test_megabatch_plan_modes_padding_and_argument_errors():
    """Layout decisions of one megabatch round, without communication: mode, per-rank counts,
    padded shard sizes, where each input is written, and the argument errors (the reference checks
    the missing ``global_comm_dim_size`` error with a one-rank gloo group,
    tests/test_megabatch_empty_shard.py:116-143)."""
    from dion_b200.ops import newton_schulz as NS
    from dion_b200.parallel.megabatch import MegabatchPlan
    dev = torch.device("cpu")
    pg = object()                                            # never used for communication here
    single = MegabatchPlan((8, 16), 3, dev, None, 0, 1, None)
    assert (single.mode, single.per_rank, single.n_total) == ("single", 3, 3)
    views = single.input_views()
    for i, v in enumerate(views):
        v.copy_(torch.randn(8, 16))
    out = run_to_completion(single.run(NS.polar_express, False, 1e-6))
    assert out.shape == (3, 8, 16) and torch.isfinite(out.float()).all()

    rep = MegabatchPlan((8, 16), 5, dev, None, 1, 4, pg)    # DDP: 5 matrices over 4 ranks
    assert (rep.mode, rep.per_rank, rep.n_total) == ("replicated", 2, 8)
    owned = [i for i, v in enumerate(rep.input_views()) if v is not None]
    assert owned == [2, 3]                                   # rank 1 owns matrices 2 and 3

    sh = MegabatchPlan((3, 16), 6, dev, -2, 0, 4, pg, global_comm_dim_size=10)
    assert sh.mode == "sharded" and sh.padded_local == 3 and sh.padded_shape == (3, 16)
    short = MegabatchPlan((1, 16), 6, dev, -2, 3, 4, pg, global_comm_dim_size=10)   # last rank
    assert short.padded_shape == (3, 16) and short.input_views()[0].shape == (1, 16)
    empty = MegabatchPlan((0, 16), 2, dev, -2, 3, 4, pg, global_comm_dim_size=3)
    assert empty.padded_shape == (1, 16) and empty.input_views()[1].shape == (0, 16)

    with pytest.raises(ValueError, match="global_comm_dim_size"):
        MegabatchPlan((4, 16), 2, dev, -2, 0, 2, pg)
    with pytest.raises(ValueError, match="negative"):
        MegabatchPlan((4, 16), 2, dev, 0, 0, 2, pg, global_comm_dim_size=8)
    with pytest.raises(RuntimeError, match="padded_local_size"):
        MegabatchPlan((9, 16), 2, dev, -2, 0, 2, pg, global_comm_dim_size=10)
    with pytest.raises(NotImplementedError, match="divisible"):
        MegabatchPlan((5, 16), 2, dev, -2, 0, 2, pg, global_comm_dim_size=9, split_sizes=(4, 5))
    with pytest.raises(NotImplementedError, match="local_comm_size"):
        MegabatchPlan((4, 16), 2, dev, -2, 0, 2, pg, global_comm_dim_size=8, local_comm_size=2,
                      split_sizes=(4, 4))
