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
