"""Cooperative scheduling of optimizer tasks.

A task is a Python generator that yields whenever it has put a collective in flight.  The
runtime keeps a bounded window of tasks alive and advances them round-robin, so the host keeps
issuing compute for one bucket while another bucket's collective runs on its own stream
(the role of dion/opt_utils.py:97-163 in the reference).
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Generator, Iterable, Iterator, Optional


class AsyncTask:
    """Wraps a generator and runs it up to its first yield on construction."""

    def __init__(self, generator: Generator[None, None, None]):
        self._gen = generator
        self._alive = True
        self.run()

    def run(self) -> bool:
        """Advance to the next yield.  Returns False once the generator has finished."""
        if not self._alive:
            return False
        try:
            next(self._gen)
        except StopIteration:
            self._alive = False
        return self._alive


class AsyncRuntime:
    """Runs tasks produced lazily by ``task_gen`` with at most ``max_concurrent_tasks`` alive."""

    def __init__(self, task_gen: Iterable[AsyncTask], max_concurrent_tasks: int):
        if max_concurrent_tasks <= 0:
            raise ValueError(f"{max_concurrent_tasks=} cannot be <= 0")
        self._source: Iterator[AsyncTask] = iter(task_gen)
        self._window = max_concurrent_tasks

    def run(self) -> None:
        live: Deque[AsyncTask] = deque()
        exhausted = False
        while not exhausted or live:
            # Start one new task per sweep while there is room (creating it runs its first leg).
            if not exhausted and len(live) < self._window:
                new: Optional[AsyncTask] = next(self._source, None)
                if new is None:
                    exhausted = True
            else:
                new = None
            # Advance the older tasks by one leg each, oldest first.
            for _ in range(len(live)):
                task = live.popleft()
                if task.run():
                    live.append(task)
            if new is not None and new._alive:
                live.append(new)


def run_to_completion(gen: Generator):
    """Drive a task generator synchronously and return its ``return`` value."""
    try:
        while True:
            next(gen)
    except StopIteration as stop:
        return stop.value
