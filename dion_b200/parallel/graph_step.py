"""Whole training step as one CUDA graph, with a capturable data-parallel gradient all-reduce.

A small model's step is hundreds of short kernels; launched one by one from Python the GPU idles
between them.  :class:`GraphedTrainStep` records forward, backward, the gradient all-reduce and
the optimizer step once and replays the recording, so a step costs one launch on the host.  The
optimizers of this package are built for that: they read the learning rate from device tensors,
keep their counters on the device and never synchronize with the host (the per-optimizer variant
is ``dion_b200.optim.cuda_graph.CudaGraphOptimizer``, the counterpart of dion/cuda_graph.py in
the reference, which captures ``optimizer.step()`` only).

:class:`BucketedGradSync` is the data-parallel piece: post-accumulate hooks launch one coalesced
NCCL all-reduce per bucket on a side stream as soon as the bucket's last gradient exists, so the
reduction overlaps the rest of backward.  It works eagerly and under stream capture (the side
stream is forked from and joined to the capturing stream with events), which the hook machinery
of ``torch.nn.parallel.DistributedDataParallel`` does not.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from ..utils import trace


class BucketedGradSync:
    """Average gradients over ``process_group`` in buckets, overlapped with backward.

    Parameters are bucketed in reverse registration order (the order in which backward produces
    their gradients).  ``finish()`` must be called after ``backward()``: it joins the side stream
    and re-arms the buckets."""

    def __init__(self, params: Sequence[Tensor], process_group=None, bucket_mb: float = 64.0):
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.params = [p for p in params if p.requires_grad]
        self.buckets: List[List[Tensor]] = []
        limit = int(bucket_mb * (1 << 20))
        cur: List[Tensor] = []
        size = 0
        for p in reversed(self.params):
            cur.append(p)
            size += p.numel() * p.element_size()
            if size >= limit:
                self.buckets.append(cur)
                cur, size = [], 0
        if cur:
            self.buckets.append(cur)
        self._bucket_of: Dict[Tensor, int] = {}
        for bi, bucket in enumerate(self.buckets):
            for p in bucket:
                self._bucket_of[p] = bi
        self._pending = [len(b) for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._stream: Optional[torch.cuda.Stream] = None
        self._handles = []
        self._events: List = []  # (bucket index, event) in launch order on the side stream
        self.active = True       # False: let gradients accumulate locally (like DDP.no_sync)
        self.enabled = self.world > 1
        if self.enabled:
            for p in self.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    # ----------------------------------------------------------------------------------------
    def _on_grad(self, p: Tensor) -> None:
        if not self.active:
            return
        bi = self._bucket_of[p]
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            self._reduce_bucket(bi)

    def _reduce_bucket(self, bi: int) -> None:
        grads = [p.grad for p in self.buckets[bi] if p.grad is not None]
        self._launched[bi] = True
        if not grads:
            return
        if grads[0].is_cuda:
            if self._stream is None:
                self._stream = torch.cuda.Stream(device=grads[0].device)
            # Fork: the side stream starts after everything recorded so far on this stream.
            self._stream.wait_stream(torch.cuda.current_stream(grads[0].device))
            with torch.cuda.stream(self._stream):
                self._all_reduce(grads)
                ev = torch.cuda.Event()
                ev.record(self._stream)
                self._events.append((bi, ev))
        else:
            self._all_reduce(grads)

    def _all_reduce(self, grads: List[Tensor]) -> None:
        nccl = grads[0].is_cuda
        op = dist.ReduceOp.AVG if nccl else dist.ReduceOp.SUM
        manager = getattr(dist, "_coalescing_manager", None)
        if nccl and manager is not None:
            with manager(group=self.pg, async_ops=False):
                for g in grads:
                    dist.all_reduce(g, op=op, group=self.pg)
        else:
            for g in grads:
                dist.all_reduce(g, op=op, group=self.pg)
        if not nccl:
            torch._foreach_div_(grads, float(self.world))

    def finish(self, deferrable: Optional[Sequence[Tensor]] = None) -> bool:
        """Reduce buckets whose parameters did not all receive a gradient this step, make the
        current stream wait for the reductions and re-arm.  With ``deferrable`` (parameters whose
        gradients are not needed until :meth:`join` is called) the wait stops at the last bucket
        that holds any other parameter; returns True when something was left for ``join``."""
        if not self.enabled:
            return False
        for bi in range(len(self.buckets)):
            if not self._launched[bi]:
                self._reduce_bucket(bi)
        self._pending = [len(b) for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        if self._stream is None:
            self._events.clear()
            return False
        cur = torch.cuda.current_stream(self._stream.device)
        if deferrable is not None and self._events:
            later = set(id(p) for p in deferrable)
            needed = None  # position (in launch order) of the last bucket needed right away
            for pos, (bi, _) in enumerate(self._events):
                if any(id(p) not in later for p in self.buckets[bi]):
                    needed = pos
            if needed is None or needed != len(self._events) - 1:
                if needed is not None:
                    cur.wait_event(self._events[needed][1])
                self._events.clear()
                return True
        cur.wait_stream(self._stream)
        self._events.clear()
        return False

    def join(self) -> None:
        """Make the current stream wait for everything :meth:`finish` deferred."""
        if self.enabled and self._stream is not None:
            torch.cuda.current_stream(self._stream.device).wait_stream(self._stream)


class GraphedTrainStep:
    """``loss = step(*inputs)`` runs ``loss_fn(*inputs)`` under autocast, ``backward()``, the
    gradient all-reduce (when ``process_group`` spans more than one rank) and
    ``optimizer.step()``.  The first ``warmup`` calls run eagerly on a side stream, the next one
    is captured, later ones replay the graph.  Inputs are copied into static buffers (so they may
    be pinned host tensors: the copy is the host-to-device transfer); the returned loss is a
    static device tensor that the next call overwrites.

    ``use_graph=False`` keeps the same step eager (for debugging and as the fallback on CPU).
    With ``accumulation_steps = k > 1`` every input carries a leading dimension ``k``: the step
    runs ``k`` forward/backward passes whose gradients accumulate (the loss is their mean) and
    reduces / applies them once.
    """

    def __init__(self, loss_fn: Callable[..., Tensor], params: Sequence[Tensor],
                 optimizer: torch.optim.Optimizer, example_inputs: Sequence[Tensor], *,
                 device: torch.device, process_group=None,
                 autocast_dtype: Optional[torch.dtype] = torch.bfloat16,
                 warmup: int = 3, use_graph: bool = True, bucket_mb: float = 64.0,
                 accumulation_steps: int = 1):
        self.loss_fn = loss_fn
        self.params = [p for p in params]
        self.optimizer = optimizer
        self.device = device
        self.autocast_dtype = autocast_dtype
        self.warmup = max(1, warmup)
        self.use_graph = use_graph and device.type == "cuda"
        if self.use_graph:
            from ..optim.cuda_graph import require_graph_replay_support

            require_graph_replay_support(optimizer, "GraphedTrainStep(use_graph=True)")
        self.sync = BucketedGradSync(self.params, process_group, bucket_mb)
        self._deferrable = self._scalar_group_params(optimizer)
        if accumulation_steps < 1:
            raise ValueError("accumulation_steps must be >= 1")
        self.accumulation_steps = accumulation_steps
        lead = (accumulation_steps,) if accumulation_steps > 1 else ()
        self.static_inputs = [torch.empty(lead + tuple(t.shape), dtype=t.dtype, device=device)
                              for t in example_inputs]
        self.static_loss: Optional[Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._calls = 0
        self._side: Optional[torch.cuda.Stream] = None

    @staticmethod
    def _scalar_group_params(optimizer) -> Optional[List[Tensor]]:
        """Parameters updated by the element-wise algorithms of an optimizer of this package that
        runs them after its matrix tasks (``DistributedOrthoBase.step``); their gradient
        reductions may run past the start of the step."""
        from ..optim.ortho_base import DistributedOrthoBase

        if not isinstance(optimizer, DistributedOrthoBase):
            return None
        out = [p for g in optimizer.param_groups if g.get("algorithm") in ("adamw", "lion")
               for p in g["params"]]
        return out or None

    # ----------------------------------------------------------------------------------------
    def _autocast(self):
        if self.autocast_dtype is None:
            return contextlib.nullcontext()
        return torch.autocast(device_type=self.device.type, dtype=self.autocast_dtype)

    def _one_step(self) -> Tensor:
        k = self.accumulation_steps
        if k == 1:
            with trace.span("forward"), self._autocast():
                loss = self.loss_fn(*self.static_inputs)
            with trace.span("backward"):
                loss.backward()
        else:
            # Micro-batches accumulate into the same gradients; only the last backward hands
            # them to the bucketed all-reduce.
            total = None
            for i in range(k):
                self.sync.active = i == k - 1
                with trace.span("forward"), self._autocast():
                    part = self.loss_fn(*[t[i] for t in self.static_inputs]) / k
                with trace.span("backward"):
                    part.backward()
                total = part.detach() if total is None else total + part.detach()
            self.sync.active = True
            loss = total
        with trace.span("grad_sync"):
            deferred = self.sync.finish(self._deferrable)
        if deferred:
            self.optimizer.before_scalar_tasks = self.sync.join
        try:
            with trace.span("optimizer"):
                self.optimizer.step()
        finally:
            if deferred:
                self.optimizer.before_scalar_tasks = None
                self.sync.join()  # a no-op when the hook already ran; keeps capture joined
        # Gradients are dropped, not zeroed: under capture the next backward re-creates them in
        # the graph's private pool at the same addresses.
        for p in self.params:
            p.grad = None
        return loss.detach()

    def _load_inputs(self, inputs: Sequence[Tensor]) -> None:
        assert len(inputs) == len(self.static_inputs)
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)

    def _pre_replay(self) -> None:
        for name in ("_sync_hyperparam_tensors", "_poll_device_status"):
            fn = getattr(self.optimizer, name, None)
            if fn is not None:
                fn()

    def _post_replay(self) -> None:
        for name in ("_snapshot_device_status", "_advance_host_step_counters"):
            fn = getattr(self.optimizer, name, None)
            if fn is not None:
                fn()

    def __call__(self, *inputs: Tensor) -> Tensor:
        self._load_inputs(inputs)
        self._calls += 1
        if not self.use_graph:
            self.static_loss = self._one_step()
            return self.static_loss
        if self.graph is not None:
            self._pre_replay()
            self.graph.replay()
            self._post_replay()
            return self.static_loss
        cur = torch.cuda.current_stream(self.device)
        if self._calls <= self.warmup:
            # Eager warm-up on a side stream (allocates optimizer state, workspaces, caches).
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                loss = self._one_step()
            cur.wait_stream(self._side)
            self.static_loss = loss
            return loss
        self._pre_replay()
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loss = self._one_step()
        self.graph, self.static_loss = graph, loss
        # Capturing ran the host side of the step once (counters included) without executing
        # anything on the device; this replay is that step's device work.
        graph.replay()
        return self.static_loss

    def release(self) -> None:
        """Drop the graph (before ``destroy_process_group()`` when it holds collectives)."""
        graph, self.graph = self.graph, None
        if graph is not None:
            torch.cuda.synchronize(self.device)
            graph.reset()
        self.sync.remove()
