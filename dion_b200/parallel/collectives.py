"""Thin collective helpers on plain tensors that behave the same on NCCL and gloo.

gloo has no ``avg`` reduction and no reduce-scatter; both are expressed through ``all_reduce``
there, which keeps the CPU multi-process tests on the same code path as the GPU runs.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh

Group = Union[ProcessGroup, DeviceMesh, None]


def as_groups(g: Group) -> List[ProcessGroup]:
    """Process groups behind ``g``: a DeviceMesh contributes one group per mesh dimension."""
    if g is None:
        return []
    if isinstance(g, DeviceMesh):
        return [g.get_group(i) for i in range(g.ndim)]
    return [g]


def group_size(g: Group) -> int:
    if g is None:
        return 1
    if isinstance(g, DeviceMesh):
        return g.size()
    return dist.get_world_size(g)


def group_rank(g: Group) -> int:
    if g is None:
        return 0
    if isinstance(g, DeviceMesh):
        assert g.ndim == 1
        return g.get_local_rank()
    return dist.get_rank(g)


def _is_gloo(pg: ProcessGroup) -> bool:
    return dist.get_backend(pg) == "gloo"


class _Done:
    def wait(self):
        return None


class _Chain:
    """Completes several works and then runs an epilogue (e.g. the division of an average)."""

    def __init__(self, works, epilogue=None):
        self.works, self.epilogue = works, epilogue

    def wait(self):
        for w in self.works:
            w.wait()
        if self.epilogue is not None:
            self.epilogue()
            self.epilogue = None


def _symmetric_route(ts: Sequence[Tensor], pg: ProcessGroup) -> bool:
    """``DION_B200_SYMM_ALLREDUCE=1`` sends CUDA fp32/bf16 all-reduces of a single NCCL group
    through the NVLS / peer-memory kernel of :mod:`dion_b200.parallel.symm` instead of NCCL."""
    import os

    if os.environ.get("DION_B200_SYMM_ALLREDUCE", "0") != "1" or _is_gloo(pg):
        return False
    if dist.get_world_size(pg) > 8:
        return False
    return all(t.is_cuda and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16)
               for t in ts)


def all_reduce_(tensors: Union[Tensor, Sequence[Tensor]], group: Group, op: str = "sum",
                async_op: bool = False):
    """In-place all-reduce (``sum`` or ``avg``) of one tensor or a list over every group of
    ``group``.  Returns an object with ``wait()`` when ``async_op``."""
    ts = [tensors] if isinstance(tensors, Tensor) else list(tensors)
    ts = [t for t in ts if t.numel()]
    pgs = as_groups(group)
    if not ts or not pgs:
        return _Done() if async_op else None
    works = []
    scale = 1.0
    live = [pg for pg in pgs if dist.get_world_size(pg) > 1]
    if len(live) == 1 and _symmetric_route(ts, live[0]):
        from . import symm

        for t in ts:
            symm.symmetric_all_reduce_(t, live[0], op)
        return _Done() if async_op else None
    for i, pg in enumerate(live):
        n = dist.get_world_size(pg)
        use_avg = op == "avg" and not _is_gloo(pg)
        if op == "avg" and not use_avg:
            scale /= n
        red = dist.ReduceOp.AVG if use_avg else dist.ReduceOp.SUM
        works = [dist.all_reduce(t, op=red, group=pg, async_op=True) for t in ts]
        if i + 1 < len(live):
            # reductions over successive mesh dimensions must not overlap on the same buffer
            for w in works:
                w.wait()
            works = []

    def epilogue():
        if scale != 1.0:
            for t in ts:
                t.mul_(scale)

    chain = _Chain(works, epilogue)
    if async_op:
        return chain
    chain.wait()
    return None


def reduce_scatter_dim0(x: Tensor, pg: Optional[ProcessGroup], op: str = "sum",
                        async_op: bool = False):
    """``x`` is ``[W*c, ...]`` on every rank; returns ``(out [c, ...], work)`` holding this
    rank's reduced slice."""
    if pg is None or dist.get_world_size(pg) == 1:
        return x, _Done()
    W, rank = dist.get_world_size(pg), dist.get_rank(pg)
    c = x.size(0) // W
    x = x.contiguous()
    if _is_gloo(pg):
        w = dist.all_reduce(x, op=dist.ReduceOp.SUM, group=pg, async_op=True)
        out = x[rank * c:(rank + 1) * c]

        def epi():
            if op == "avg":
                out.div_(W)
        work = _Chain([w], epi)
    else:
        out = torch.empty((c,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        red = dist.ReduceOp.AVG if op == "avg" else dist.ReduceOp.SUM
        work = _Chain([dist.reduce_scatter_tensor(out, x, op=red, group=pg, async_op=True)])
    if not async_op:
        work.wait()
    return out, work


def all_gather_dim0(x: Tensor, pg: Optional[ProcessGroup], async_op: bool = False):
    """Concatenate every rank's ``x`` along dim 0: ``(out [W*c, ...], work)``."""
    if pg is None or dist.get_world_size(pg) == 1:
        return x, _Done()
    W = dist.get_world_size(pg)
    x = x.contiguous()
    out = torch.empty((W * x.size(0),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    work = _Chain([dist.all_gather_into_tensor(out, x, group=pg, async_op=True)])
    if not async_op:
        work.wait()
    return out, work


def all_gather_last_dim(x: Tensor, pg: Optional[ProcessGroup]) -> Tensor:
    """Concatenate every rank's ``x`` along the last dim (synchronous)."""
    if pg is None or dist.get_world_size(pg) == 1:
        return x
    W = dist.get_world_size(pg)
    out, _ = all_gather_dim0(x.unsqueeze(0), pg)
    return out.movedim(0, -2).reshape(tuple(x.shape[:-1]) + (W * x.size(-1),))


def broadcast_(t: Tensor, group: Group, src: int = 0) -> None:
    for pg in as_groups(group):
        if dist.get_world_size(pg) > 1:
            dist.broadcast(t, group=pg, group_src=src)
