"""FSDP2 parameter all-gather carried by a kernel of this package over symmetric memory.

``torch.distributed.fsdp`` lets a module replace its all-gather (``set_custom_all_gather``).
:class:`SymmetricAllGather` allocates the all-gather output in symmetric memory and, instead of
an NCCL collective, launches one kernel in which every rank pushes its shard into all ranks'
output buffers - with NVLS one ``multimem.st`` per 16 bytes that the NVSwitch replicates, so a
GPU sends each byte once; otherwise plain stores to every peer - bracketed by the bounded flag
barriers of :class:`dion_b200.parallel.symm.SymmetricAllReduce`.  FSDP's copy-in already places
the local shard at its slot of the output, so the gather is in place and copy-free.

The output buffers form a small ring (FSDP keeps the current and the prefetched all-gather
alive); a buffer is handed out again only when nothing references it any more, and all ranks
walk the ring in the same order.  Requests that do not fit (size, 16-byte slot granularity) fall
back to NCCL.  This is the all-gather half of the reference's reliance on FSDP2's NCCL
collectives (models/gpt_model.py:338-398); fusing it into the first GEMM that consumes the
gathered weight is not done.

    comm = use_symmetric_all_gather(model, fsdp_group, device)     # after fully_shard(...)
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from . import symm

try:  # the extension point exists from torch 2.8 on
    from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather as _AllGatherBase
except Exception:  # pragma: no cover
    _AllGatherBase = object


def _storage_users(t: Tensor) -> int:
    return torch._C._storage_Use_Count(t.untyped_storage()._cdata)


class SymmetricAllGather(_AllGatherBase):
    def __init__(self, group: dist.ProcessGroup, device: torch.device, max_bytes: int,
                 num_buffers: int = 4):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_bytes = max_bytes
        self.rings: List[symm.SymmetricAllReduce] = [
            symm.SymmetricAllReduce(group, max_bytes, device) for _ in range(num_buffers)]
        self._by_ptr: Dict[int, symm.SymmetricAllReduce] = {
            r.view((1,), torch.uint8).data_ptr(): r for r in self.rings}
        # References that exist while a buffer is idle (the workspace's own tensors and views).
        self._idle_users = [_storage_users(r.buf.local) for r in self.rings]
        self._next = 0
        self.calls = 0           # all-gathers done by the kernel
        self.fallbacks = 0       # all-gathers handed to NCCL

    # -- Comm interface ----------------------------------------------------------------------
    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> Tensor:
        n = 1
        for s in size:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.max_bytes or nbytes == 0:
            return torch.empty(tuple(size), dtype=dtype, device=device)
        k = self._next % len(self.rings)
        self._next += 1
        ring = self.rings[k]
        if _storage_users(ring.buf.local) > self._idle_users[k]:
            raise RuntimeError(
                "SymmetricAllGather: the next output buffer of the ring is still referenced; "
                "raise num_buffers (more all-gathers are in flight than buffers exist)")
        return ring.view(tuple(size), dtype)

    def __call__(self, output_tensor: Tensor, input_tensor: Tensor, group: dist.ProcessGroup,
                 async_op: bool = False):
        ring = self._by_ptr.get(output_tensor.data_ptr())
        slot = input_tensor.numel() * input_tensor.element_size()
        in_place = input_tensor.data_ptr() == output_tensor.data_ptr() + self.rank * slot
        if ring is None or slot % 16 or slot == 0:
            self.fallbacks += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group,
                                               async_op=async_op)
        if not in_place:
            flat = output_tensor.view(-1).view(torch.uint8)
            flat[self.rank * slot:(self.rank + 1) * slot].copy_(
                input_tensor.reshape(-1).view(torch.uint8))
        ring.all_gather_(slot)
        self.calls += 1
        return None  # the work is ordered on the current (all-gather) stream


def use_symmetric_all_gather(model: torch.nn.Module, group: dist.ProcessGroup,
                             device: torch.device, max_bytes: Optional[int] = None,
                             num_buffers: int = 4) -> Optional[SymmetricAllGather]:
    """Install one shared :class:`SymmetricAllGather` on every FSDP2 module of ``model``.
    ``max_bytes`` defaults to the largest unsharded parameter group (in the all-gather dtype
    FSDP reports, at most 4 bytes per element).  Returns None when symmetric memory is not
    available for ``group``."""
    from torch.distributed.fsdp import FSDPModule

    if not symm.symmetric_memory_available(group):
        return None
    modules = [m for m in model.modules() if isinstance(m, FSDPModule)]
    if not modules:
        return None
    if max_bytes is None:
        # Every parameter belongs to the innermost FSDP module that contains it; a module's
        # all-gather moves its whole group (FSDP pads each shard, hence the slack).  Larger
        # requests than estimated here simply fall back to NCCL.
        owner: Dict[int, int] = {}
        for mi, m in enumerate(model.modules()):       # pre-order: inner modules come later
            if isinstance(m, FSDPModule):
                for p in m.parameters():
                    owner[id(p)] = mi
        sizes: Dict[int, int] = {}
        for p in model.parameters():
            mi = owner.get(id(p))
            if mi is not None:
                sizes[mi] = sizes.get(mi, 0) + p.numel()
        largest = max(sizes.values()) if sizes else 0
        max_bytes = int(4 * largest * 1.05) + (1 << 20)
    comm = SymmetricAllGather(group, device, int(max_bytes), num_buffers)
    for m in modules:
        m.set_custom_all_gather(comm)
    return comm
