"""Symmetric (peer-mapped) device memory over NVLink.

A ``SymmetricBuffer`` is one allocation of the same size on every rank of a process group, with
every rank holding the device addresses of all peers' copies.  Kernels of this package store to
and poll those addresses directly; nothing here moves data.  Built on
``torch.distributed._symmetric_memory`` (CUDA virtual memory + handle exchange through the
process group's store), which is available for NCCL groups on one node.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from ..ops import _backend


_capability: Dict[int, bool] = {}


def symmetric_memory_available(pg: Optional[ProcessGroup]) -> bool:
    """Whether kernels may address the memory of every rank of ``pg`` directly: an NCCL group
    whose ranks all sit on one host, each on a GPU of its own that every other rank's GPU can
    reach by peer access.  Decided once per group by a collective exchange (host name and device
    index of every rank) and a MIN-reduction of each rank's verdict, then cached, so that all
    ranks take the same path; the first call for a group is therefore collective."""
    if pg is None or not torch.cuda.is_available():
        return False
    try:
        if dist.get_backend(pg) != "nccl":
            return False
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except Exception:
        return False
    key = id(pg)
    known = _capability.get(key)
    if known is not None:
        return known
    import socket

    world = dist.get_world_size(pg)
    me = (socket.gethostname(), torch.cuda.current_device())
    everyone: List = [None] * world
    dist.all_gather_object(everyone, me, group=pg)
    ok = len({h for h, _ in everyone}) == 1 and len({d for _, d in everyone}) == world
    if ok:
        for _, d in everyone:
            if d != me[1]:
                try:
                    ok = ok and torch.cuda.can_device_access_peer(me[1], d)
                except Exception:
                    ok = False
    verdict = torch.tensor([1 if ok else 0], dtype=torch.int32,
                           device=torch.device("cuda", me[1]))
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=pg)
    known = _capability[key] = bool(verdict.item())
    return known


class SymmetricBuffer:
    """``nbytes`` of zero-initialised symmetric memory on the current CUDA device."""

    def __init__(self, nbytes: int, pg: ProcessGroup):
        import torch.distributed._symmetric_memory as symm_mem

        self.pg = pg
        self.rank = dist.get_rank(pg)
        self.world = dist.get_world_size(pg)
        nbytes = (nbytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        import warnings

        try:   # needed by older releases, a deprecated no-op in newer ones
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                symm_mem.enable_symm_mem_for_group(pg.group_name)
        except Exception:
            pass
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        try:
            self.handle = symm_mem.rendezvous(self.local, group=pg)
        except TypeError:
            self.handle = symm_mem.rendezvous(self.local, pg.group_name)
        self.local.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=pg)
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        assert self.peer_ptrs[self.rank] == self.local.data_ptr()

    def view(self, offset: int, shape, dtype: torch.dtype) -> Tensor:
        """Local tensor view of ``shape``/``dtype`` starting ``offset`` bytes into the buffer."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(tuple(shape))

    def peer_address(self, peer: int, offset: int) -> int:
        return self.peer_ptrs[peer] + offset


class Layout:
    """Bump allocator for sections of a symmetric buffer (256-byte aligned)."""

    def __init__(self) -> None:
        self.size = 0
        self.sections: Dict[str, Tuple[int, int]] = {}

    def add(self, name: str, nbytes: int) -> int:
        off = (self.size + 255) // 256 * 256
        self.sections[name] = (off, nbytes)
        self.size = off + nbytes
        return off


def _c(p: int):
    return ctypes.c_void_p(p)


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def bump_seq(seq: Tensor) -> None:
    rc = _backend.lib("comm_ops").dion_bump_seq(_c(seq.data_ptr()), _stream(seq.device))
    if rc != 0:
        raise RuntimeError("dion_bump_seq failed")


def signal_peers(peer_flag_addresses: Tensor, slot: int, seq: Tensor) -> None:
    """Set ``flag[slot] = *seq`` in every peer's flag array (``peer_flag_addresses``: int64 device
    tensor with one base address per peer).  Stores issued by earlier kernels on the stream are
    visible to a peer that observes the flag."""
    rc = _backend.lib("comm_ops").dion_signal_peers(
        _c(peer_flag_addresses.data_ptr()), peer_flag_addresses.numel(), slot,
        _c(seq.data_ptr()), _stream(seq.device))
    if rc != 0:
        raise RuntimeError("dion_signal_peers failed")


def wait_flags(flags: Tensor, seq: Tensor, delta: int, status: Tensor) -> None:
    """Block the stream (bounded) until every ``flags[i] >= *seq + delta``."""
    rc = _backend.lib("comm_ops").dion_wait_flags(
        _c(flags.data_ptr()), flags.numel(), _c(seq.data_ptr()), delta, _c(status.data_ptr()),
        _stream(seq.device))
    if rc != 0:
        raise RuntimeError("dion_wait_flags failed")


def scale_from_partials(partials: Tensor, n_mats: int, n_src: int, mult: float, eps: float,
                        scale: Tensor, clear: bool) -> None:
    rc = _backend.lib("comm_ops").dion_scale_from_partials(
        _c(partials.data_ptr()), n_mats, n_src, ctypes.c_float(mult), ctypes.c_float(eps),
        _c(scale.data_ptr()), int(clear), _stream(partials.device))
    if rc != 0:
        raise RuntimeError("dion_scale_from_partials failed")


def address_table(addresses: List[int], device: torch.device) -> Tensor:
    """int64 device tensor holding raw addresses."""
    return torch.tensor(addresses, dtype=torch.int64).to(device)


# ------------------------------------------------------------------------------------------------
# All-reduce inside symmetric memory (NVLS multimem through the NVSwitch, or plain peer access)
# ------------------------------------------------------------------------------------------------
def nvls_enabled(world: int = 8) -> bool:
    """``DION_B200_NVLS``: "1" multimem, "0" plain peer access; unset: multimem for more than two
    ranks (between two GPUs the switch has nothing to combine and plain peer access measured
    faster: 638 against 390 GB/s bus bandwidth at 256 MiB)."""
    import os
    v = os.environ.get("DION_B200_NVLS")
    if v is None:
        return world > 2
    return v != "0"


class SymmetricAllReduce:
    """In-place all-reduce of up to ``capacity`` bytes that live in a symmetric buffer.

    Two-shot, one kernel launch per call: after a flag barrier every rank reduces its 1/W slice
    over all ranks and writes the result into every rank's copy; a second flag barrier (by the
    block that finishes last) publishes the result.  With NVLS the
    slice is read with ``multimem.ld_reduce`` (the switch adds the ranks' copies) and written
    with ``multimem.st`` (the switch replicates it); with ``DION_B200_NVLS=0`` or without
    multicast support the kernel loads from and stores to the peers' copies one by one.  This is
    the communication step of Dion's compressed data-parallel sync (all-reduce of the small
    ``P``/``R`` factors; dion/dion.py:1162-1194 of the reference uses NCCL) and of
    ``synchronize_for_checkpoint``.  All waits are bounded; a missing peer surfaces through
    ``dion_b200.ops.gemm.check_status``.

    ``view(shape, dtype)`` exposes the start of the buffer, so a producer (e.g. ``torch.bmm(...,
    out=view)``) can write its result in place and no copy is needed; ``all_reduce_tensor_``
    copies an ordinary tensor in and out."""

    def __init__(self, pg: ProcessGroup, capacity: int, device: torch.device):
        from ..ops import gemm

        self.pg, self.device = pg, device
        self.rank, self.world = dist.get_rank(pg), dist.get_world_size(pg)
        lay = Layout()
        self.capacity = (capacity + 4095) // 4096 * 4096
        self.off_data = lay.add("data", self.capacity)
        self.off_in = lay.add("in", self.world * 4)
        self.off_out = lay.add("out", self.world * 4)
        self.buf = SymmetricBuffer(lay.size, pg)
        self.flags_in = self.buf.view(self.off_in, (self.world,), torch.int32)
        self.flags_out = self.buf.view(self.off_out, (self.world,), torch.int32)
        self.in_table = address_table(
            [self.buf.peer_address(p, self.off_in) for p in range(self.world)], device)
        self.out_table = address_table(
            [self.buf.peer_address(p, self.off_out) for p in range(self.world)], device)
        self.data_table = address_table(
            [self.buf.peer_address(p, self.off_data) for p in range(self.world)], device)
        self.seq = torch.zeros((), dtype=torch.int32, device=device)
        self.counter = torch.zeros((), dtype=torch.int32, device=device)
        self.status = gemm.status_tensor(device)
        mc = 0
        if nvls_enabled(self.world):
            try:
                mc = int(getattr(self.buf.handle, "multicast_ptr", 0) or 0)
            except Exception:
                mc = 0
        self.multicast_base = mc + self.off_data if mc else 0
        self.num_blocks = 4 * torch.cuda.get_device_properties(device).multi_processor_count

    @property
    def uses_multimem(self) -> bool:
        return self.multicast_base != 0

    def view(self, shape, dtype: torch.dtype) -> Tensor:
        return self.buf.view(self.off_data, shape, dtype)

    def all_reduce_(self, numel: int, dtype: torch.dtype, op: str = "sum") -> None:
        """Reduce the first ``numel`` elements of ``dtype`` in place on every rank."""
        esize = 4 if dtype == torch.float32 else 2
        if dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("SymmetricAllReduce handles fp32 and bf16")
        nbytes = numel * esize
        if nbytes > self.capacity:
            raise ValueError("tensor exceeds the symmetric all-reduce buffer")
        nvec = (nbytes + 15) // 16
        per = (nvec + self.world - 1) // self.world
        begin, end = self.rank * per, min(nvec, (self.rank + 1) * per)
        scale = 1.0 / self.world if op == "avg" else 1.0
        self._launch(begin, end, 0 if dtype == torch.float32 else 1, scale, gather=False)

    def all_gather_(self, slot_bytes: int) -> None:
        """All-gather in place: every rank's ``slot_bytes`` (a multiple of 16) already lie at
        byte offset ``rank * slot_bytes`` of its own copy; afterwards every copy holds all
        slots."""
        if slot_bytes % 16 or slot_bytes * self.world > self.capacity:
            raise ValueError("slot size must be a multiple of 16 bytes and fit the buffer")
        per = slot_bytes // 16
        self._launch(self.rank * per, (self.rank + 1) * per, 0, 1.0, gather=True)

    def _launch(self, begin: int, end: int, dt: int, scale: float, gather: bool) -> None:
        rc = _backend.lib("comm_ops").dion_allreduce_fused(
            _c(self.multicast_base), _c(self.data_table.data_ptr()),
            _c(self.in_table.data_ptr()), _c(self.out_table.data_ptr()),
            _c(self.flags_in.data_ptr()), _c(self.flags_out.data_ptr()),
            _c(self.seq.data_ptr()), _c(self.counter.data_ptr()), _c(self.status.data_ptr()),
            self.world, self.rank, ctypes.c_longlong(begin), ctypes.c_longlong(end),
            dt, ctypes.c_float(scale), 1 if gather else 0, self.num_blocks,
            _stream(self.device))
        if rc != 0:
            raise RuntimeError(f"dion_allreduce_fused failed (code {rc})")

    def all_reduce_tensor_(self, t: Tensor, op: str = "sum") -> Tensor:
        flat = self.view((t.numel(),), t.dtype)
        flat.copy_(t.reshape(-1))
        self.all_reduce_(t.numel(), t.dtype, op)
        t.copy_(flat.view(t.shape))
        return t


_all_reducers: Dict[Tuple[int, int], SymmetricAllReduce] = {}


def symmetric_all_reduce_(t: Tensor, pg: ProcessGroup, op: str = "sum") -> Tensor:
    """All-reduce ``t`` in place through a cached :class:`SymmetricAllReduce` of ``pg`` (created
    collectively on first use, regrown when a larger tensor comes; every rank must call this with
    the same sizes in the same order)."""
    key = (id(pg), t.device.index or 0)
    red = _all_reducers.get(key)
    need = t.numel() * t.element_size()
    if red is None or need > red.capacity:
        red = _all_reducers[key] = SymmetricAllReduce(pg, max(need, 1 << 22), t.device)
    return red.all_reduce_tensor_(t, op)
