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
from ..ops.tables import build_ptr_array


def symmetric_memory_available(pg: Optional[ProcessGroup]) -> bool:
    if pg is None or not torch.cuda.is_available():
        return False
    try:
        if dist.get_backend(pg) != "nccl":
            return False
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except Exception:
        return False
    return True


class SymmetricBuffer:
    """``nbytes`` of zero-initialised symmetric memory on the current CUDA device."""

    def __init__(self, nbytes: int, pg: ProcessGroup):
        import torch.distributed._symmetric_memory as symm_mem

        self.pg = pg
        self.rank = dist.get_rank(pg)
        self.world = dist.get_world_size(pg)
        nbytes = (nbytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        try:
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
