"""Device-side tensor tables for the multi-tensor kernels.

A table is one int64 device tensor ``[n, chunk_prefix[n+1], numel[n], ptr_0[n], ptr_1[n], ...]``.
Tables are cached by the data pointers they describe, so a steady-state optimizer step (same
parameter, gradient and state buffers every iteration) performs no host-to-device copy; when a
gradient buffer moves (``zero_grad(set_to_none=True)``) the table is rebuilt.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

CHUNK = 4096  # must match kChunk in csrc/foreach_ops.cu

_cache: Dict[Tuple, "TensorTable"] = {}
_CACHE_LIMIT = 4096
# Tables that a CUDA graph recorded: replays read their device memory, so they must outlive the
# cache (which is dropped wholesale when it grows past its limit).
_recorded: Dict[Tuple, "TensorTable"] = {}


def _remember_if_capturing(key: Tuple, tb: "TensorTable") -> None:
    if tb.device_tensor.is_cuda and torch.cuda.is_current_stream_capturing():
        _recorded.setdefault(key, tb)

# Pinned staging memory for the host->device copies of tables.  Eager rebuilds take slices of a
# ring; rebuilds that happen while a CUDA graph is being captured take slices that are never
# reused, because every replay of the graph re-reads them.
_RING_WORDS = 1 << 18
_PERSIST_WORDS = 1 << 19
_ring: Optional[Tensor] = None
_ring_pos = 0
_persist: Optional[Tensor] = None
_persist_pos = 0


def _ensure_staging() -> None:
    global _ring, _persist
    if _ring is None:
        _ring = torch.empty(_RING_WORDS, dtype=torch.int64).pin_memory()
        _persist = torch.empty(_PERSIST_WORDS, dtype=torch.int64).pin_memory()


def _upload(host: Tensor, device: torch.device) -> Tensor:
    """Copy a small int64 host tensor to ``device`` through pinned staging memory."""
    global _ring_pos, _persist_pos
    n = host.numel()
    capturing = torch.cuda.is_current_stream_capturing()
    if _ring is None:
        if capturing:
            raise RuntimeError(
                "pointer table needed during CUDA graph capture before any eager step ran")
        _ensure_staging()
    flat = host.reshape(-1)
    if capturing:
        if _persist_pos + n > _PERSIST_WORDS:
            raise RuntimeError("pinned staging for graph-captured pointer tables is exhausted")
        stage = _persist[_persist_pos:_persist_pos + n]
        _persist_pos += n
    else:
        if n > _RING_WORDS:
            return host.pin_memory().to(device, non_blocking=True)
        if _ring_pos + n > _RING_WORDS:
            # About to overwrite staging words whose copies were queued long ago; make sure the
            # stream has drained them (once per ~2 MB of tables, so the wait is rare and short).
            torch.cuda.current_stream(device).synchronize()
            _ring_pos = 0
        stage = _ring[_ring_pos:_ring_pos + n]
        _ring_pos += n
    stage.copy_(flat)
    return stage.to(device, non_blocking=True).view(host.shape)


class TensorTable:
    __slots__ = ("device_tensor", "n", "n_chunks", "keepalive")

    def __init__(self, device_tensor: Tensor, n: int, n_chunks: int, keepalive):
        self.device_tensor = device_tensor
        self.n = n
        self.n_chunks = n_chunks
        self.keepalive = keepalive


class RawPointer:
    """A bare device address standing in for a tensor in a pointer table (e.g. a location in
    another GPU's peer-mapped buffer)."""

    __slots__ = ("address",)

    def __init__(self, address: int):
        self.address = int(address)

    def data_ptr(self) -> int:
        return self.address


def _ptr(t) -> int:
    if t is None:
        return 0
    ptr = t.data_ptr()
    if ptr == 0 and not isinstance(t, RawPointer) and t.numel():
        raise RuntimeError(f"{type(t).__name__} has no device storage to hand to a kernel")
    return ptr


def build_table(
    lists: Sequence[Sequence[Optional[Tensor]]],
    numels: Optional[Sequence[int]] = None,
    chunk: int = CHUNK,
    tag: str = "",
) -> TensorTable:
    """``lists[j][i]`` is pointer ``j`` of tensor ``i``.  ``numels`` defaults to ``lists[0]``."""
    n = len(lists[0])
    if numels is None:
        numels = [t.numel() for t in lists[0]]
    key = (tag, chunk, tuple(numels)) + tuple(tuple(_ptr(t) for t in lst) for lst in lists)
    hit = _cache.get(key)
    if hit is not None:
        _remember_if_capturing(key, hit)
        return hit
    device = next(t.device for lst in lists for t in lst if isinstance(t, Tensor))
    prefix = [0]
    for ne in numels:
        prefix.append(prefix[-1] + (ne + chunk - 1) // chunk)
    flat: List[int] = [n] + prefix + list(numels)
    for lst in lists:
        assert len(lst) == n
        flat.extend(_ptr(t) for t in lst)
    host = torch.tensor(flat, dtype=torch.int64)
    dev = _upload(host, device) if device.type == "cuda" else host
    if len(_cache) > _CACHE_LIMIT:
        _cache.clear()
    # The key holds every address in the table, so a buffer that moved misses the cache and a
    # fresh table is built; nothing is kept alive here (that would pin freed gradients).
    tb = TensorTable(dev, n, prefix[-1], None)
    _cache[key] = tb
    _remember_if_capturing(key, tb)
    return tb


def build_ptr_array(lists: Sequence[Sequence[Optional[Tensor]]], tag: str = "") -> Tensor:
    """Plain ``[len(lists)][n]`` int64 device array of data pointers (cached)."""
    key = ("ptrs", tag) + tuple(tuple(_ptr(t) for t in lst) for lst in lists)
    hit = _cache.get(key)
    if hit is not None:
        _remember_if_capturing(key, hit)
        return hit.device_tensor
    device = next((t.device for lst in lists for t in lst if isinstance(t, Tensor)), None)
    if device is None:  # only raw addresses: they belong to the current CUDA device
        device = torch.device("cuda", torch.cuda.current_device())
    host = torch.tensor([[_ptr(t) for t in lst] for lst in lists], dtype=torch.int64)
    dev = _upload(host, device) if device.type == "cuda" else host
    if len(_cache) > _CACHE_LIMIT:
        _cache.clear()
    tb = _cache[key] = TensorTable(dev, len(lists[0]), 0, None)
    _remember_if_capturing(key, tb)
    return dev


def clear_cache() -> None:
    """Drop cached tables (those recorded by CUDA graphs stay alive)."""
    _cache.clear()
