"""Reduce-scatter carried by a GEMM epilogue, followed by an all-gather, over peer-mapped memory.

Legacy Dion synchronizes its low-rank factors instead of the gradients: ``P = M Q`` is summed (or
averaged) over the ranks with each rank keeping the matrices it will orthogonalize, the
orthonormal ``P`` is gathered again, and ``R = M^T P`` is averaged over the data-parallel ranks
(reference: dion/dion.py:797-843, 917-956, all-reduce helper :1162-1194 - NCCL reduce-scatter,
all-gather and all-reduce around cuBLAS products).

Here the factors live in one symmetric buffer ``[W*L, rows, cols]`` (fp32) per rank, laid out as
the gathered result.  Rank ``q`` owns the slots ``[q*L, (q+1)*L)``.

1. ``begin()``: wait until every owner has cleared its slots after the previous round.
2. The GEMM that produces the factor runs with ``reduce_into=targets``: its epilogue adds each
   output tile with ``red.global.add`` straight into the owner's slot over NVLink (the local
   slots included), so when all ranks have run it every owner holds the sum of its matrices -
   the product never exists as a separate tensor and no collective is called.
3. ``after_gemm()``: publish "my contributions are stored" and wait for everybody's.
4. The owner may now work on ``own()`` in place (orthogonalize ``P``).
5. ``gather()``: one kernel pushes the owner's slots into every peer's buffer (``multimem.st``
   through the NVSwitch, or plain peer stores) between two flag barriers; afterwards every rank
   reads the full stack from its own memory.
6. ``release()``: the stack has been consumed; clear the own slots and tell the peers.

All waits are bounded and report through the device status word (``ops.gemm.check_status``).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from ..ops import gemm
from . import symm


def fused_lowrank_enabled() -> bool:
    """``DION_B200_FUSED_LOWRANK=1`` turns this path on.  It is off by default: measured on the
    GPT-1B block matrices it ties with the NCCL reduce-scatter / all-gather at 2 GPUs (29.3
    against 29.0 ms per step) and loses at 4 (30.0 against 26.8 ms) - the factors are large
    (0.8 GB per step) against the 0.2 ms product that produces them, so there is little to
    overlap, and 16-byte reductions use an NVLink far less well than NCCL's bulk copies."""
    return os.environ.get("DION_B200_FUSED_LOWRANK", "0") == "1"


def eligible(pg: Optional[ProcessGroup], device: torch.device) -> bool:
    """Rank-independent decision (the capability check behind it is collective and cached)."""
    if not fused_lowrank_enabled() or pg is None or device.type != "cuda":
        return False
    world = dist.get_world_size(pg)
    if world < 2 or world > 8:
        return False
    return symm.symmetric_memory_available(pg)


class FusedReduceGather:
    """Workspace for one stack of ``world * per_rank`` matrices ``[rows, cols]`` in fp32."""

    def __init__(self, pg: ProcessGroup, per_rank: int, rows: int, cols: int,
                 device: torch.device):
        self.pg, self.device = pg, device
        self.rank, self.world = dist.get_rank(pg), dist.get_world_size(pg)
        self.L, self.rows, self.cols = per_rank, rows, cols
        self.slot_bytes = per_rank * rows * cols * 4
        if self.slot_bytes % 16:
            raise ValueError("per-rank slice of the stack must be a multiple of 16 bytes")
        self.red = symm.SymmetricAllReduce(pg, self.slot_bytes * self.world, device)
        lay = symm.Layout()
        self.off_zero = lay.add("zero", self.world * 4)
        self.off_added = lay.add("added", self.world * 4)
        self.fbuf = symm.SymmetricBuffer(lay.size, pg)
        self.flags_zero = self.fbuf.view(self.off_zero, (self.world,), torch.int32)
        self.flags_added = self.fbuf.view(self.off_added, (self.world,), torch.int32)
        self.peer_zero = symm.address_table(
            [self.fbuf.peer_address(p, self.off_zero) for p in range(self.world)], device)
        self.peer_added = symm.address_table(
            [self.fbuf.peer_address(p, self.off_added) for p in range(self.world)], device)
        self.seq = torch.zeros((), dtype=torch.int32, device=device)
        self.status = gemm.status_tensor(device)
        n = self.world * per_rank
        base = [self.red.buf.peer_address(b // per_rank, self.red.off_data + b * rows * cols * 4)
                for b in range(n)]
        # where matrix b is accumulated: its own slot in the buffer of the rank that owns it
        self.targets = symm.address_table(base, device)
        self.stack = self.red.view((n, rows, cols), torch.float32)
        self.seq_open = False   # host-side: a round has begun and not been released yet

    def begin(self) -> None:
        self.seq_open = True
        symm.bump_seq(self.seq)
        # flag value s-1 = "cleared after round s-1" (0 at start: freshly zeroed memory)
        symm.wait_flags(self.flags_zero, self.seq, -1, self.status)

    def after_gemm(self) -> None:
        symm.signal_peers(self.peer_added, self.rank, self.seq)
        symm.wait_flags(self.flags_added, self.seq, 0, self.status)

    def own(self) -> Tensor:
        return self.stack[self.rank * self.L:(self.rank + 1) * self.L]

    def gather(self) -> Tensor:
        self.red.all_gather_(self.slot_bytes)
        return self.stack

    def release(self) -> None:
        self.seq_open = False
        self.own().zero_()
        symm.signal_peers(self.peer_zero, self.rank, self.seq)
