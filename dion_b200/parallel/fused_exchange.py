"""Megabatch exchange of row-sharded matrices fused into the Newton-Schulz kernels.

The NCCL path of :class:`MegabatchPlan` packs shards, runs an all-to-all, concatenates, runs
Newton-Schulz, splits, runs a second all-to-all and unpacks.  Here the data movement is done by
the compute kernels themselves over peer-mapped memory (NVLink / NVSwitch):

1. the momentum kernel stores its bf16 output directly into the receive buffers of the ranks
   that own the matrices, at the row offset of this rank's shard, so the owner finds whole
   matrices with nothing to concatenate, and adds its shard's sum of squares to the owner's
   per-source partial sums (the Frobenius norm travels with the data);
2. the first Gram GEMM of the Newton-Schulz iteration starts immediately; its TMA producer polls
   the arrival flag of the ranks that own the rows (or K-slabs) a tile needs, so tiles are
   computed as their inputs land; the epilogue assembles the normalization from the partial sums;
3. the last update GEMM stores every output row straight into the return buffer of the rank that
   holds that row's shard;
4. the weight-update kernel waits for the flag of the producing rank and reads the update in
   place.

Flags carry a per-workspace sequence number kept in device memory, buffers are handed back with
explicit acknowledgement flags (a rank never overwrites data its peer has not consumed), and every
wait is bounded (a timeout sets the status word that ``dion_b200.ops.gemm.check_status`` reads).
This replaces dion/megabatch_base.py:713-834 of the reference for 2-D parameters sharded by
rows (evenly or not) or evenly by columns; other layouts use the collective path.

Column shards (a ``Shard(1)`` placement, e.g. the FSDP dimension of a row-parallel weight) take
the same four steps with the roles of the two dimensions exchanged: the momentum kernel stores
its ``[rows, cols/W]`` block at its column offset of the owner's ``[rows, cols]`` matrix (a
strided store), the first Gram GEMM gates on K-slabs where the row form gates on tile rows (and
the other way round), and the last update GEMM sends every 16-byte piece of an output row to the
rank that owns its columns.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from ..ops import gemm
from ..ops.tables import RawPointer
from . import symm


def fused_exchange_enabled() -> bool:
    return os.environ.get("DION_B200_FUSED_EXCHANGE", "1") != "0"


def get_exchange(cache: dict, key, pg, n: int, rows_local: int, cols: int,
                 device: torch.device, by_columns: bool = False) -> "FusedRowExchange":
    """Workspace of a bucket, created (collectively, on first use) and then kept."""
    fx = cache.get(key)
    if fx is None:
        fx = cache[key] = FusedRowExchange(pg, n, rows_local, cols, device, by_columns)
    return fx


def eligible(local_shape: Sequence[int], comm_dim: Optional[int], global_rows: Optional[int],
             world: int, pg: Optional[ProcessGroup], ns_func, flatten: bool,
             split_sizes, allow_uneven: bool = False, allow_columns: bool = False) -> bool:
    """All ranks must reach the same decision, so only rank-independent facts are used (the
    number of local rows is not one of them).  ``allow_uneven``: the caller copes with ranks that
    hold fewer than ``ceil(global_rows / world)`` rows, or none; every rank's slice of the
    assembled matrix then has that padded height, the missing rows staying zero as in the
    collective path (reference: dion/megabatch_base.py:740-782).  ``allow_columns``: the caller
    also handles even column shards (``comm_dim == -1``; ``global_rows`` is then the unsharded
    number of columns)."""
    if not fused_exchange_enabled() or pg is None or len(local_shape) != 2:
        return False
    if comm_dim != -2 and not (allow_columns and comm_dim == -1):
        return False
    if flatten or split_sizes is not None or world < 2 or world > 8:
        return False
    if getattr(ns_func, "ns_spec", None) is None:
        return False
    if global_rows is None or global_rows < 1:
        return False
    if comm_dim == -1:
        # Column shards (``global_rows`` is the size of the sharded dimension): even blocks of
        # whole 32-column chunks, so that every 16-byte piece of an output row and every
        # 32-column epilogue chunk has one destination.
        if global_rows % world != 0 or (global_rows // world) % 32 or local_shape[0] % 8:
            return False
        if local_shape[1] * world != global_rows:   # also sharded over another mesh dimension
            return False
        return symm.symmetric_memory_available(pg)
    if global_rows % world != 0 and not allow_uneven:
        return False
    padded = -(-global_rows // world) * world
    if padded % 8:      # the Gram matrix of the assembled rows is itself a TMA operand
        return False
    if local_shape[1] % 8:
        return False
    return symm.symmetric_memory_available(pg)


class FusedRowExchange:
    """Persistent symmetric workspace and flag protocol for one bucket of ``n`` matrices whose
    local shards are ``[rows_local, cols]``, sharded over ``world`` ranks by rows (assembled:
    ``[world*rows_local, cols]``) or, with ``by_columns``, by columns (assembled:
    ``[rows_local, world*cols]``)."""

    def __init__(self, pg: ProcessGroup, n: int, rows_local: int, cols: int,
                 device: torch.device, by_columns: bool = False):
        self.pg = pg
        self.by_columns = by_columns
        self.rank = dist.get_rank(pg)
        self.world = W = dist.get_world_size(pg)
        self.n = n
        self.per_rank = (n + W - 1) // W
        self.n_total = self.per_rank * W
        self.pl, self.cols = rows_local, cols
        self.device = device

        lay = symm.Layout()
        self.off_recv = lay.add("recv", self.per_rank * W * rows_local * cols * 2)
        self.off_ret = lay.add("ret", self.n_total * rows_local * cols * 2)
        self.off_part = lay.add("partials", self.per_rank * W * 4)
        self.off_flags = {name: lay.add(name, W * 4)
                          for name in ("data", "ack", "ret", "ret_ack")}
        self.buf = symm.SymmetricBuffer(lay.size, pg)
        b = self.buf
        full = (rows_local, W * cols) if by_columns else (W * rows_local, cols)
        self.recv = b.view(self.off_recv, (self.per_rank,) + full, torch.bfloat16)
        self.ret = b.view(self.off_ret, (self.n_total, rows_local, cols), torch.bfloat16)
        self.partials = b.view(self.off_part, (self.per_rank, W), torch.float32)
        self.flags = {k: b.view(off, (W,), torch.int32) for k, off in self.off_flags.items()}
        self.peer_flag_tables = {
            k: symm.address_table([b.peer_address(p, off) for p in range(W)], device)
            for k, off in self.off_flags.items()}
        self.seq = torch.zeros((), dtype=torch.int32, device=device)
        self.scale = torch.empty(self.per_rank, dtype=torch.float32, device=device)
        self.status = gemm.status_tensor(device)
        self.norm_mult, self.eps = 1.0, 1e-7

    # -- producer side ------------------------------------------------------------------------
    def begin(self) -> None:
        """Open a round: advance the sequence number and wait until every owner has consumed
        what this rank pushed in the previous round."""
        symm.bump_seq(self.seq)
        symm.wait_flags(self.flags["ack"], self.seq, -1, self.status)

    def push_targets(self) -> Tuple[List[RawPointer], List[int]]:
        """Per matrix ``i``: where this rank's bf16 shard goes (rows ``rank*pl ...``, or columns
        ``rank*cols ...``, of matrix ``i % per_rank`` on rank ``i // per_rank``) and where its
        sum of squares is added."""
        W, pl, cols, pr = self.world, self.pl, self.cols, self.per_rank
        outs, sums = [], []
        for i in range(self.n):
            owner, j = divmod(i, pr)
            if self.by_columns:
                data_off = self.off_recv + (j * W * pl * cols + self.rank * cols) * 2
            else:
                data_off = self.off_recv + ((j * W + self.rank) * pl * cols) * 2
            outs.append(RawPointer(self.buf.peer_address(owner, data_off)))
            sums.append(self.buf.peer_address(owner, self.off_part + (j * W + self.rank) * 4))
        return outs, sums

    def push_block(self) -> Optional[Tuple[int, int]]:
        """``(columns, row pitch)`` of the strided store a column shard needs (else ``None``)."""
        return (self.cols, self.world * self.cols) if self.by_columns else None

    def publish(self) -> None:
        """Tell every owner that this rank's shards (and partial sums) have been stored."""
        symm.signal_peers(self.peer_flag_tables["data"], self.rank, self.seq)

    # -- hooks used by the Newton-Schulz driver -----------------------------------------------
    def first_gram(self, tall: bool) -> gemm.GemmExtra:
        ex = gemm.GemmExtra()
        ex.wait_flags = self.flags["data"].data_ptr()
        ex.seq_ptr = self.seq.data_ptr()
        # The sharded dimension indexes the Gram matrix's rows and columns when it is the
        # shorter one of the assembled matrix, and is the contraction otherwise.
        ex.n_src, ex.rows_per_src = self.world, (self.cols if self.by_columns else self.pl)
        contracted = (not tall) if self.by_columns else tall
        ex.wait_a = ex.wait_b = 0 if contracted else 1
        ex.wait_k = 1 if contracted else 0
        ex.scale_partials = self.partials.data_ptr()
        ex.scale_mult, ex.scale_eps = self.norm_mult, self.eps
        return ex

    def scale_after_first_gram(self) -> Tensor:
        symm.scale_from_partials(self.partials, self.per_rank, self.world, self.norm_mult,
                                 self.eps, self.scale, clear=True)
        return self.scale

    def after_first_iteration(self) -> None:
        """The received shards have been read for the last time: hand the buffer back."""
        symm.signal_peers(self.peer_flag_tables["ack"], self.rank, self.seq)

    def last_update(self) -> gemm.GemmExtra:
        symm.wait_flags(self.flags["ret_ack"], self.seq, -1, self.status)
        ex = gemm.GemmExtra()
        for p in range(self.world):
            ex.remote_c[p] = self.buf.peer_address(p, self.off_ret)
        ex.rows_per_dst = self.pl
        ex.cols_per_dst = self.cols if self.by_columns else 0
        ex.remote_slot = self.rank * self.per_rank
        return ex

    def finish(self) -> None:
        """All result rows have been stored into their owners' return buffers."""
        symm.signal_peers(self.peer_flag_tables["ret"], self.rank, self.seq)

    # -- consumer side ------------------------------------------------------------------------
    def result_views(self, rows: Optional[int] = None) -> List[Tensor]:
        """Updates of this rank's shards; ``rows`` < padded height when the shard is ragged."""
        if rows is None or rows == self.pl:
            return [self.ret[i] for i in range(self.n)]
        return [self.ret[i][:rows] for i in range(self.n)]

    def result_wait(self):
        """Argument for ``foreach.muon_post(wait=...)``: matrix ``i`` was produced by rank
        ``i // per_rank``."""
        return (self.flags["ret"], self.seq, self.per_rank, self.status)

    def wait_results(self) -> None:
        """Stream-level wait (bounded) until every producing rank has stored its results; for
        consumers that do not poll the flags themselves."""
        symm.wait_flags(self.flags["ret"], self.seq, 0, self.status)

    def result_stack(self) -> Tensor:
        """``[n, rows_local, cols]`` view of the returned updates."""
        return self.ret[: self.n]

    def release(self) -> None:
        """The update has been applied: producers may overwrite the return buffer."""
        symm.signal_peers(self.peer_flag_tables["ret_ack"], self.rank, self.seq)

    def input_matrix(self) -> Tensor:
        return self.recv
