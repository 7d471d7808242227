"""Megabatch orthogonalization: every same-shape matrix of a parameter group goes through one
communication round and one batched Newton-Schulz call.

Four layouts (reference: dion/megabatch_base.py:635-881):

* sharded     every rank holds a slice of every matrix along ``comm_dim`` (FSDP2).  One
              all-to-all assembles ``N/W`` whole matrices per rank, Newton-Schulz runs on them,
              and one all-to-all returns the slices.  Shards are zero-padded to a uniform size
              so that uneven or empty shards exchange equal-sized messages.
* replicated  every rank holds every matrix (DDP).  Rank ``r`` orthogonalizes matrices
              ``[r*N/W, (r+1)*N/W)`` and the results are all-gathered.
* single      one matrix, or no process group: local batched Newton-Schulz.

The exchange buffers are laid out so that the producer kernel can write its bf16 output straight
into the send buffer (``MegabatchPlan.input_views``) and the consumer reads the received update
in place.  The collectives use the tensor forms (``all_to_all_single`` /
``all_gather_into_tensor``), which both NCCL and gloo implement.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Callable, Generator, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup

from ..utils.arena import StepArena, alloc as _alloc
from .async_runtime import run_to_completion


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def newton_schulz_dispatch(
    X: Tensor,
    newton_schulz_func: Callable,
    flatten: bool,
    epsilon,
    split_sizes: Optional[Tuple[int, ...]] = None,
    split_scales: Optional[Tuple[float, ...]] = None,
) -> Tensor:
    """Shape handling around the Newton-Schulz callable.  ``X`` is a stack ``[N, *param_shape]``.
    With ``flatten`` every parameter is folded to ``[shape[0], prod(shape[1:])]`` (convolution
    kernels); otherwise parameters with more than two dims are batches of matrices and their
    leading dims join the batch.  ``split_sizes`` orthogonalizes row blocks independently
    (reference: megabatch_base.py:884-949; there the fold is applied to whatever tensor reaches
    the function, which for a stack of several parameters also folds the parameter's own first
    dim - here the documented per-parameter meaning is applied for any number of parameters, and
    the two agree for a single parameter)."""
    if split_sizes is not None:
        assert not flatten, "split_sizes is incompatible with flatten=True"
        return _row_block_newton_schulz(X, split_sizes, split_scales, newton_schulz_func, epsilon)
    shape = X.shape
    if flatten:
        if X.ndim >= 4:
            X = X.flatten(start_dim=2)
    elif X.ndim >= 4:
        X = X.flatten(end_dim=-3)
    return newton_schulz_func(X, epsilon=epsilon).reshape(shape)


def _row_block_newton_schulz(X, split_sizes, split_scales, newton_schulz_func, epsilon) -> Tensor:
    if X.size(-2) != sum(split_sizes):
        raise AssertionError(
            f"dim -2 of input ({X.size(-2)}) does not match sum of split_sizes ({split_sizes})")
    blocks = X.split(list(split_sizes), dim=-2)
    by_height = defaultdict(list)
    for i, blk in enumerate(blocks):
        by_height[blk.size(-2)].append(i)
    done: List[Optional[Tensor]] = [None] * len(blocks)
    for ids in by_height.values():
        group = torch.stack([blocks[i] for i in ids], dim=0)
        flat = group.flatten(end_dim=-3) if group.ndim > 3 else group
        ortho = newton_schulz_func(flat, epsilon=epsilon).reshape(group.shape)
        for j, i in enumerate(ids):
            blk = ortho[j]
            if split_scales is not None:
                blk = blk * split_scales[i]
            done[i] = blk
    return torch.cat(done, dim=-2)


class MegabatchPlan:
    """Buffer layout and schedule of one megabatch round.

    ``local_shape`` is the shape of one rank-local input (a shard on the sharded path), ``n``
    the number of matrices.  ``comm_dim`` (negative) is the sharded matrix dimension or None.
    """

    def __init__(
        self,
        local_shape: Sequence[int],
        n: int,
        device: torch.device,
        comm_dim: Optional[int],
        device_rank: int,
        world_size: int,
        process_group: Optional[ProcessGroup],
        global_comm_dim_size: Optional[int] = None,
        local_comm_size: Optional[int] = None,
        split_sizes: Optional[Tuple[int, ...]] = None,
        arena: Optional[StepArena] = None,
    ):
        self.arena = arena
        self.n = n
        self.local_shape = tuple(local_shape)
        self.device = device
        self.rank = device_rank
        self.world = world_size
        self.pg = process_group
        self.comm_dim = comm_dim
        if process_group is not None and comm_dim is not None:
            self.mode = "sharded"
        elif process_group is not None and n > 1:
            self.mode = "replicated"
        else:
            self.mode = "single"

        if self.mode == "single":
            self.n_total, self.per_rank = n, n
        else:
            self.n_total = _ceil_div(n, world_size) * world_size
            self.per_rank = self.n_total // world_size

        self.padded_shape = self.local_shape
        if self.mode == "sharded":
            if comm_dim >= 0:
                raise ValueError("comm_dim must be a negative index")
            if global_comm_dim_size is None:
                raise ValueError(
                    "global_comm_dim_size must be passed when comm_dim is not None; callers "
                    "should pass the unsharded DTensor's global size along comm_dim.")
            original = self.local_shape[comm_dim]
            if local_comm_size is not None:
                if split_sizes is not None:
                    raise NotImplementedError(
                        "local_comm_size (row-sharded 'local' selection) is not supported "
                        "together with split_sizes; the per-rank pad-to-k would intersperse "
                        "zero rows within the assembled row blocks.")
                padded = local_comm_size
            else:
                padded = _ceil_div(global_comm_dim_size, world_size)
            if (split_sizes is not None and comm_dim == -2
                    and padded * world_size != global_comm_dim_size):
                raise NotImplementedError(
                    f"split_sizes requires dim 0 of the parameter ({global_comm_dim_size}) to be "
                    f"divisible by the sharding world_size ({world_size}) so the assembled "
                    f"matrices have no interspersed padding rows.")
            if padded < original:
                raise RuntimeError(
                    f"padded_local_size ({padded}) < this rank's local size ({original}); "
                    f"contiguous-chunk sharding assumption violated "
                    f"(global_comm_dim_size={global_comm_dim_size}, world_size={world_size}).")
            self.original_local = original
            self.padded_local = padded
            shp = list(self.local_shape)
            shp[comm_dim] = padded
            self.padded_shape = tuple(shp)
        self._send: Optional[Tensor] = None

    # -- producer side ------------------------------------------------------------------------
    def _alloc_send(self) -> Tensor:
        if self.mode == "sharded":
            needs_zero = self.n_total != self.n or self.padded_shape != self.local_shape
            shape = (self.world, self.per_rank) + self.padded_shape
        elif self.mode == "replicated":
            needs_zero = self.n_total != self.n
            shape = (self.per_rank,) + self.local_shape
        else:
            needs_zero = False
            shape = (self.n,) + self.local_shape
        return _alloc(self.arena, shape, torch.bfloat16, self.device, zero=needs_zero)

    def input_views(self) -> List[Optional[Tensor]]:
        """Where the bf16 Newton-Schulz input of matrix ``i`` has to be written.  ``None`` means
        that this rank does not need matrix ``i`` (replicated path, another rank owns it).
        Views are contiguous unless a column shard is padded."""
        self._send = self._alloc_send()
        s = self._send
        if self.mode == "sharded":
            flat = s.view((self.n_total,) + self.padded_shape)
            views = [flat[i] for i in range(self.n)]
            if self.padded_shape != self.local_shape:
                views = [v.narrow(self.comm_dim, 0, self.original_local) for v in views]
            return views
        if self.mode == "replicated":
            lo = self.rank * self.per_rank
            return [s[i - lo] if lo <= i < lo + self.per_rank else None for i in range(self.n)]
        return [s[i] for i in range(self.n)]

    def load(self, U: Sequence[Tensor]) -> None:
        """Copy already computed inputs into the exchange buffer."""
        for v, u in zip(self.input_views(), U):
            if v is not None and v.numel():
                v.copy_(u)

    def _stable(self, t: Tensor) -> Tensor:
        """Move a result into arena memory so that its address is the same every step."""
        if self.arena is None:
            return t
        out = self.arena.alloc(t.shape, t.dtype, t.device)
        out.copy_(t)
        return out

    # -- schedule -----------------------------------------------------------------------------
    def run(
        self,
        newton_schulz_func: Callable,
        flatten: bool,
        epsilon,
        split_sizes: Optional[Tuple[int, ...]] = None,
        split_scales: Optional[Tuple[float, ...]] = None,
    ) -> Generator[None, None, Tensor]:
        """Generator: yields while a collective is in flight; returns the orthogonalized stack
        ``[n, *local_shape]`` in parameter order."""
        assert self._send is not None, "call input_views() or load() first"
        send, self._send = self._send, None
        ns = lambda X: newton_schulz_dispatch(  # noqa: E731
            X, newton_schulz_func, flatten, epsilon, split_sizes, split_scales)

        if self.mode == "single":
            return self._stable(ns(send))

        if self.mode == "replicated":
            mine = ns(send).contiguous()
            gathered = _alloc(self.arena, (self.n_total,) + self.local_shape, mine.dtype,
                              self.device)
            work = dist.all_gather_into_tensor(gathered, mine, group=self.pg, async_op=True)
            yield
            work.wait()
            return gathered[: self.n]

        # sharded
        W, pr, cd = self.world, self.per_rank, self.comm_dim
        recv = _alloc(self.arena, send.shape, send.dtype, self.device)
        work = dist.all_to_all_single(recv, send, group=self.pg, async_op=True)
        yield
        work.wait()
        nd = len(self.padded_shape)
        # recv[src, j] is rank src's slice of my j-th matrix: concatenate slices along comm_dim.
        dst_dim = 1 + (nd + cd)            # position of comm_dim in [per_rank, *shape]
        full = recv.movedim(0, dst_dim)    # [pr, ..., W, padded_local, ...]
        full_shape = list(self.padded_shape)
        full_shape[cd] = W * self.padded_local
        full = full.reshape([pr] + full_shape)
        full = ns(full)
        # Split back into per-destination slices: [W, pr, *padded_shape]
        parts = full.reshape([pr] + list(self.padded_shape[: nd + cd]) + [W, self.padded_local]
                             + list(self.padded_shape[nd + cd + 1:]))
        back = parts.movedim(dst_dim, 0).contiguous()
        ret = _alloc(self.arena, back.shape, back.dtype, self.device)
        work = dist.all_to_all_single(ret, back, group=self.pg, async_op=True)
        yield
        work.wait()
        out = ret.view((self.n_total,) + self.padded_shape)[: self.n]
        if self.padded_shape != self.local_shape:
            out = out.narrow(cd, 0, self.original_local)
        return out


def megabatch_orthogonalize_async(
    U: List[Tensor],
    comm_dim: Optional[int],
    device_rank: int,
    world_size: int,
    process_group: Optional[ProcessGroup],
    newton_schulz_func: Callable,
    flatten: bool,
    epsilon,
    global_comm_dim_size: Optional[int],
    split_sizes: Optional[Tuple[int, ...]] = None,
    split_scales: Optional[Tuple[float, ...]] = None,
    return_stacked: bool = False,
    local_comm_size: Optional[int] = None,
    arena: Optional[StepArena] = None,
) -> Generator[None, None, Union[List[Tensor], Tensor]]:
    """List-in/list-out form of a megabatch round with the reference's signature
    (dion/megabatch_base.py:635-649).  ``result = yield from megabatch_orthogonalize_async(...)``."""
    plan = MegabatchPlan(
        U[0].shape, len(U), U[0].device, comm_dim, device_rank, world_size, process_group,
        global_comm_dim_size=global_comm_dim_size, local_comm_size=local_comm_size,
        split_sizes=split_sizes, arena=arena)
    plan.load(U)
    out = yield from plan.run(newton_schulz_func, flatten, epsilon, split_sizes, split_scales)
    return out if return_stacked else list(out.unbind(0))


def megabatch_orthogonalize(*args, **kwargs):
    """Synchronous form of :func:`megabatch_orthogonalize_async`."""
    return run_to_completion(megabatch_orthogonalize_async(*args, **kwargs))
