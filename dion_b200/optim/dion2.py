"""Dion2: orthogonalize only a fraction of the rows (or columns) of the momentum each step, with
error feedback on the selected part (reference: dion/dion2.py:19-740).

Per bucket: ``M += G``; the ``k`` slices with the largest L1 norm are gathered into a dense bf16
sub-matrix and decayed by ``ef_decay`` inside ``M``; the sub-matrices go through the megabatch
Newton-Schulz; then ``X`` is decayed everywhere and updated on the selected slices with a single
rounding.  Selection, gather and error feedback are three kernels of ``csrc/select_ops.cu``;
the post-update of all parameters is one launch.

``selection_scope="local"`` (default) selects per shard before communication, so traffic and
Newton-Schulz work shrink by ``fraction``; ``"global"`` sends whole shards and takes the exact
top-k on the assembled matrix.
"""
from __future__ import annotations

import math
from typing import Callable, Generator, Iterable, List, Optional, Tuple, Union

import torch
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh
from torch.optim.optimizer import ParamsT

from ..ops import foreach as F
from ..ops import newton_schulz as NS
from ..parallel import fused_exchange as FX
from ..ops.select import _as_matrices, dion2_select, scatter_selected
from ..parallel.async_runtime import AsyncTask
from ..parallel.megabatch import MegabatchPlan
from ..utils.tensors import group_by_shape, to_local
from .muon import _validate_common, contiguous_list, global_comm_size
from .ortho_base import DistributedOrthoBase, lr_ratio


def _validate_dion2(fraction, selection_scope):
    if not (0.0 < fraction <= 1.0):
        raise ValueError(f"fraction must be in (0, 1], got {fraction}")
    if selection_scope not in ("local", "global"):
        raise ValueError(f"selection_scope must be 'local' or 'global', got {selection_scope!r}")


class Dion2(DistributedOrthoBase):
    """Distributed Dion2.

    Args beyond :class:`Muon`: ``fraction`` of rows/columns orthogonalized per step,
    ``ef_decay`` applied to the selected part of the momentum, ``selection_scope``
    (``"local"`` / ``"global"``), ``verbose`` (print the row/column choice once per shape).
    ``triton_post_ortho`` is accepted and ignored: the single-rounding fused post-update is the
    only implementation here.  ``split_sizes`` groups are not supported.
    """

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        lr: float = 0.01,
        fraction: float = 0.25,
        ef_decay: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: Union[float, Tensor] = 0.01,
        epsilon: float = 1e-8,
        adjust_lr: Optional[str] = "spectral_norm",
        flatten: bool = False,
        use_triton: bool = False,
        use_polar_express: bool = True,
        use_gram_newton_schulz: bool = False,
        newton_schulz_func: Optional[Callable] = None,
        verbose: bool = False,
        triton_post_ortho: bool = False,
        selection_scope: str = "local",
    ):
        _validate_common(lr, None, betas, adjust_lr)
        _validate_dion2(fraction, selection_scope)
        if ef_decay < 0.0:
            raise ValueError(f"Invalid ef_decay: {ef_decay}")
        defaults = dict(
            lr=lr, ef_decay=ef_decay, fraction=float(fraction), beta1=betas[0], beta2=betas[1],
            weight_decay=weight_decay, epsilon=epsilon, flatten=flatten, adjust_lr=adjust_lr,
            algorithm="dion2", step=0, selection_scope=selection_scope)
        super().__init__(
            params, distributed_mesh, "dion2", defaults,
            use_gram_newton_schulz=use_gram_newton_schulz, use_triton=use_triton,
            use_polar_express=use_polar_express, newton_schulz_func=newton_schulz_func)
        self.verbose = verbose
        self._triton_post_ortho = triton_post_ortho

    def _create_ortho_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            assert all(p.ndim >= 2 for p in group["params"]), \
                "Dion2 only supports matrix parameters."
            with_grad = [p for p in group["params"] if p.grad is not None]
            if not with_grad:
                continue
            num_heads = self._resolve_num_heads(group)
            if group.get("split_sizes") is not None:
                raise NotImplementedError(
                    "split_sizes is currently supported only by Muon and NorMuon.")
            for params in group_by_shape(with_grad).values():
                grads = [p.grad for p in params]
                moms = [self._get_or_initialize_state(p, self._algo_name)["momentum"]
                        for p in params]
                pg, shard_dim = self._bucket_layout(group, params, num_heads)
                if num_heads is not None:
                    params, grads, moms = self._prepare_head_split(num_heads, params, grads, moms)
                yield AsyncTask(dion2_update_megabatch_async(
                    X=params, G=grads, M=moms, lr=group["lr"], ef_decay=group["ef_decay"],
                    fraction=group["fraction"], weight_decay=group["weight_decay"],
                    epsilon=group["epsilon"], flatten=group["flatten"],
                    adjust_lr=group["adjust_lr"], device_rank=self._device_rank,
                    world_size=self._world_size, shard_dim=shard_dim, process_group=pg,
                    newton_schulz_func=self._newton_schulz_func, arena=self._arena,
                    fused_cache=self._fused_exchanges, verbose=self.verbose,
                    selection_scope=group["selection_scope"]))


def choose_select_dim(shape, shard_dim: Optional[int], ndim: int) -> int:
    """Sharded matrices select along the sharded dim; whole matrices along the shorter one."""
    if shard_dim is not None:
        neg = shard_dim if shard_dim < 0 else shard_dim - ndim
        if neg in (-1, -2):
            return neg
    rows, cols = shape[-2:]
    return -2 if rows <= cols else -1


def selection_count(fraction: float, comm_dim, global_dim_size, world_size) -> Optional[int]:
    """Per-rank number of selected slices on the sharded "local" path: every rank uses
    ``ceil(fraction * ceil(global / W))`` so that the exchange stays uniform."""
    if comm_dim is None:
        return None
    padded_local = (global_dim_size + world_size - 1) // world_size
    return max(1, int(math.ceil(fraction * padded_local)))


def dion2_update_megabatch_async(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    lr,
    ef_decay,
    fraction: float,
    weight_decay,
    epsilon,
    flatten: bool,
    adjust_lr: Optional[str],
    device_rank: int,
    world_size: int,
    shard_dim: Optional[int] = None,
    process_group: Optional[ProcessGroup] = None,
    newton_schulz_func: Optional[Callable] = None,
    verbose: bool = False,
    triton_post_ortho: bool = False,
    selection_scope: str = "local",
    arena=None,
    fused_cache=None,
) -> Generator[None, None, None]:
    assert len(X) == len(G) == len(M)
    ndim = X[0].ndim
    select_dim = choose_select_dim(X[0].shape, shard_dim, ndim)
    if verbose:
        _print_selection_choice(X[0].shape, shard_dim, select_dim, ndim)
    comm_dim = select_dim if shard_dim is not None else None
    global_dim = global_comm_size(X[0], comm_dim)
    Xl, Gl, Ml = to_local(X), to_local(G), to_local(M)
    ratio = lr_ratio(adjust_lr, X[0].shape, flatten)
    N = len(X)

    if selection_scope == "global" and comm_dim is not None:
        plan = MegabatchPlan(Ml[0].shape, N, Ml[0].device, comm_dim, device_rank, world_size,
                             process_group, global_comm_dim_size=global_dim, arena=arena)
        F.muon_pre(Gl, Ml, 0.0, False, out=plan.input_views(), add_only=True)
        select_ns = make_select_and_orthogonalize(
            newton_schulz_func, fraction, select_dim, global_select_size=global_dim)
        U = yield from plan.run(select_ns, flatten, epsilon)
        dion2_post_orthogonalize_masked(Xl, Ml, list(U.unbind(0)), lr, ratio, weight_decay,
                                        float(ef_decay), select_dim)
        return

    k = selection_count(fraction, comm_dim, global_dim, world_size)
    num_select = Ml[0].size(select_dim)
    if k is None:
        k = max(1, int(math.ceil(fraction * num_select)))
    k_topk = min(k, num_select)
    if fused_cache is not None and FX.eligible(Ml[0].shape, comm_dim, global_dim, world_size,
                                               process_group, newton_schulz_func, flatten, None):
        # Row-sharded "local" selection with the exchange inside the kernels: the gather kernel
        # stores each rank's k selected rows straight into the owners' receive buffers, the
        # Newton-Schulz kernels consume them as they arrive and return their rows to the shards.
        fx = FX.get_exchange(fused_cache, (id(X[0]), N, k, Ml[0].shape[1]), process_group, N, k,
                             Ml[0].shape[1], Ml[0].device)
        fx.begin()
        outs, sums = fx.push_targets()
        _, idx, maps = dion2_select(Gl, Ml, k, select_dim, float(ef_decay),
                                    out_addresses=[o.address for o in outs],
                                    sumsq_addresses=sums)
        fx.publish()
        NS.iterate_with_exchange(fx.input_matrix(), newton_schulz_func, epsilon, fx)
        fx.finish()
        F.dion2_post(Xl, list(fx.result_stack().unbind(0)), list(idx.unbind(0)),
                     list(maps.unbind(0)), lr, weight_decay, ratio, select_dim,
                     wait=fx.result_wait())
        fx.release()
        yield
        return
    U_sel, idx, maps = dion2_select(Gl, Ml, k_topk, select_dim, float(ef_decay))
    batch_shape = Ml[0].shape[:-2]
    sel_shape = tuple(batch_shape) + tuple(U_sel.shape[-2:])
    plan = MegabatchPlan(sel_shape, N, Ml[0].device, comm_dim, device_rank, world_size,
                         process_group, global_comm_dim_size=global_dim,
                         local_comm_size=k if comm_dim is not None else None, arena=arena)
    plan.load(U_sel.reshape((N,) + sel_shape).unbind(0))
    U = yield from plan.run(newton_schulz_func, flatten, epsilon)
    if num_select == 0:
        return  # empty shard: nothing of these parameters lives on this rank
    Um = contiguous_list(U.reshape((-1,) + tuple(U.shape[-2:])))
    F.dion2_post(_as_matrices(Xl), Um, list(idx.unbind(0)),
                 list(maps.unbind(0)) if maps is not None else None,
                 lr, weight_decay, ratio, select_dim)


def make_select_and_orthogonalize(
    newton_schulz_func: Callable,
    fraction: float,
    select_dim: int,
    global_select_size: Optional[int] = None,
) -> Callable:
    """Wrap a Newton-Schulz callable so that it orthogonalizes only the exact top-``k`` slices of
    each (assembled) matrix and returns a full-size tensor that is zero elsewhere.  ``k`` comes
    from the true unsharded size, not from the zero-padded matrix (reference: dion2.py:565-617)."""

    def select_ns(X: Tensor, epsilon=None) -> Tensor:
        size = X.size(select_dim)
        num = size if global_select_size is None else global_select_size
        k = min(max(1, int(math.ceil(fraction * num))), size)
        X3 = X if X.ndim == 3 else X.reshape((-1,) + tuple(X.shape[-2:]))
        sub, idx, _ = dion2_select(None, list(X3.unbind(0)), k, select_dim, 1.0, apply_ef=False)
        ortho = newton_schulz_func(sub, epsilon=epsilon).to(X.dtype)
        return scatter_selected(ortho.contiguous(), idx, size, select_dim).reshape(X.shape)

    return select_ns


def dion2_post_orthogonalize_masked(
    X: List[Tensor], M: List[Tensor], U: List[Tensor], lr, ratio: float, weight_decay,
    ef_decay: float, select_dim: int,
) -> None:
    """Global-scope post step: ``U`` is full-size and exactly zero off the selected slices, which
    are recognised by being non-zero (orthonormal slices have unit norm).  Decays ``X``, applies
    ``ef_decay`` to the selected slices of ``M`` and adds the update."""
    F.dion2_post_masked(X, M, U, lr, weight_decay, ratio, ef_decay, select_dim)


def dion2_pre_orthogonalize(G, M, fraction, ef_decay, select_dim, k_override=None):
    """List form of the select step: ``-> (U_selected list, indices list)``
    (reference: dion/dion2.py:437-547)."""
    num = M[0].size(select_dim)
    k = k_override if k_override is not None else max(1, int(math.ceil(fraction * num)))
    k = min(k, num)
    U, idx, _ = dion2_select(G, M, k, select_dim, float(ef_decay))
    if num == 0:
        return [m.to(torch.bfloat16) for m in M], \
            [torch.empty(0, dtype=torch.long, device=M[0].device) for _ in M]
    n = len(M)
    U = U.reshape((n,) + tuple(M[0].shape[:-2]) + tuple(U.shape[-2:]))
    idx = idx.reshape((n,) + tuple(M[0].shape[:-2]) + (k,))
    return list(U.unbind(0)), list(idx.unbind(0))


def dion2_post_orthogonalize(X, U, indices, base_lr, adjusted_lr, weight_decay, select_dim):
    """List form of the post step (single rounding; reference: dion/dion2.py:701-740)."""
    ratio = adjusted_lr / base_lr
    ratio = float(ratio) if not isinstance(ratio, float) else ratio
    F.dion2_post(X, U, indices, None, base_lr, weight_decay, ratio, select_dim)


dion2_post_orthogonalize_fused = dion2_post_orthogonalize

_printed_configs: set = set()


def _print_selection_choice(shape, shard_dim, select_dim, ndim) -> None:
    key = (tuple(shape), shard_dim, select_dim)
    if key in _printed_configs:
        return
    _printed_configs.add(key)
    rows, cols = shape[-2:]
    what = "rows" if select_dim == -2 else "columns"
    if shard_dim is None:
        why = f"unsharded, shorter dim = {'rows' if rows <= cols else 'cols'} ({min(rows, cols)})"
    else:
        neg = shard_dim if shard_dim < 0 else shard_dim - ndim
        why = {-2: "row-sharded", -1: "column-sharded"}.get(neg, f"batch-sharded (dim {shard_dim})")
    print(f"[Dion2] shape {tuple(shape)}: {why} -> select top-fraction {what} by L1 norm")
