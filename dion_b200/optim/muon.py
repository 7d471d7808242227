"""Muon: momentum, Newton-Schulz orthogonalization of the update, decoupled weight decay.

Public surface and numerics follow dion/muon.py:20-347 of the reference; the step itself is
organised around :class:`MegabatchPlan`: the momentum kernel writes the bf16 Newton-Schulz input
straight into the exchange buffer, the batched tcgen05 Newton-Schulz runs on whole matrices, and
one multi-tensor kernel applies weight decay and the update.
"""
from __future__ import annotations

from typing import Callable, Generator, Iterable, List, Optional, Tuple, Union

import torch
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor
from torch.optim.optimizer import ParamsT

from ..ops import foreach as F
from ..ops import newton_schulz as NS
from ..parallel import fused_exchange as FX
from ..parallel.async_runtime import AsyncTask
from ..parallel.megabatch import MegabatchPlan
from ..utils.tensors import group_by_shape, to_local
from .ortho_base import DistributedOrthoBase, compute_split_lr_scales, lr_ratio


def _validate_common(lr, mu=None, betas=(0.9, 0.95), adjust_lr="spectral_norm"):
    if lr < 0.0:
        raise ValueError(f"Invalid learning rate: {lr}")
    if mu is not None and mu < 0.0:
        raise ValueError(f"Invalid momentum factor (mu): {mu}")
    if len(betas) != 2 or betas[0] < 0.0 or betas[1] < 0.0:
        raise ValueError(f"Invalid betas: {betas}")
    if adjust_lr not in ("spectral_norm", "rms_norm", None):
        raise ValueError(
            f"Invalid adjust_lr value: {adjust_lr}. Must be 'spectral_norm', 'rms_norm', or None.")


def global_comm_size(X0: Tensor, comm_dim: Optional[int]) -> Optional[int]:
    """Unsharded size along ``comm_dim``; needs the DTensor, whose ``.shape`` is global."""
    if comm_dim is None:
        return None
    if not isinstance(X0, DTensor):
        raise TypeError(
            "Sharded path requires X[0] to be a DTensor so .shape gives the global size; "
            f"got {type(X0).__name__}.")
    return X0.shape[comm_dim]


def contiguous_list(stack: Tensor) -> List[Tensor]:
    views = list(stack.unbind(0))
    if views and not views[0].is_contiguous():
        views = list(stack.contiguous().unbind(0))
    return views


class Muon(DistributedOrthoBase):
    """Distributed Muon for FSDP2 (DeviceMesh), DDP (ProcessGroup) or a single device.

    Args:
        params: parameters or param groups.  Groups select their update rule with
            ``algorithm``: ``"muon"`` (default) for matrices, ``"adamw"`` / ``"lion"`` for
            embeddings, heads and vectors.
        distributed_mesh: 1-D DeviceMesh (FSDP2 / HSDP shard mesh) or ProcessGroup (DDP).
        lr: base learning rate; matrix groups scale it by ``adjust_lr``.
        mu: momentum.  betas: AdamW / Lion betas.  weight_decay: float, or a Tensor to keep it
            live under CUDA-graph replay.  cautious_wd: decay only where update and weight agree
            in sign.  nesterov: Nesterov momentum.
        adjust_lr: ``"spectral_norm"`` (sqrt(fan_out/fan_in)), ``"rms_norm"``
            (0.2*sqrt(max(fan_out, fan_in))) or None.
        flatten: treat >=3-D tensors as one ``[d0, prod(rest)]`` matrix instead of a batch.
        use_gram_newton_schulz / use_polar_express / newton_schulz_func: choice of the
            orthogonalization driver (``func(X, epsilon) -> Tensor``); ``use_triton`` is accepted
            and ignored - CUDA tensors always run on this package's kernels.
    Param groups may set ``num_heads`` (per-head orthogonalization of a 2-D weight) or
    ``split_sizes`` (independent row blocks, e.g. fused QKV).
    """

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        lr: float = 0.01,
        mu: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: Union[float, Tensor] = 0.01,
        cautious_wd: bool = False,
        epsilon: float = 1e-8,
        nesterov: bool = False,
        adjust_lr: Optional[str] = "spectral_norm",
        flatten: bool = False,
        use_gram_newton_schulz: bool = False,
        use_triton: bool = False,
        use_polar_express: bool = True,
        newton_schulz_func: Optional[Callable] = None,
    ):
        _validate_common(lr, mu, betas, adjust_lr)
        defaults = dict(
            lr=lr, mu=mu, beta1=betas[0], beta2=betas[1], weight_decay=weight_decay,
            cautious_wd=cautious_wd, algorithm="muon", step=0, epsilon=epsilon,
            nesterov=nesterov, flatten=flatten, adjust_lr=adjust_lr)
        super().__init__(
            params, distributed_mesh, "muon", defaults,
            use_gram_newton_schulz=use_gram_newton_schulz, use_triton=use_triton,
            use_polar_express=use_polar_express, newton_schulz_func=newton_schulz_func)

    def _create_ortho_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            assert all(p.ndim >= 2 for p in group["params"]), \
                "Muon optimizer only supports matrix parameters."
            with_grad = [p for p in group["params"] if p.grad is not None]
            if not with_grad:
                continue
            num_heads = self._resolve_num_heads(group)
            split_sizes = self._resolve_split_sizes(group)
            for params in group_by_shape(with_grad).values():
                grads = [p.grad for p in params]
                moms = [self._get_or_initialize_state(p, "muon")["momentum"] for p in params]
                split_scales = None
                if split_sizes is not None:
                    self._validate_split_shape(split_sizes, params)
                    split_scales = compute_split_lr_scales(
                        split_sizes, params[0].shape, group["adjust_lr"])
                pg, shard_dim = self._bucket_layout(group, params, num_heads)
                if num_heads is not None:
                    params, grads, moms = self._prepare_head_split(num_heads, params, grads, moms)
                yield AsyncTask(muon_update_megabatch_async(
                    X=params, G=grads, M=moms, lr=group["lr"], momentum=group["mu"],
                    weight_decay=group["weight_decay"], epsilon=group["epsilon"],
                    nesterov=group["nesterov"], flatten=group["flatten"],
                    adjust_lr=group["adjust_lr"], device_rank=self._device_rank,
                    world_size=self._world_size, shard_dim=shard_dim, process_group=pg,
                    newton_schulz_func=self._newton_schulz_func, arena=self._arena,
                    fused_cache=self._fused_exchanges,
                    cautious_wd=group["cautious_wd"], split_sizes=split_sizes,
                    split_scales=split_scales))


def muon_update_megabatch_async(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    lr,
    momentum,
    weight_decay,
    epsilon,
    nesterov: bool,
    flatten: bool,
    adjust_lr: Optional[str],
    device_rank: int,
    world_size: int,
    shard_dim: Optional[int] = None,
    process_group: Optional[ProcessGroup] = None,
    newton_schulz_func: Optional[Callable] = None,
    cautious_wd: bool = False,
    split_sizes: Optional[Tuple[int, ...]] = None,
    split_scales: Optional[Tuple[float, ...]] = None,
    arena=None,
    fused_cache=None,
) -> Generator[None, None, None]:
    """One Muon update of all same-shape parameters ``X`` (generator; yields during collectives)."""
    assert len(X) == len(G) == len(M)
    Xl, Gl, Ml = to_local(X), to_local(G), to_local(M)
    comm_dim = (shard_dim - X[0].ndim) if shard_dim is not None else None
    ratio = lr_ratio(adjust_lr, X[0].shape, flatten)
    global_rows = global_comm_size(X[0], comm_dim)
    if fused_cache is not None and FX.eligible(Ml[0].shape, comm_dim, global_rows, world_size,
                                               process_group, newton_schulz_func, flatten,
                                               split_sizes, allow_uneven=True,
                                               allow_columns=True):
        # The exchange is carried by the kernels themselves.  Row shards: every rank's slice of
        # an assembled matrix is `pl` rows high; a rank with fewer rows (or none) fills only what
        # it has, the rest of its slice stays zero.  Column shards are even by eligibility.
        by_cols = comm_dim == -1
        rows, cols = Ml[0].shape
        pl = rows if by_cols else (global_rows + world_size - 1) // world_size
        key = (id(X[0]), len(X), pl, cols, by_cols)
        fx = FX.get_exchange(fused_cache, key, process_group, len(X), pl, cols, Ml[0].device,
                             by_columns=by_cols)
        fx.begin()
        if rows > 0:
            outs, sums = fx.push_targets()
            F.muon_pre(Gl, Ml, float(momentum), nesterov, out=outs, sumsq_targets=sums,
                       out_block=fx.push_block())
        fx.publish()
        NS.iterate_with_exchange(fx.input_matrix(), newton_schulz_func, epsilon, fx)
        fx.finish()
        if rows > 0:
            F.muon_post(Xl, fx.result_views(rows), lr, weight_decay, ratio, cautious_wd,
                        wait=fx.result_wait())
        fx.release()
        yield
        return
    plan = MegabatchPlan(
        Ml[0].shape, len(X), Ml[0].device, comm_dim, device_rank, world_size, process_group,
        global_comm_dim_size=global_comm_size(X[0], comm_dim), split_sizes=split_sizes,
        arena=arena)
    # Momentum update; the bf16 Newton-Schulz input lands in the exchange buffer.
    F.muon_pre(Gl, Ml, float(momentum), nesterov, out=plan.input_views())
    U = yield from plan.run(newton_schulz_func, flatten, epsilon, split_sizes, split_scales)
    F.muon_post(Xl, contiguous_list(U), lr, weight_decay, ratio, cautious_wd)


def muon_update_pre_orthogonalize(G: List[Tensor], M: List[Tensor], momentum, nesterov: bool):
    """List form of the momentum step (reference: dion/muon.py:283-311)."""
    return F.muon_pre(G, M, float(momentum), nesterov)


def muon_update_post_orthogonalize(X, U, base_lr, adjusted_lr, weight_decay, cautious_wd=False):
    """List form of the apply step (reference: dion/muon.py:314-347)."""
    ratio = float(adjusted_lr / base_lr) if not isinstance(adjusted_lr, float) or base_lr else 1.0
    F.muon_post(X, [u.to(torch.bfloat16) if u.dtype != torch.bfloat16 and X[0].is_cuda else u
                    for u in U], base_lr, weight_decay, ratio, cautious_wd)
