"""NorMuon: Muon followed by a per-neuron (per-row) second-moment normalization of the
orthogonalized update (https://arxiv.org/abs/2510.05491; reference: dion/normuon.py:20-399).

After Newton-Schulz, ``V <- lerp(V, mean(U**2, dim=-1), 1 - muon_beta2)``, the update is divided
by ``sqrt(V) + 1e-8`` row-wise and rescaled to keep its Frobenius norm.  Here the row statistics
are one kernel over the stacked update and the division and rescale are folded into the
weight-update kernel, so the normalized update is never written to memory.  On the sharded path
the norms are taken per local shard, as in the reference (normuon.py:301-309).
"""
from __future__ import annotations

from typing import Callable, Generator, Iterable, List, Optional, Tuple, Union

import torch
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh
from torch.optim.optimizer import ParamsT

from ..ops import foreach as F
from ..ops import newton_schulz as NS
from ..parallel import fused_exchange as FX
from ..parallel.async_runtime import AsyncTask
from ..parallel.megabatch import MegabatchPlan
from ..utils.tensors import group_by_shape, to_local
from .muon import _validate_common, global_comm_size
from .ortho_base import DistributedOrthoBase, compute_split_lr_scales, lr_ratio


class NorMuon(DistributedOrthoBase):
    """Distributed NorMuon.  Arguments as :class:`Muon` plus ``muon_beta2`` (EMA factor of the
    per-row second moment).  State per matrix: ``momentum`` and ``variance_neuron`` of shape
    ``[..., rows, 1]``.  Parameters sharded along their last dimension are rejected."""

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        lr: float = 0.01,
        mu: float = 0.95,
        muon_beta2: float = 0.95,
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
        if muon_beta2 < 0.0:
            raise ValueError(f"Invalid muon_beta2: {muon_beta2}")
        defaults = dict(
            lr=lr, mu=mu, muon_beta2=muon_beta2, beta1=betas[0], beta2=betas[1],
            weight_decay=weight_decay, cautious_wd=cautious_wd, algorithm="normuon", step=0,
            epsilon=epsilon, nesterov=nesterov, flatten=flatten, adjust_lr=adjust_lr)
        super().__init__(
            params, distributed_mesh, "normuon", defaults,
            use_gram_newton_schulz=use_gram_newton_schulz, use_triton=use_triton,
            use_polar_express=use_polar_express, newton_schulz_func=newton_schulz_func)

    def _get_or_initialize_state(self, param: Tensor, algo: str) -> dict:
        state = super()._get_or_initialize_state(param, algo)
        if algo == self._algo_name and "variance_neuron" not in state:
            state["variance_neuron"] = torch.zeros_like(param[..., 0:1])
        return state

    def _get_shard_info(self, param: Tensor, group: dict):
        info = super()._get_shard_info(param, group)
        if info[1] and info[2] == param.ndim - 1:
            raise NotImplementedError(
                "NorMuon currently does not support parameters sharded along the last dimension. "
                "Please avoid shards at dim -1.")
        return info

    def _create_ortho_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            assert all(p.ndim >= 2 for p in group["params"]), \
                "NorMuon optimizer only supports matrix parameters."
            with_grad = [p for p in group["params"] if p.grad is not None]
            if not with_grad:
                continue
            num_heads = self._resolve_num_heads(group)
            split_sizes = self._resolve_split_sizes(group)
            for params in group_by_shape(with_grad).values():
                grads = [p.grad for p in params]
                states = [self._get_or_initialize_state(p, "normuon") for p in params]
                moms = [s["momentum"] for s in states]
                var = [s["variance_neuron"] for s in states]
                split_scales = None
                if split_sizes is not None:
                    self._validate_split_shape(split_sizes, params)
                    split_scales = compute_split_lr_scales(
                        split_sizes, params[0].shape, group["adjust_lr"])
                pg, shard_dim = self._bucket_layout(group, params, num_heads)
                if num_heads is not None:
                    params, grads, moms, var = self._prepare_head_split(
                        num_heads, params, grads, moms, var)
                yield AsyncTask(normuon_update_megabatch_async(
                    X=params, G=grads, M=moms, V=var, lr=group["lr"], momentum=group["mu"],
                    muon_beta2=group["muon_beta2"], weight_decay=group["weight_decay"],
                    epsilon=group["epsilon"], nesterov=group["nesterov"],
                    flatten=group["flatten"], adjust_lr=group["adjust_lr"],
                    device_rank=self._device_rank, world_size=self._world_size,
                    shard_dim=shard_dim, process_group=pg,
                    newton_schulz_func=self._newton_schulz_func, arena=self._arena,
                    fused_cache=self._fused_exchanges,
                    cautious_wd=group["cautious_wd"], split_sizes=split_sizes,
                    split_scales=split_scales))


def normuon_update_megabatch_async(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    V: List[Tensor],
    lr,
    momentum,
    muon_beta2,
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
    assert len(X) == len(G) == len(M) == len(V)
    Xl, Gl, Ml, Vl = to_local(X), to_local(G), to_local(M), to_local(V)
    comm_dim = (shard_dim - X[0].ndim) if shard_dim is not None else None
    ratio = lr_ratio(adjust_lr, X[0].shape, flatten)
    global_rows = global_comm_size(X[0], comm_dim)
    if fused_cache is not None and FX.eligible(Ml[0].shape, comm_dim, global_rows, world_size,
                                               process_group, newton_schulz_func, flatten,
                                               split_sizes):
        # Row shards travel through peer-mapped memory inside the kernels (see fused_exchange;
        # shards along the last dimension are refused at construction, as in the reference).
        fx = FX.get_exchange(fused_cache, (id(X[0]), len(X), tuple(Ml[0].shape)), process_group,
                             len(X), Ml[0].shape[0], Ml[0].shape[1], Ml[0].device)
        fx.begin()
        outs, sums = fx.push_targets()
        F.muon_pre(Gl, Ml, float(momentum), nesterov, out=outs, sumsq_targets=sums)
        fx.publish()
        NS.iterate_with_exchange(fx.input_matrix(), newton_schulz_func, epsilon, fx)
        fx.finish()
        fx.wait_results()
        normuon_normalize_and_apply(Xl, fx.result_stack(), Vl, float(muon_beta2), lr,
                                    weight_decay, ratio, cautious_wd, None,
                                    wait=fx.result_wait())
        fx.release()
        yield
        return
    plan = MegabatchPlan(
        Ml[0].shape, len(X), Ml[0].device, comm_dim, device_rank, world_size, process_group,
        global_comm_dim_size=global_rows, split_sizes=split_sizes,
        arena=arena)
    F.muon_pre(Gl, Ml, float(momentum), nesterov, out=plan.input_views())
    U = yield from plan.run(newton_schulz_func, flatten, epsilon, split_sizes, split_scales)
    # Row blocks keep their own Frobenius norm only where whole matrices are local.
    norm_split = split_sizes if (comm_dim is None or process_group is None) else None
    normuon_normalize_and_apply(Xl, U, Vl, float(muon_beta2), lr, weight_decay, ratio,
                                cautious_wd, norm_split)


def normuon_normalize_and_apply(
    X: List[Tensor],
    U: Tensor,
    V: List[Tensor],
    muon_beta2: float,
    lr,
    weight_decay,
    ratio: float,
    cautious_wd: bool,
    split_sizes: Optional[Tuple[int, ...]] = None,
    wait: Optional[tuple] = None,
) -> None:
    """Update ``V`` from the stacked orthogonalized update ``U`` (``[N, ..., rows, cols]``) and
    apply the row-normalized, norm-preserving update to ``X``.  ``wait`` (fused exchange, see
    ``foreach.muon_post``): ``V`` and ``X`` stay untouched once the status word is set."""
    if U.numel() == 0:
        return
    if not U.is_contiguous():
        U = U.contiguous()
    N = U.size(0)
    rows, cols = U.shape[-2], U.shape[-1]
    inner = U[0].numel() // (rows * cols)  # matrices per parameter (batch dims, per-head views)
    if split_sizes is None:
        U3 = U.reshape(N * inner, rows, cols)
        Vm = _matrix_views(V, rows)
        rinv, n_u2, n_new2 = F.normuon_rowstats(U3, Vm, muon_beta2,
                                                guard=wait[3] if wait else None)
        if inner == 1:
            F.muon_post(X, list(U.unbind(0)), lr, weight_decay, ratio, cautious_wd,
                        rowscale=list(rinv.unbind(0)), normU2=n_u2, normNew2=n_new2, wait=wait)
        else:
            Xm = [x.reshape(-1, rows, cols)[j] for x in X for j in range(inner)]
            F.muon_post(Xm, list(U3.unbind(0)), lr, weight_decay, ratio, cautious_wd,
                        rowscale=list(rinv.unbind(0)), normU2=n_u2, normNew2=n_new2)
        return
    # Independent row blocks: each block is a matrix of its own.
    assert inner == 1 and sum(split_sizes) == rows
    start = 0
    for size in split_sizes:
        Ub = U[:, start:start + size].contiguous()
        Vb = [v[start:start + size] for v in V]
        Xb = [x[start:start + size] for x in X]
        rinv, n_u2, n_new2 = F.normuon_rowstats(Ub, Vb, muon_beta2)
        F.muon_post(Xb, list(Ub.unbind(0)), lr, weight_decay, ratio, cautious_wd,
                    rowscale=list(rinv.unbind(0)), normU2=n_u2, normNew2=n_new2)
        start += size


def _matrix_views(V: List[Tensor], rows: int) -> List[Tensor]:
    out: List[Tensor] = []
    for v in V:
        if v.ndim <= 2:
            out.append(v)
        else:
            out.extend(v.reshape(-1, rows, 1).unbind(0))
    return out


def normuon_normalization_stacked(U: Tensor, V: Tensor, muon_beta2,
                                  split_sizes: Optional[Tuple[int, ...]] = None):
    """Functional form on stacked tensors, ``(U [N,rows,cols], V [N,rows,1]) -> (U_hat, V_new)``
    (reference: dion/normuon.py:344-399).  Plain PyTorch; used by tests as the oracle."""
    if split_sizes is not None:
        parts = [normuon_normalization_stacked(u, v, muon_beta2)
                 for u, v in zip(U.split(list(split_sizes), dim=-2),
                                 V.split(list(split_sizes), dim=-2))]
        return torch.cat([p[0] for p in parts], dim=-2), torch.cat([p[1] for p in parts], dim=-2)
    Uc = U.to(V.dtype)
    norm_u = Uc.norm(p=2, dim=(-2, -1), keepdim=True)
    V = torch.lerp(V, (Uc * Uc).mean(dim=-1, keepdim=True), 1 - muon_beta2)
    Un = Uc / (V.sqrt() + 1e-8)
    norm_new = Un.norm(p=2, dim=(-2, -1), keepdim=True).clamp(min=1e-8)
    return Un * (norm_u / norm_new), V
