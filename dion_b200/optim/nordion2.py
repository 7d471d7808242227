"""NorDion2 (alias Dion3): Dion2's row selection with NorMuon's per-row normalization of the
orthogonalized sub-matrix (reference: dion/nordion2.py:26-497).  Selection is always along rows
and the error-feedback decay equals the momentum factor ``mu``.
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
from ..ops.select import _as_matrices, dion2_select
from ..parallel.async_runtime import AsyncTask
from ..parallel.megabatch import MegabatchPlan
from ..utils.tensors import group_by_shape, to_local
from .dion2 import _validate_dion2, make_select_and_orthogonalize, selection_count
from .muon import _validate_common, global_comm_size
from .normuon import _matrix_views, normuon_normalization_stacked
from .ortho_base import DistributedOrthoBase, lr_ratio


class NorDion2(DistributedOrthoBase):
    """Distributed NorDion2.  Arguments: see :class:`Dion2` (``fraction``, ``selection_scope``)
    and :class:`NorMuon` (``mu``, ``muon_beta2``).  State per matrix: ``momentum`` and
    ``variance_neuron``.  Last-dimension shards and ``split_sizes`` are not supported."""

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        lr: float = 0.01,
        fraction: float = 0.25,
        mu: float = 0.95,
        muon_beta2: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: Union[float, Tensor] = 0.01,
        epsilon: float = 1e-8,
        adjust_lr: Optional[str] = "spectral_norm",
        flatten: bool = False,
        use_triton: bool = False,
        use_polar_express: bool = True,
        use_gram_newton_schulz: bool = False,
        newton_schulz_func: Optional[Callable] = None,
        triton_post_ortho: bool = False,
        selection_scope: str = "local",
    ):
        _validate_common(lr, mu, betas, adjust_lr)
        _validate_dion2(fraction, selection_scope)
        if muon_beta2 < 0.0:
            raise ValueError(f"Invalid muon_beta2: {muon_beta2}")
        defaults = dict(
            lr=lr, fraction=float(fraction), mu=mu, muon_beta2=muon_beta2, beta1=betas[0],
            beta2=betas[1], weight_decay=weight_decay, epsilon=epsilon, flatten=flatten,
            adjust_lr=adjust_lr, algorithm="nordion2", step=0, selection_scope=selection_scope)
        super().__init__(
            params, distributed_mesh, "nordion2", defaults,
            use_gram_newton_schulz=use_gram_newton_schulz, use_triton=use_triton,
            use_polar_express=use_polar_express, newton_schulz_func=newton_schulz_func)
        self._triton_post_ortho = triton_post_ortho

    def _get_or_initialize_state(self, param: Tensor, algo: str) -> dict:
        state = super()._get_or_initialize_state(param, algo)
        if algo == self._algo_name and "variance_neuron" not in state:
            state["variance_neuron"] = torch.zeros_like(param[..., 0:1])
        return state

    def _get_shard_info(self, param: Tensor, group: dict):
        info = super()._get_shard_info(param, group)
        if info[1] and info[2] == param.ndim - 1:
            raise NotImplementedError(
                "NorDion2 currently does not support parameters sharded along the last dimension. "
                "Please avoid shards at dim -1.")
        return info

    def _create_ortho_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            assert all(p.ndim >= 2 for p in group["params"]), \
                "NorDion2 optimizer only supports matrix parameters."
            with_grad = [p for p in group["params"] if p.grad is not None]
            if not with_grad:
                continue
            num_heads = self._resolve_num_heads(group)
            if group.get("split_sizes") is not None:
                raise NotImplementedError(
                    "split_sizes is currently supported only by Muon and NorMuon.")
            for params in group_by_shape(with_grad).values():
                grads = [p.grad for p in params]
                states = [self._get_or_initialize_state(p, self._algo_name) for p in params]
                moms = [s["momentum"] for s in states]
                var = [s["variance_neuron"] for s in states]
                pg, shard_dim = self._bucket_layout(group, params, num_heads)
                if num_heads is not None:
                    params, grads, moms, var = self._prepare_head_split(
                        num_heads, params, grads, moms, var)
                yield AsyncTask(nordion2_update_megabatch_async(
                    X=params, G=grads, M=moms, V=var, lr=group["lr"],
                    fraction=group["fraction"], momentum=group["mu"],
                    muon_beta2=group["muon_beta2"], weight_decay=group["weight_decay"],
                    epsilon=group["epsilon"], flatten=group["flatten"],
                    adjust_lr=group["adjust_lr"], device_rank=self._device_rank,
                    world_size=self._world_size, shard_dim=shard_dim, process_group=pg,
                    newton_schulz_func=self._newton_schulz_func, arena=self._arena,
                    fused_cache=self._fused_exchanges,
                    selection_scope=group["selection_scope"]))


def nordion2_update_megabatch_async(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    V: List[Tensor],
    lr,
    fraction: float,
    momentum,
    muon_beta2,
    weight_decay,
    epsilon,
    flatten: bool,
    adjust_lr: Optional[str],
    device_rank: int,
    world_size: int,
    shard_dim: Optional[int] = None,
    process_group: Optional[ProcessGroup] = None,
    newton_schulz_func: Optional[Callable] = None,
    triton_post_ortho: bool = False,
    selection_scope: str = "local",
    arena=None,
    fused_cache=None,
) -> Generator[None, None, None]:
    assert len(X) == len(G) == len(M) == len(V)
    select_dim = -2
    comm_dim = select_dim if shard_dim is not None else None
    global_dim = global_comm_size(X[0], comm_dim)
    Xl, Gl, Ml, Vl = to_local(X), to_local(G), to_local(M), to_local(V)
    ratio = lr_ratio(adjust_lr, X[0].shape, flatten)
    N = len(X)

    if selection_scope == "global" and comm_dim is not None:
        plan = MegabatchPlan(Ml[0].shape, N, Ml[0].device, comm_dim, device_rank, world_size,
                             process_group, global_comm_dim_size=global_dim, arena=arena)
        F.muon_pre(Gl, Ml, 0.0, False, out=plan.input_views(), add_only=True)
        select_ns = make_select_and_orthogonalize(
            newton_schulz_func, fraction, select_dim, global_select_size=global_dim)
        U = yield from plan.run(select_ns, flatten, epsilon)
        nordion2_post_orthogonalize_masked(Xl, Ml, Vl, list(U.unbind(0)), lr, ratio,
                                           weight_decay, float(momentum), float(muon_beta2))
        return

    k = selection_count(fraction, comm_dim, global_dim, world_size)
    num_select = Ml[0].size(select_dim)
    if k is None:
        k = max(1, int(math.ceil(fraction * num_select)))
    k_topk = min(k, num_select)
    if fused_cache is not None and FX.eligible(Ml[0].shape, comm_dim, global_dim, world_size,
                                               process_group, newton_schulz_func, flatten, None):
        # Exchange carried by the kernels (see Dion2 and parallel/fused_exchange.py).
        fx = FX.get_exchange(fused_cache, (id(X[0]), N, k, Ml[0].shape[1]), process_group, N, k,
                             Ml[0].shape[1], Ml[0].device)
        fx.begin()
        outs, sums = fx.push_targets()
        _, idx, maps = dion2_select(Gl, Ml, k, select_dim, float(momentum),
                                    out_addresses=[o.address for o in outs],
                                    sumsq_addresses=sums)
        fx.publish()
        NS.iterate_with_exchange(fx.input_matrix(), newton_schulz_func, epsilon, fx)
        fx.finish()
        fx.wait_results()
        U3 = fx.result_stack()
        idx_list = list(idx.unbind(0))
        rinv, n_u2, n_new2 = F.normuon_rowstats(U3, _matrix_views(Vl, num_select),
                                                float(muon_beta2), vmaps=idx_list,
                                                guard=fx.status)
        F.dion2_post(Xl, list(U3.unbind(0)), idx_list, list(maps.unbind(0)), lr, weight_decay,
                     ratio, select_dim, rowscale=list(rinv.unbind(0)), normU2=n_u2,
                     normNew2=n_new2, wait=fx.result_wait())
        fx.release()
        yield
        return
    U_sel, idx, maps = dion2_select(Gl, Ml, k_topk, select_dim, float(momentum))
    sel_shape = tuple(Ml[0].shape[:-2]) + tuple(U_sel.shape[-2:])
    plan = MegabatchPlan(sel_shape, N, Ml[0].device, comm_dim, device_rank, world_size,
                         process_group, global_comm_dim_size=global_dim,
                         local_comm_size=k if comm_dim is not None else None, arena=arena)
    plan.load(U_sel.reshape((N,) + sel_shape).unbind(0))
    U = yield from plan.run(newton_schulz_func, flatten, epsilon)
    if num_select == 0:
        return
    U3 = U.reshape((-1,) + tuple(U.shape[-2:]))
    if not U3.is_contiguous():
        U3 = U3.contiguous()
    idx_list = list(idx.unbind(0))
    rinv, n_u2, n_new2 = F.normuon_rowstats(U3, _matrix_views(Vl, num_select),
                                            float(muon_beta2), vmaps=idx_list)
    F.dion2_post(_as_matrices(Xl), list(U3.unbind(0)), idx_list,
                 list(maps.unbind(0)) if maps is not None else None,
                 lr, weight_decay, ratio, select_dim,
                 rowscale=list(rinv.unbind(0)), normU2=n_u2, normNew2=n_new2)


def nordion2_post_orthogonalize_masked(
    X: List[Tensor], M: List[Tensor], V: List[Tensor], U: List[Tensor], lr, ratio: float,
    weight_decay, ef_decay: float, muon_beta2: float,
) -> None:
    """Global-scope post step.  ``U`` is full-size and zero off the selected rows.  Normalizing
    the full matrix equals normalizing the selected sub-matrix (zero rows contribute nothing);
    the variance buffer is written back only on selected rows."""
    torch._foreach_mul_(X, 1 - lr * weight_decay)
    step = lr * ratio
    for x, m, v, u in zip(X, M, V, U):
        sel = u.to(torch.float32).abs().sum(dim=-1, keepdim=True) > 0
        m.mul_(torch.where(sel, ef_decay, 1.0).to(m.dtype))
        u_hat, v_new = normuon_normalization_stacked(u, v.to(torch.float32), muon_beta2)
        v.copy_(torch.where(sel, v_new.to(v.dtype), v))
        x.sub_((step * u_hat).to(x.dtype))


def nordion2_normalize_selected_stacked(U: Tensor, V_full: Tensor, indices: Tensor, muon_beta2):
    """Functional form: normalize the selected rows ``U [N,k,cols]`` against the rows
    ``indices [N,k]`` of ``V_full [N,rows,1]``; returns ``(U_hat, V_full_new)``
    (reference: dion/nordion2.py:430-447)."""
    idx = indices.unsqueeze(-1)
    v_sel = torch.gather(V_full, -2, idx).to(torch.float32)
    u_hat, v_new = normuon_normalization_stacked(U, v_sel, muon_beta2)
    return u_hat, V_full.scatter(-2, idx, v_new.to(V_full.dtype))
