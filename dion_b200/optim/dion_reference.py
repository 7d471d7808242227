"""Paper-faithful, unbatched Dion (reference: dion/dion_reference.py:64-984).

One parameter at a time, every rank of a sharding group performing the small factorizations
redundantly.  Compared with :class:`dion_b200.optim.dion.Dion` it supports several power
iterations per step and three orthogonalization methods: ``"qr"`` (Householder),
``"cqr"`` (Cholesky-QR, falling back to the randomized variant when the Cholesky factorization
fails, and replaced by it during the first ``cqr_warmup_steps`` steps) and ``"rcqr"``.
It shares parameter-layout detection, state layout and seeding with the batched class and, like
it, issues its collectives explicitly on local shards.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor

from ..ops import foreach as F
from ..ops import lowrank as LR
from ..parallel import collectives as C
from ..utils.tensors import to_local
from .dion import Dion as _BatchedDion
from .dion import DionMixedPrecisionConfig  # noqa: F401  (re-exported)


def _sum_over(t: Tensor, pg: Optional[ProcessGroup]) -> Tensor:
    if pg is not None and dist.get_world_size(pg) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=pg)
    return t


def orthogonalize_rows_sharded(P: Tensor, qr_method: str, oversample: float,
                               inner_pg: Optional[ProcessGroup],
                               generator: Optional[torch.Generator]) -> Tensor:
    """Orthonormalize the columns of ``P`` (``[m_loc, r]``, rows sharded over ``inner_pg`` or
    whole when it is None) with the requested method; every rank computes the small factors."""
    dtype = P.dtype
    W = dist.get_world_size(inner_pg) if inner_pg is not None else 1
    m_loc, r = P.shape
    m = m_loc * W
    P32 = P.to(torch.float32)
    if qr_method == "cqr":
        R, info = torch.linalg.cholesky_ex(_sum_over(P32.T @ P32, inner_pg), upper=True)
        if int(info) == 0:
            return LR.right_solve_upper(R, P32).to(dtype)
        qr_method = "rcqr"
    if qr_method == "qr" or m <= r:
        if W > 1:
            full, _ = C.all_gather_dim0(P32, inner_pg)
            rank = dist.get_rank(inner_pg)
            return torch.linalg.qr(full)[0][rank * m_loc:(rank + 1) * m_loc].to(dtype)
        return torch.linalg.qr(P32)[0].to(dtype)
    k = LR.sketch_rows(r, oversample)
    S = LR.random_sketch(1, k, m_loc, dtype, P.device, generator)[0]
    R1 = LR.qr_r_factor(_sum_over((S @ P).to(torch.float32), inner_pg))
    P32 = LR.right_solve_upper(R1, P32)
    R2 = LR.cholesky_upper(_sum_over(P32.T @ P32, inner_pg))
    return LR.right_solve_upper(R2, P32).to(dtype)


class Dion(_BatchedDion):
    """Unbatched Dion.  Arguments as :class:`dion_b200.optim.dion.Dion`, with ``power_iters >= 1``
    and ``qr_method`` in ``{"qr", "cqr", "rcqr"}``."""

    def __init__(
        self,
        params,
        replicate_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        outer_shard_mesh: Optional[DeviceMesh] = None,
        inner_shard_mesh: Optional[DeviceMesh] = None,
        replicate_mesh_grad_sync: bool = True,
        rank_fraction: float = 1.0,
        rank_multiple_of: int = 1,
        lr: float = 0.01,
        mu: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: float = 0.01,
        epsilon: float = 1e-8,
        power_iters: int = 1,
        qr_method: str = "rcqr",
        cqr_warmup_steps: int = 150,
        rcqr_oversample: float = 1.25,
        mixed_precision_config: Optional[DionMixedPrecisionConfig] = None,
    ):
        if power_iters <= 0:
            raise ValueError(f"Invalid power iterations: {power_iters}")
        if qr_method not in ("qr", "cqr", "rcqr"):
            raise ValueError(f"Unknown QR method: {qr_method}")
        super().__init__(
            params, replicate_mesh=replicate_mesh, outer_shard_mesh=outer_shard_mesh,
            inner_shard_mesh=inner_shard_mesh, replicate_mesh_grad_sync=replicate_mesh_grad_sync,
            rank_fraction=rank_fraction, rank_multiple_of=rank_multiple_of, lr=lr, mu=mu,
            betas=betas, weight_decay=weight_decay, epsilon=epsilon, power_iters=1,
            qr_method="rcqr", cqr_warmup_steps=cqr_warmup_steps, rcqr_oversample=rcqr_oversample,
            mixed_precision_config=mixed_precision_config)
        self._power_iters = power_iters
        self._qr_method = qr_method
        self._cqr_warmup_steps = cqr_warmup_steps

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        rep = self._replicate_mesh
        sync = self._replicate_mesh_grad_sync and rep is not None
        pid = 0
        for group in self.param_groups:
            algo = group["algorithm"]
            group["step"] += 1
            step = group["step"]
            for param in group["params"]:
                pid += 1
                if param.grad is None:
                    continue
                state = self._get_or_initialize_state(param, group)
                grad = to_local(param.grad)
                if algo == "dion":
                    cfg = self._get_dion_param_config(param)
                    compressed = sync and cfg.compressed_all_reduce
                    if sync and not compressed:
                        C.all_reduce_(grad, rep, op="avg")
                    method = self._qr_method
                    if method == "cqr" and step <= self._cqr_warmup_steps:
                        method = "rcqr"
                    self._update_one(param, grad, state, cfg, group, method, compressed, pid)
                elif algo == "adamw":
                    if sync:
                        C.all_reduce_(grad, rep, op="avg")
                    F.adamw([to_local(param)], [grad], [to_local(state["momentum"])],
                            [to_local(state["variance"])], group["lr"], group["beta1"],
                            group["beta2"], group["weight_decay"], group["epsilon"], step=step)
                elif algo == "lion":
                    if sync:
                        C.all_reduce_(grad, rep, op="avg")
                    F.lion([to_local(param)], [grad], [to_local(state["momentum"])], group["lr"],
                           group["beta1"], group["beta2"], group["weight_decay"])
                else:
                    raise ValueError(f"Unknown algorithm: {algo}")
        return loss

    def _update_one(self, param, G, state, cfg, group, qr_method, compressed, pid) -> None:
        lr, mu, wd, eps = group["lr"], group["mu"], group["weight_decay"], group["epsilon"]
        mesh = param.device_mesh if isinstance(param, DTensor) else None
        outer_pg = mesh.get_group(cfg.outer_shard_mesh_dim) \
            if mesh is not None and cfg.outer_shard_mesh_dim is not None else None
        inner_pg = mesh.get_group(cfg.inner_shard_mesh_dim) \
            if mesh is not None and cfg.inner_shard_mesh_dim is not None else None
        rep = self._replicate_mesh
        X, M, Qs = to_local(param), to_local(state["momentum"]), to_local(state["Q"])
        Q = C.all_gather_last_dim(Qs, inner_pg).to(M.dtype) if inner_pg is not None else Qs.to(M.dtype)
        Q_init = Q
        M.add_(G.to(M.dtype))
        Mt = M.T if cfg.is_transposed else M
        i_rank = dist.get_rank(inner_pg) if inner_pg is not None else 0
        gen = self._generator(X.device, group["step"], pid, i_rank)
        for _ in range(self._power_iters):
            P = _sum_over(Mt @ Q, outer_pg)
            if compressed:
                C.all_reduce_(P, rep, op="avg")
            P = orthogonalize_rows_sharded(P, qr_method, group["oversample"], inner_pg, gen)
            Q = _sum_over(Mt.T @ P, inner_pg)
            if compressed:
                C.all_reduce_(Q, rep, op="avg")
        R = Q
        P3, R3 = LR.fix_all_zero_or_nan(P[None], R[None], Q_init[None], Mt[None])
        P, R = P3[0], R3[0]
        M.add_((R @ P.T) if cfg.is_transposed else (P @ R.T), alpha=-(1 - mu))
        ss = LR.local_column_sum_sq(R)
        if outer_pg is not None:
            _sum_over(ss, outer_pg)
        Q_new = (R.to(torch.float32) / (ss.sqrt() + eps)).to(P.dtype)
        fan_out, fan_in = param.shape
        X.mul_(1 - lr * wd)
        upd = (Q_new @ P.T) if cfg.is_transposed else (P @ Q_new.T)
        X.add_(upd.to(X.dtype), alpha=-math.sqrt(fan_out / fan_in) * lr)
        if inner_pg is not None:
            W = dist.get_world_size(inner_pg)
            c = Q_new.size(-1) // W
            Q_new = Q_new[:, i_rank * c:(i_rank + 1) * c]
        Qs.copy_(Q_new.to(Qs.dtype))
