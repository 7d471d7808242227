"""Dion: low-rank orthonormal updates by one step of power iteration with error feedback
(https://arxiv.org/abs/2504.05295; reference: dion/dion.py:57-1599).

Per matrix (in the orientation ``Mt`` that puts the sharded-for-orthogonalization dimension on
the rows): ``M += G``; ``P = Mt Q``; orthonormalize ``P`` (randomized Cholesky-QR);
``R = Mt^T P``; error feedback ``Mt -= (1-mu) P R^T``; ``Q <- R / ||R||_col``;
``Xt <- (1 - lr*wd) Xt - lr*sqrt(fan_out/fan_in) P Q^T``.

Three layouts, each processing a batch of ``B`` same-shape matrices so that every rank of the
batching group factorizes one matrix:

* ``ddp``      plain tensors replicated over a process group (``B`` = its size);
* ``fsdp``     DTensors sharded over ``outer_shard_mesh`` (``B`` = its size): the partial products
               are reduce-scattered over the batch dimension;
* ``fsdp_tp``  additionally sharded over ``inner_shard_mesh`` (``B`` = its size): ``P`` stays
               row-sharded and is orthonormalized with a distributed Cholesky-QR.

With ``replicate_mesh_grad_sync`` the optimizer averages over the data-parallel replicas itself,
and when the factors are smaller than the matrix (``(m+n) r < m n``) it averages the low-rank
``P`` and ``R`` instead of the gradient ("compressed" synchronization).  Unlike the reference,
which leans on DTensor's implicit redistribution, every collective here is an explicit call on
local shards (``parallel/collectives.py``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from itertools import chain
from typing import Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor, Replicate, Shard
from torch.optim.optimizer import Optimizer, ParamsT

try:  # pragma: no cover - depends on the torch build
    from torch.distributed.tensor.placement_types import _StridedShard
except ImportError:  # pragma: no cover
    _StridedShard = None

from ..ops import foreach as F
from ..ops import lowrank as LR
from ..parallel import collectives as C
from ..parallel import lowrank_sync as LS
from ..parallel.async_runtime import AsyncRuntime, AsyncTask
from ..utils.tensors import create_param_batches, group_by_shape, to_local
from .status import DeviceStatusMixin


@dataclass
class DionMixedPrecisionConfig:
    """dtypes of the optimizer state; ``None`` keeps the parameter's dtype."""

    momentum_dtype: Optional[torch.dtype] = None
    Q_dtype: Optional[torch.dtype] = None
    variance_dtype: Optional[torch.dtype] = None


@dataclass
class _DionParamConfig:
    """How one parameter is sharded and oriented."""

    outer_shard_tensor_dim: Optional[int] = None
    inner_shard_tensor_dim: Optional[int] = None
    outer_shard_mesh_dim: Optional[int] = None
    inner_shard_mesh_dim: Optional[int] = None
    is_transposed: bool = False
    compressed_all_reduce: bool = False
    Q_sharded_placements: Optional[tuple] = None
    Q_inner_unsharded_placements: Optional[tuple] = None


def _mesh_check(name: str, mesh, others) -> None:
    if mesh is None:
        return
    if not isinstance(mesh, DeviceMesh):
        raise TypeError(f"{name} shard mesh must be a DeviceMesh, but got {type(mesh)}.")
    if mesh.ndim != 1:
        raise ValueError(
            f"{name} shard mesh must be 1D, but got {mesh.ndim}D. Try using a 1D sub-mesh.")
    for oname, other in others:
        if other is not None and mesh == other:
            raise ValueError(f"{name} shard mesh must be different from {oname}.")


class Dion(DeviceStatusMixin, Optimizer):
    """Distributed Dion.

    Args:
        params: parameters or param groups (``algorithm``: ``"dion"`` default, ``"adamw"``,
            ``"lion"``).
        replicate_mesh: DeviceMesh (HSDP replicate dimension) or ProcessGroup (DDP).
        outer_shard_mesh: 1-D DeviceMesh the parameters are sharded over but replicated during
            orthogonalization (FSDP).
        inner_shard_mesh: 1-D DeviceMesh that stays sharded during orthogonalization (TP).
        replicate_mesh_grad_sync: the optimizer performs the data-parallel synchronization
            (compressed where possible) instead of expecting averaged gradients.
        rank_fraction, rank_multiple_of: ``r = min(mult*ceil(frac*min(m,n)/mult), m, n)``.
        lr, mu, betas, weight_decay, epsilon: hyper-parameters.
        power_iters, qr_method: only ``1`` and ``"rcqr"`` are supported by this class.
        rcqr_oversample: sketch oversampling factor.
        mixed_precision_config: state dtypes.
    Parameters are either all DTensors (with DeviceMeshes) or all plain tensors (with a
    ProcessGroup); shards are assumed to be evenly sized.
    """

    def __init__(
        self,
        params: ParamsT,
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
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if mu < 0.0:
            raise ValueError(f"Invalid momentum factor (mu): {mu}")
        if len(betas) != 2 or betas[0] < 0.0 or betas[1] < 0.0:
            raise ValueError(f"Invalid betas: {betas}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        if rank_fraction <= 0 or rank_fraction > 1:
            raise ValueError(f"Invalid rank fraction: {rank_fraction}")
        if rank_multiple_of <= 0:
            raise ValueError(f"Invalid rank multiple of: {rank_multiple_of}")
        if power_iters != 1:
            raise ValueError("Async Dion only supports power_iters=1")
        if qr_method != "rcqr":
            raise ValueError("Async Dion only supports qr_method='rcqr'")
        if replicate_mesh is not None and not isinstance(replicate_mesh, (DeviceMesh, ProcessGroup)):
            raise TypeError(
                f"Replicate mesh must be a DeviceMesh or ProcessGroup, but got {type(replicate_mesh)}.")
        _mesh_check("Outer", outer_shard_mesh, [("replicate mesh", replicate_mesh)])
        _mesh_check("Inner", inner_shard_mesh,
                    [("replicate mesh", replicate_mesh), ("outer shard mesh", outer_shard_mesh)])

        defaults = dict(
            rank_fraction=rank_fraction, rank_multiple_of=rank_multiple_of, lr=lr, mu=mu,
            beta1=betas[0], beta2=betas[1], weight_decay=weight_decay, epsilon=epsilon,
            oversample=rcqr_oversample, algorithm="dion", step=0)
        super().__init__(params, defaults)

        self._param_config: Dict[Tensor, _DionParamConfig] = {}  # never checkpointed
        self._replicate_mesh = replicate_mesh
        self._outer_shard_mesh = outer_shard_mesh
        self._inner_shard_mesh = inner_shard_mesh
        self._replicate_mesh_grad_sync = replicate_mesh_grad_sync
        self._replicate_world_size = C.group_size(replicate_mesh)
        self._outer_shard_ranks = (dist.get_process_group_ranks(outer_shard_mesh.get_group())
                                   if outer_shard_mesh is not None else None)
        self._inner_shard_ranks = (dist.get_process_group_ranks(inner_shard_mesh.get_group())
                                   if inner_shard_mesh is not None else None)
        self._mixed_precision_config = mixed_precision_config or DionMixedPrecisionConfig()
        # Sketches and Q initialisation must agree across replicas: all randomness is drawn
        # from generators seeded by (base seed, step, task, shard coordinates).
        self._base_seed = self._agree_on_seed()
        self._generators: Dict[torch.device, torch.Generator] = {}
        self._q_counter = 0
        self._momentum_stacks: Dict[tuple, Tensor] = {}
        self._side_streams: Dict[torch.device, list] = {}
        self._streams_to_join: set = set()
        self._lowrank_sync: Dict[tuple, tuple] = {}

    # ------------------------------------------------------------------ randomness ----------
    def _agree_on_seed(self) -> int:
        seed = torch.initial_seed() % (1 << 31)
        if dist.is_available() and dist.is_initialized() and any(
                m is not None for m in (self._replicate_mesh, self._outer_shard_mesh,
                                        self._inner_shard_mesh)):
            dev = torch.device("cuda", torch.cuda.current_device()) \
                if dist.get_backend() == "nccl" else torch.device("cpu")
            t = torch.tensor([seed], dtype=torch.int64, device=dev)
            dist.broadcast(t, src=0)
            seed = int(t.item())
        return seed

    def _generator(self, device: torch.device, *coords: int) -> torch.Generator:
        g = self._generators.get(device)
        if g is None:
            g = torch.Generator(device=device)
            self._generators[device] = g
        h = self._base_seed
        for c in coords:
            h = (h * 1000003 + int(c) + 12345) % ((1 << 61) - 1)
        g.manual_seed(h)
        return g

    # ------------------------------------------------------------------ step ----------------
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._poll_device_status()
        groups = {"dion": [], "lion": [], "adamw": []}
        for group in self.param_groups:
            group["step"] += 1
            algo = group["algorithm"]
            if algo not in groups:
                raise ValueError(f"Unknown algorithm: {algo}")
            groups[algo].append(group)
        tasks = chain(self._create_dion_tasks(groups["dion"]),
                      self._create_lion_tasks(groups["lion"]),
                      self._create_adamw_tasks(groups["adamw"]))
        AsyncRuntime(tasks, max_concurrent_tasks=3).run()
        for side in self._streams_to_join:   # batches ran on side streams (see _on_side_stream)
            torch.cuda.current_stream(side.device).wait_stream(side)
        self._streams_to_join.clear()
        self._snapshot_device_status()
        return loss

    @torch.no_grad()
    def synchronize_for_checkpoint(self):
        """Average every state tensor over the replicate mesh.  Compressed synchronization lets
        the momentum drift apart between replicas; call this before saving a checkpoint.  No-op
        without a replicate mesh or when the optimizer does not own the gradient sync."""
        self.check_device_status()
        if self._replicate_mesh is None or not self._replicate_mesh_grad_sync:
            return
        tensors = [to_local(v) for st in self.state.values() for v in st.values()
                   if isinstance(v, Tensor)]
        C.all_reduce_(tensors, self._replicate_mesh, op="avg")

    # ------------------------------------------------------------------ tasks ---------------
    def _create_dion_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        task_id = 0
        for group in param_groups:
            with_grad = [p for p in group["params"] if p.grad is not None]
            if not with_grad:
                continue
            for kind, plist in self._split_params_by_sharding(with_grad).items():
                if not plist:
                    continue
                if kind == "inner_sharded":
                    batches = create_param_batches(plist, self._inner_shard_mesh.size())
                elif kind == "outer_sharded":
                    batches = create_param_batches(plist, self._outer_shard_mesh.size())
                else:
                    batches = self._replicated_batches(plist)
                for params in batches:
                    if kind == "inner_sharded":
                        batch = self._inner_shard_mesh.size()
                    elif kind == "outer_sharded":
                        batch = self._outer_shard_mesh.size()
                    else:
                        W = self._replicate_world_size
                        batch = W * ((len(params) + W - 1) // W)
                    states = [self._get_or_initialize_state(p, group) for p in params]
                    cfg = self._get_dion_param_config(params[0])
                    task_id += 1
                    update = self._dion_update(
                        kind, batch, params, [p.grad for p in params],
                        [s["momentum"] for s in states], [s["Q"] for s in states], cfg, group,
                        task_id)
                    yield AsyncTask(self._on_side_stream(update, task_id, to_local(params[0])))

    # Batches are independent of one another, and the factorization kernels of a batch (one CTA
    # per matrix, long dependent chains) leave most of the GPU idle when the batch is smaller
    # than the number of SMs.  Each batch therefore runs on one of a few side streams, so that
    # the kernels of different batches share the GPU; the side streams start after the work
    # already queued on the caller's stream and are joined before step() returns.
    _SIDE_STREAMS = 3

    def _on_side_stream(self, gen, task_id: int, sample: Tensor):
        if not sample.is_cuda or torch.cuda.is_current_stream_capturing():
            yield from gen
            return
        dev = sample.device
        pool = self._side_streams.get(dev)
        if pool is None:
            pool = self._side_streams[dev] = [torch.cuda.Stream(device=dev)
                                              for _ in range(self._SIDE_STREAMS)]
        side = pool[task_id % len(pool)]
        main = torch.cuda.current_stream(dev)
        side.wait_stream(main)
        self._streams_to_join.add(side)
        while True:
            with torch.cuda.stream(side):
                try:
                    next(gen)
                except StopIteration:
                    return
            yield

    # Stacked copies of the momentum of one batch are kept below this many bytes.
    _BATCH_BYTES = 2 << 30

    def _replicated_batches(self, plist: List[Tensor]) -> Iterable[List[Tensor]]:
        """Unsharded parameters: every rank orthogonalizes ``L`` matrices of a batch of
        ``world * L`` instead of one of ``world`` (the reference's layout, dion/dion.py:419-424),
        so that the batched kernels see all same-shape matrices at once; ``L`` is bounded by the
        size of the stacked momentum."""
        W = self._replicate_world_size
        for bucket in group_by_shape(plist).values():
            nbytes = max(1, bucket[0].numel() * 4)
            per_rank = max(1, min((len(bucket) + W - 1) // W, self._BATCH_BYTES // (nbytes * W)))
            size = W * per_rank
            for start in range(0, len(bucket), size):
                yield bucket[start:start + size]

    def _scalar_lists(self, group, keys):
        params = [p for p in group["params"] if p.grad is not None]
        states = [self._get_or_initialize_state(p, group) for p in params]
        return params, [p.grad for p in params], [[s[k] for s in states] for k in keys]

    def _create_lion_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            params, grads, (moms,) = self._scalar_lists(group, ["momentum"])
            if params:
                yield AsyncTask(self._scalar_update("lion", group, params, grads, moms, None))

    def _create_adamw_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        for group in param_groups:
            params, grads, (moms, var) = self._scalar_lists(group, ["momentum", "variance"])
            if params:
                yield AsyncTask(self._scalar_update("adamw", group, params, grads, moms, var))

    def _scalar_update(self, algo, group, params, grads, moms, var):
        X, G, M = to_local(params), to_local(grads), to_local(moms)
        if self._replicate_mesh_grad_sync and self._replicate_mesh is not None:
            work = C.all_reduce_(G, self._replicate_mesh, op="avg", async_op=True)
            yield
            work.wait()
        if algo == "adamw":
            F.adamw(X, G, M, to_local(var), group["lr"], group["beta1"], group["beta2"],
                    group["weight_decay"], group["epsilon"], step=group["step"])
        else:
            F.lion(X, G, M, group["lr"], group["beta1"], group["beta2"], group["weight_decay"])

    # ------------------------------------------------------------------ state ---------------
    def _get_or_initialize_state(self, param: Tensor, group: dict) -> dict:
        state = self.state[param]
        if state:
            return state
        algo = group["algorithm"]
        mp = self._mixed_precision_config
        if algo == "dion":
            self._init_opt_state_dion(param, state, group["rank_fraction"],
                                      group["rank_multiple_of"])
        elif algo == "adamw":
            state["momentum"] = torch.zeros_like(param, dtype=mp.momentum_dtype)
            state["variance"] = torch.zeros_like(param, dtype=mp.variance_dtype)
        elif algo in ("lion", "clion"):
            state["momentum"] = torch.zeros_like(param, dtype=mp.momentum_dtype)
        else:
            raise ValueError(f"Unknown algorithm: {algo}")
        return state

    def _init_opt_state_dion(self, param: Tensor, state: dict, rank_fraction: float,
                             rank_multiple_of: int) -> None:
        if param.ndim != 2:
            raise ValueError(
                f"Expected Dion parameters to be 2D matrix, but got {param.ndim}D. "
                f"For scalar parameters, set 'algorithm' to 'lion' or 'adamw' when creating param group.")
        cfg = self._get_dion_param_config(param)
        mp = self._mixed_precision_config
        state["momentum"] = torch.zeros_like(param, dtype=mp.momentum_dtype)
        m, n = param.shape
        r = rank_multiple_of * math.ceil(rank_fraction * min(m, n) / rank_multiple_of)
        r = min(r, m, n)
        if rank_fraction < 1 and (m + n) * r < m * n:
            cfg.compressed_all_reduce = True
        q_rows = m if cfg.is_transposed else n
        q_dtype = mp.Q_dtype if mp.Q_dtype is not None else param.dtype
        self._q_counter += 1
        if isinstance(param, DTensor):
            mesh = param.device_mesh
            placements = [Replicate() for _ in range(mesh.ndim)]
            rows_loc, cols_loc = q_rows, r
            o_rank = i_rank = 0
            if cfg.outer_shard_mesh_dim is not None:
                placements[cfg.outer_shard_mesh_dim] = Shard(0)
                rows_loc = q_rows // mesh.size(cfg.outer_shard_mesh_dim)
                o_rank = mesh.get_local_rank(cfg.outer_shard_mesh_dim)
            if cfg.inner_shard_mesh_dim is not None:
                placements[cfg.inner_shard_mesh_dim] = Shard(1)
                cols_loc = r // mesh.size(cfg.inner_shard_mesh_dim)
                i_rank = mesh.get_local_rank(cfg.inner_shard_mesh_dim)
            cfg.Q_sharded_placements = tuple(placements)
            if cfg.inner_shard_mesh_dim is not None:
                unsh = list(placements)
                unsh[cfg.inner_shard_mesh_dim] = Replicate()
                cfg.Q_inner_unsharded_placements = tuple(unsh)
            dev = param.to_local().device
            gen = self._generator(dev, 7, self._q_counter, o_rank, i_rank)
            q_local = torch.randn((rows_loc, cols_loc), device=dev, dtype=torch.float32,
                                  generator=gen).to(q_dtype)
            state["Q"] = DTensor.from_local(q_local, device_mesh=mesh, placements=placements,
                                            run_check=False)
        else:
            Q = torch.randn((q_rows, r), device=param.device, dtype=q_dtype)
            C.broadcast_(Q, self._replicate_mesh, src=0)
            state["Q"] = Q

    def _get_dion_param_config(self, x: Tensor) -> _DionParamConfig:
        cfg = self._param_config.get(x)
        if cfg is not None:
            return cfg
        if x.ndim > 2:
            raise NotImplementedError(
                f"Tensors with more than 2 dimensions are not supported. Got {x.ndim}D tensor.")
        using_mesh = any(isinstance(m, DeviceMesh) for m in
                         (self._replicate_mesh, self._outer_shard_mesh, self._inner_shard_mesh))
        if using_mesh and not isinstance(x, DTensor):
            raise TypeError("When using DeviceMesh, all parameters must be DTensor.")
        if isinstance(self._replicate_mesh, ProcessGroup) and isinstance(x, DTensor):
            raise TypeError(
                "When using DTensor parameters, the data parallel group must be specified by a "
                "DeviceMesh instead of ProcessGroup.")
        cfg = _DionParamConfig()
        if x.ndim == 2:
            cfg.is_transposed = x.shape[0] < x.shape[1]
        if isinstance(x, DTensor) and x.ndim == 2:
            mesh = x.device_mesh
            taken: List[Optional[int]] = [None, None]
            for mesh_dim, pl in enumerate(x.placements):
                if _StridedShard is not None and isinstance(pl, _StridedShard):
                    raise NotImplementedError(
                        "StridedShard is not supported. Ensure that FSDP and TP shard different "
                        "dimensions of each matrix.")
                if not pl.is_shard():
                    continue
                if taken[pl.dim] is not None:
                    raise RuntimeError(f"Got double-sharded DTensor for tensor dimension {pl.dim}.")
                taken[pl.dim] = mesh_dim
                ranks = dist.get_process_group_ranks(mesh.get_group(mesh_dim))
                is_outer = ranks == self._outer_shard_ranks
                is_inner = ranks == self._inner_shard_ranks
                if is_outer and is_inner:
                    raise RuntimeError(
                        "Cannot have outer and inner sharding over the same process group.")
                if is_outer:
                    cfg.outer_shard_tensor_dim, cfg.outer_shard_mesh_dim = pl.dim, mesh_dim
                elif is_inner:
                    cfg.inner_shard_tensor_dim, cfg.inner_shard_mesh_dim = pl.dim, mesh_dim
                elif mesh.size(mesh_dim) > 1:
                    raise RuntimeError(
                        f"Got DTensor sharded on unrecognized {mesh_dim=}, which does not match "
                        f"outer_shard_mesh or inner_shard_mesh.")
            # The orthogonalized dimension has to be the inner-sharded one, the contracted
            # dimension the outer-sharded one.
            if cfg.inner_shard_tensor_dim == 0 or cfg.outer_shard_tensor_dim == 1:
                cfg.is_transposed = False
            if cfg.outer_shard_tensor_dim == 0 or cfg.inner_shard_tensor_dim == 1:
                cfg.is_transposed = True
        self._param_config[x] = cfg
        return cfg

    def _split_params_by_sharding(self, params: List[Tensor]) -> Dict[str, List[Tensor]]:
        out: Dict[str, List[Tensor]] = {"inner_sharded": [], "outer_sharded": [], "non_sharded": []}
        for p in params:
            cfg = self._get_dion_param_config(p)
            if cfg.inner_shard_mesh_dim is not None:
                out["inner_sharded"].append(p)
            elif cfg.outer_shard_mesh_dim is not None:
                out["outer_sharded"].append(p)
            else:
                out["non_sharded"].append(p)
        return out

    def _sync_workspaces(self, first_param: Tensor, pg: ProcessGroup, batch: int, M3: Tensor,
                         Qb: Tensor, transposed: bool):
        """(workspace for P, workspace for R or None) of one batch, created collectively on
        first use.  R needs one only where it is averaged over ``pg`` (unsharded parameters)."""
        key = (id(first_param), batch, id(pg))
        ws = self._lowrank_sync.get(key)
        if ws is None:
            W = dist.get_world_size(pg)
            rows_p = M3.size(2) if transposed else M3.size(1)
            rows_r = M3.size(1) if transposed else M3.size(2)
            r = Qb.size(-1)
            dev = M3.device
            wp = LS.FusedReduceGather(pg, batch // W, rows_p, r, dev)
            wr = LS.FusedReduceGather(pg, batch // W, rows_r, r, dev) \
                if self._split_kind(first_param) == "non_sharded" else None
            ws = self._lowrank_sync[key] = (wp, wr)
        return ws

    def _split_kind(self, p: Tensor) -> str:
        cfg = self._get_dion_param_config(p)
        if cfg.inner_shard_mesh_dim is not None:
            return "inner_sharded"
        return "outer_sharded" if cfg.outer_shard_mesh_dim is not None else "non_sharded"

    def _momentum_stack(self, params: List[Tensor], batch: int) -> Tensor:
        """``[batch, rows, cols]`` tensor whose first ``len(params)`` slices ARE the (local)
        momentum tensors of ``params``: on first use (and again after ``load_state_dict``, which
        replaces the state tensors) the momentum is moved into one allocation and the state
        entries are re-pointed at its slices.  Checkpoints are unaffected: ``state_dict()`` still
        holds one tensor per parameter."""
        states = [self.state[p] for p in params]
        local = to_local([st["momentum"] for st in states])
        key = (id(params[0]), len(params), batch)
        stack = self._momentum_stacks.get(key)
        if stack is not None and all(m.data_ptr() == stack[i].data_ptr()
                                     for i, m in enumerate(local)):
            return stack
        stack = torch.zeros((batch,) + tuple(local[0].shape), dtype=local[0].dtype,
                            device=local[0].device)
        for i, (st, m) in enumerate(zip(states, local)):
            stack[i].copy_(m)
            old = st["momentum"]
            if isinstance(old, DTensor):
                st["momentum"] = DTensor.from_local(stack[i], old.device_mesh, old.placements,
                                                    run_check=False, shape=old.shape,
                                                    stride=old.stride())
            else:
                st["momentum"] = stack[i]
        self._momentum_stacks[key] = stack
        return stack

    # ------------------------------------------------------------------ the update ----------
    def _dion_update(self, kind: str, batch: int, params, grads, moms, Qs,
                     cfg: _DionParamConfig, group: dict, task_id: int):
        """Generator performing one batched Dion update; yields while collectives fly."""
        lr, mu, wd = group["lr"], group["mu"], group["weight_decay"]
        eps, oversample, step = group["epsilon"], group["oversample"], group["step"]
        fan_out, fan_in = params[0].shape  # global shape
        mesh = params[0].device_mesh if isinstance(params[0], DTensor) else None
        outer_pg = mesh.get_group(cfg.outer_shard_mesh_dim) \
            if mesh is not None and cfg.outer_shard_mesh_dim is not None else None
        inner_pg = mesh.get_group(cfg.inner_shard_mesh_dim) \
            if mesh is not None and cfg.inner_shard_mesh_dim is not None else None
        rep = self._replicate_mesh
        sync = self._replicate_mesh_grad_sync and rep is not None
        compressed = sync and cfg.compressed_all_reduce

        X, G, Q = to_local(params), to_local(grads), to_local(Qs)
        n_real = len(X)
        # The momentum of the batch lives in one stack [batch, rows, cols] (slots past n_real are
        # inert zeros), so the batched kernels read it in place and nothing is copied per step.
        M3 = self._momentum_stack(params, batch)
        M = list(M3.unbind(0))
        for lst in (X, G, Q):  # pad with inert stand-ins up to the batch size
            lst.extend(torch.zeros_like(lst[0]) for _ in range(batch - n_real))
        dev = X[0].device
        tr = cfg.is_transposed

        if sync and not compressed:
            work = C.all_reduce_(G[:n_real], rep, op="avg", async_op=True)
            yield
            work.wait()
        m_sq = None   # per-matrix sum of squares of the new momentum ("is it all zero?")
        if G[0].is_cuda and G[0].dtype in (torch.float32, torch.bfloat16) \
                and M3.dtype in (torch.float32, torch.bfloat16):
            m_sq = torch.zeros(batch, dtype=torch.float32, device=dev)
            F.muon_pre(G[:n_real], M[:n_real], 0.0, False, add_only=True, out=False,
                       sumsq=m_sq)
        else:
            torch._foreach_add_(M[:n_real], [g.to(M3.dtype) for g in G[:n_real]])

        if kind == "inner_sharded" and inner_pg is not None:
            Q_full = [C.all_gather_last_dim(q, inner_pg) for q in Q]
        else:
            Q_full = Q
        Qb = torch.stack(Q_full).to(M3.dtype)
        # Reduce-scatter of P (and of R below) inside the GEMM epilogue over peer memory where
        # the group allows it (see parallel/lowrank_sync.py); otherwise product + collective.
        rep_pg = C.as_groups(rep)[0] if rep is not None else None
        sync_pg = rep_pg if (kind == "non_sharded" and compressed) else \
            (outer_pg if kind == "outer_sharded" else None)
        fx = None
        if sync_pg is not None and LR.lr_gemm_ok(M3, Qb) and LS.eligible(sync_pg, dev):
            fx = self._sync_workspaces(params[0], sync_pg, batch, M3, Qb, tr)

        if kind == "non_sharded":
            rank = C.group_rank(rep) if rep is not None else 0
            if fx is not None:
                fxP = fx[0]
                fxP.begin()
                LR.power_iteration_p(M3, Qb, tr, reduce_into=fxP.targets,
                                     alpha=1.0 / self._replicate_world_size)
                fxP.after_gemm()
                gen = self._generator(dev, step, task_id, rank)
                fxP.own().copy_(LR.orthogonalize(fxP.own(), oversample, generator=gen))
                P = fxP.gather()
            else:
                P = LR.power_iteration_p(M3, Qb, tr)  # [B, rows_loc, r]
                if compressed:
                    P1, work = C.reduce_scatter_dim0(P, rep_pg, op="avg", async_op=True)
                    yield
                    work.wait()
                else:
                    per_rank = batch // self._replicate_world_size
                    P1 = P[rank * per_rank:(rank + 1) * per_rank]
                gen = self._generator(dev, step, task_id, rank)
                P1 = LR.orthogonalize(P1, oversample, generator=gen)
                if rep is not None:
                    P, work = C.all_gather_dim0(P1, rep_pg, async_op=True)
                    yield
                    work.wait()
                else:
                    P = P1
        elif kind == "outer_sharded":
            o_rank = dist.get_rank(outer_pg)
            if fx is not None:
                fxP = fx[0]
                fxP.begin()
                LR.power_iteration_p(M3, Qb, tr, reduce_into=fxP.targets)  # partial sums
                fxP.after_gemm()
                P1 = fxP.own()
            else:
                P = LR.power_iteration_p(M3, Qb, tr)  # partial over the sharded outer mesh
                P1, work = C.reduce_scatter_dim0(P, outer_pg, op="sum", async_op=True)
                yield
                work.wait()
            if compressed:
                work = C.all_reduce_(P1, rep, op="avg", async_op=True)
                yield
                work.wait()
            gen = self._generator(dev, step, task_id, o_rank)
            P1 = LR.orthogonalize(P1, oversample, generator=gen)
            if fx is not None:
                fxP.own().copy_(P1)
                P = fxP.gather()
            else:
                P, work = C.all_gather_dim0(P1, outer_pg, async_op=True)
                yield
                work.wait()
        else:  # inner_sharded
            P = LR.power_iteration_p(M3, Qb, tr)
            if outer_pg is not None:
                work = C.all_reduce_(P, outer_pg, op="sum", async_op=True)
                yield
                work.wait()
            if compressed:
                work = C.all_reduce_(P, rep, op="avg", async_op=True)
                yield
                work.wait()
            i_rank = dist.get_rank(inner_pg)
            gen = self._generator(dev, step, task_id, i_rank)
            P = distributed_orthogonalize(P, oversample, inner_pg, generator=gen)

        if fx is not None and kind == "non_sharded":
            fxR = fx[1]     # average of R over the replicas, again inside the epilogue
            fxR.begin()
            LR.power_iteration_r(M3, P, tr, reduce_into=fxR.targets,
                                 alpha=1.0 / self._replicate_world_size)
            fxR.after_gemm()
            R = fxR.gather()
        else:
            R = LR.power_iteration_r(M3, P, tr)  # [B, cols_loc, r]
            if kind == "inner_sharded":
                work = C.all_reduce_(R, inner_pg, op="sum", async_op=True)
                yield
                work.wait()
            if compressed:
                work = C.all_reduce_(R, rep, op="avg", async_op=True)
                yield
                work.wait()

        # Clean-up of the factors, column normalization and the write-back of Q: two fused
        # launches plus one where the kernels apply, PyTorch passes otherwise.
        fused_tail = (m_sq is not None and P.is_cuda and P.dtype == R.dtype == Qb.dtype
                      and LR._factor_kernel_ok(P.contiguous(), R.contiguous(), Qb))
        if fused_tail:
            P, R = P.contiguous(), R.contiguous()
            ss = LR.fix_factors_(P, R, Qb, m_sq)
        else:
            P, R = LR.fix_all_zero_or_nan(P, R, Qb, M3, sum_sq=m_sq)
            ss = None
        LR.rank_update_stack_(M3, P, R, alpha=-(1 - mu), beta=1.0, transpose=tr)

        if outer_pg is not None:
            if ss is None:
                ss = LR.local_column_sum_sq(R)
            work = C.all_reduce_(ss, outer_pg, op="sum", async_op=True)
            yield
            work.wait()
        direct_q = fused_tail and not (kind == "inner_sharded" and inner_pg is not None) \
            and all(q.is_contiguous() and q.dtype in (torch.float32, torch.bfloat16)
                    and q.dtype == Q[0].dtype for q in Q[:n_real])
        if fused_tail:
            Q_new = LR.normalize_columns_into(R, ss, eps, Q[:n_real] if direct_q else None)
        elif ss is not None:
            Q_new = LR.column_normalize(R, full_column_sum_sq=ss, epsilon=eps)
        else:
            Q_new = LR.column_normalize(R, epsilon=eps)

        scaled_lr = math.sqrt(fan_out / fan_in) * lr
        LR.foreach_baddbmm_(X[:n_real], P[:n_real], Q_new[:n_real], alpha=-scaled_lr,
                            beta=1 - lr * wd, transpose=tr)
        if fx is not None:   # the symmetric stacks have been read for the last time
            for w in fx:
                if w is not None and w.seq_open:
                    w.release()

        # Write the new Q back into the (possibly TP-sharded) state.
        if direct_q:
            return
        if kind == "inner_sharded" and inner_pg is not None:
            W, i_rank = dist.get_world_size(inner_pg), dist.get_rank(inner_pg)
            c = Q_new.size(-1) // W
            Q_new = Q_new[..., i_rank * c:(i_rank + 1) * c]
        torch._foreach_copy_(Q[:n_real], [q.to(Q[0].dtype) for q in Q_new.unbind(0)][:n_real])


def distributed_orthogonalize(P: Tensor, oversample: float, pg: ProcessGroup,
                              generator: Optional[torch.Generator] = None) -> Tensor:
    """Orthonormalize ``P`` whose rows are sharded over ``pg``; ``P`` is the local block
    ``[B, m/W, r]`` with ``B == W``.  The small ``[k,r]`` / ``[r,r]`` partial products are
    reduce-scattered over the batch dimension so that each rank factorizes one matrix, and the
    triangular factors are all-gathered back (reference: dion/dion.py:1310-1410)."""
    W, rank = dist.get_world_size(pg), dist.get_rank(pg)
    B, m_loc, r = P.shape
    assert B == W, "batch size must equal the size of the sharding group"
    dtype = P.dtype
    if m_loc * W <= r:
        full, _ = C.all_gather_dim0(P.transpose(0, 1).contiguous(), pg)  # [W*m_loc, B, r]
        full = full.transpose(0, 1)                                      # [B, m, r]
        q1 = LR.householder_q(full[rank:rank + 1]).to(dtype)
        allq, _ = C.all_gather_dim0(q1.contiguous(), pg)                  # [B, m, r]
        return allq[:, rank * m_loc:(rank + 1) * m_loc].contiguous()
    k = LR.sketch_rows(r, oversample)
    S = LR.random_sketch(B, k, m_loc, dtype, P.device, generator)
    SP1, _ = C.reduce_scatter_dim0(S @ P, pg, op="sum")
    R1, _ = C.all_gather_dim0(LR.qr_r_factor(SP1), pg)
    P32 = LR.right_solve_upper(R1, P.to(torch.float32))
    PP1, _ = C.reduce_scatter_dim0(P32.mT @ P32, pg, op="sum")
    R2, _ = C.all_gather_dim0(LR.cholesky_upper(PP1), pg)
    return LR.right_solve_upper(R2, P32).to(dtype).contiguous()


# Function forms kept importable under the reference's names.
orthogonalize = LR.orthogonalize
fix_all_zero_or_nan = LR.fix_all_zero_or_nan
local_column_sum_sq = LR.local_column_sum_sq
column_normalize = LR.column_normalize
foreach_baddbmm_ = LR.foreach_baddbmm_
