"""Common machinery of the megabatch optimizers (Muon, Dion2, NorMuon, NorDion2).

Covers what dion/megabatch_base.py:22-632 provides in the reference: mesh / process-group
handling, choice of the Newton-Schulz driver, state created for every parameter at construction
(so that ``state_dict()`` has the same keys on every rank), learning rate and optional weight
decay carried as persistent 0-d device tensors (so that a scheduler can drive a captured CUDA
graph), shard detection for DTensor parameters, per-head and per-row-block options, and the
AdamW / Lion tasks for the non-matrix parameter groups.
"""
from __future__ import annotations

import math
from itertools import chain
from typing import Callable, Dict, Generator, Iterable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from ..ops import foreach as F
from ..ops import newton_schulz as NS
from ..parallel.async_runtime import AsyncRuntime, AsyncTask
from ..utils.arena import StepArena
from ..utils import trace
from ..utils.tensors import to_local
from .status import DeviceStatusMixin

MAX_CONCURRENT_TASKS = 3


def adjust_lr_rms_norm(lr, param_shape, flatten: bool):
    """Scale for a constant element-wise RMS of the update: ``0.2 * sqrt(max(fan_out, fan_in))``."""
    fan_out, fan_in = _fans(param_shape, flatten)
    return lr * (0.2 * math.sqrt(max(fan_out, fan_in)))


def adjust_lr_spectral_norm(lr, param_shape, flatten: bool):
    """Scale from unit spectral norm to unit RMS->RMS operator norm: ``sqrt(fan_out / fan_in)``."""
    fan_out, fan_in = _fans(param_shape, flatten)
    return lr * math.sqrt(fan_out / fan_in)


def _fans(shape, flatten: bool) -> Tuple[int, int]:
    if flatten:
        return shape[0], math.prod(shape[1:])
    return shape[-2], shape[-1]


def lr_ratio(adjust_lr: Optional[str], param_shape, flatten: bool) -> float:
    """``adjusted_lr / lr`` for the given rule."""
    if adjust_lr is None:
        return 1.0
    if adjust_lr == "spectral_norm":
        return adjust_lr_spectral_norm(1.0, param_shape, flatten)
    if adjust_lr == "rms_norm":
        return adjust_lr_rms_norm(1.0, param_shape, flatten)
    raise ValueError(f"Unknown adjust_lr value: {adjust_lr}")


def compute_split_lr_scales(split_sizes, param_shape, adjust_lr: Optional[str]):
    """Per-block factors that turn the whole-matrix LR adjustment into the adjustment each row
    block would get as a parameter of its own (reference: megabatch_base.py:952-981)."""
    if adjust_lr is None:
        return None
    if adjust_lr not in ("spectral_norm", "rms_norm"):
        raise ValueError(f"Unknown adjust_lr value: {adjust_lr}")
    cols = param_shape[-1]
    whole = lr_ratio(adjust_lr, param_shape, False)
    return tuple(lr_ratio(adjust_lr, (rows, cols), False) / whole for rows in split_sizes)


def _mesh_coordinates(mesh) -> Tuple[int, int, Optional[ProcessGroup]]:
    """(this rank, number of ranks, process group) of the 1-D mesh or process group over which
    matrices are sharded / work is divided; ``None`` means a single device."""
    if mesh is None:
        return 0, 1, None
    if isinstance(mesh, ProcessGroup):
        return dist.get_rank(mesh), dist.get_world_size(mesh), mesh
    if isinstance(mesh, DeviceMesh):
        if mesh.ndim == 1:
            return mesh.get_local_rank(), mesh.size(), mesh.get_group()
        raise ValueError(f"Only 1D DeviceMesh supported, but got {mesh.ndim}D. "
                         f"For HSDP, provide the 1D sharded sub-mesh.")
    raise TypeError(f"Invalid distributed_mesh type: {type(mesh)}. "
                    f"Expected DeviceMesh or ProcessGroup.")


class DistributedOrthoBase(DeviceStatusMixin, Optimizer):
    """Base class; subclasses implement ``_create_ortho_tasks(groups)``."""

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]],
        algo_name: str,
        defaults: dict,
        use_gram_newton_schulz: bool = False,
        use_triton: bool = False,
        use_polar_express: bool = True,
        newton_schulz_func: Optional[Callable] = None,
    ):
        super().__init__(params, defaults)
        self._algo_name = algo_name

        self._device_rank, self._world_size, self._process_group = _mesh_coordinates(
            distributed_mesh)
        self._distributed_mesh = distributed_mesh

        # Newton-Schulz driver.  ``use_triton`` is accepted for signature compatibility: on CUDA
        # every driver below already runs on the tcgen05 kernels.
        if newton_schulz_func is not None:
            if not callable(newton_schulz_func):
                raise TypeError(
                    f"newton_schulz_func must be a callable function, got {type(newton_schulz_func)}")
            self._newton_schulz_func = newton_schulz_func
        elif use_gram_newton_schulz:
            self._newton_schulz_func = lambda X, epsilon=None: NS.gram_newton_schulz(X, epsilon)
        elif use_polar_express:
            self._newton_schulz_func = NS.polar_express
        else:
            self._newton_schulz_func = NS.newton_schulz_quintic

        # State for every parameter up front, including ones that never get a gradient, so the
        # key set of state_dict() is the same on every rank and before/after a resume.
        self._arena = StepArena()
        self._fused_exchanges: dict = {}  # symmetric workspaces of the fused megabatch exchange
        self._hyperparam_tensors: Dict[Tuple[int, str], Tensor] = {}
        self._live_hyperparams_by_group: Dict[int, Tuple[str, ...]] = {}
        self._state_prepopulated = False
        for group in self.param_groups:
            self._prepopulate_group_state(group)
        self._sync_hyperparam_tensors()
        self._state_prepopulated = True

    # ------------------------------------------------------------------ state ---------------
    def _prepopulate_group_state(self, group: dict) -> None:
        for p in group["params"]:
            self._get_or_initialize_state(p, group["algorithm"])

    def add_param_group(self, param_group: dict) -> None:
        super().add_param_group(param_group)
        if not getattr(self, "_state_prepopulated", False):
            return  # still inside __init__: the constructor finishes the job for every group
        newest = len(self.param_groups) - 1
        for hyper in self._live_hyperparams(newest):
            self._ensure_hyperparam_tensor(newest, hyper)
        self._prepopulate_group_state(self.param_groups[newest])

    def _get_or_initialize_state(self, param: Tensor, algo: str) -> dict:
        state = self.state[param]
        is_adamw = algo == "adamw"
        if len(state) == 0:
            state["momentum"] = torch.zeros_like(param)
            if is_adamw:
                state["variance"] = torch.zeros_like(param)
        if is_adamw and state.get("step_dev") is None:
            # The bias-correction counter lives on the device so that it advances under graph
            # replay; fp32 because a bf16 counter stops counting at 256.
            state["step_dev"] = torch.zeros((), dtype=torch.float32,
                                            device=to_local(param).device)
        return state

    # ------------------------------------------------------------------ step ----------------
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._sync_hyperparam_tensors()
        self._poll_device_status()
        self._arena.reset()

        buckets = {"ortho": [], "lion": [], "adamw": []}
        for group in self.param_groups:
            group["step"] += 1
            algo = group["algorithm"]
            if algo == self._algo_name:
                buckets["ortho"].append(group)
            elif algo in ("lion", "adamw"):
                buckets[algo].append(group)
            else:
                raise ValueError(f"Unknown algorithm: {algo}")

        def scalar_tasks():
            # Runs when the runtime first asks for a scalar task, i.e. after every matrix task
            # has been started.  A data-parallel driver may hang a callback here that makes the
            # stream wait for gradient reductions it let run past the start of the step (the
            # embedding gradient is produced last in backward; its all-reduce then overlaps the
            # orthogonalization work, which does not read it).
            hook = getattr(self, "before_scalar_tasks", None)
            if hook is not None:
                hook()
            yield from self._create_lion_tasks(buckets["lion"])
            yield from self._create_adamw_tasks(buckets["adamw"])

        tasks = chain(self._create_ortho_tasks(buckets["ortho"]), scalar_tasks())
        with trace.span(f"{self._algo_name}.step"):
            AsyncRuntime(tasks, max_concurrent_tasks=MAX_CONCURRENT_TASKS).run()
        self._snapshot_device_status()
        return loss

    def _create_ortho_tasks(self, param_groups: List[dict]) -> Iterable[AsyncTask]:
        raise NotImplementedError

    def _create_lion_tasks(self, param_groups: List[dict]) -> Generator[AsyncTask, None, None]:
        for group in param_groups:
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            states = [self._get_or_initialize_state(p, "lion") for p in params]
            yield AsyncTask(_as_task(
                F.lion,
                to_local(params), to_local([p.grad for p in params]),
                to_local([s["momentum"] for s in states]),
                lr=group["lr"], beta1=group["beta1"], beta2=group["beta2"],
                weight_decay=group["weight_decay"], cautious_wd=group.get("cautious_wd", False)))

    def _create_adamw_tasks(self, param_groups: List[dict]) -> Generator[AsyncTask, None, None]:
        for group in param_groups:
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            states = [self._get_or_initialize_state(p, "adamw") for p in params]
            yield AsyncTask(_as_task(
                F.adamw,
                to_local(params), to_local([p.grad for p in params]),
                to_local([s["momentum"] for s in states]),
                to_local([s["variance"] for s in states]),
                lr=group["lr"], beta1=group["beta1"], beta2=group["beta2"],
                weight_decay=group["weight_decay"], epsilon=group["epsilon"],
                state_steps=[s["step_dev"] for s in states],
                cautious_wd=group.get("cautious_wd", False)))

    # ------------------------------------------------------------------ group options -------
    def _resolve_num_heads(self, group: dict) -> Optional[int]:
        """``num_heads`` > 1 turns a 2-D weight into ``num_heads`` independent matrices."""
        num_heads = group.get("num_heads")
        if num_heads is None:
            return None
        if isinstance(num_heads, bool) or not isinstance(num_heads, int) or num_heads < 1:
            raise ValueError(f"num_heads must be a positive integer if set, got {num_heads!r}.")
        if num_heads == 1:
            return None
        if group.get("flatten"):
            raise ValueError(
                "num_heads > 1 is incompatible with flatten=True: flattening the per-head 3D "
                "view collapses heads back into a single 2D matrix, defeating per-head "
                "Newton-Schulz.")
        return num_heads

    def _resolve_split_sizes(self, group: dict) -> Optional[Tuple[int, ...]]:
        """``split_sizes`` partitions dim 0 of a fused 2-D weight (e.g. QKV under GQA) into row
        blocks that are orthogonalized and LR-adjusted independently."""
        split_sizes = group.get("split_sizes")
        if split_sizes is None:
            return None
        if not isinstance(split_sizes, (tuple, list)) or len(split_sizes) < 2:
            raise ValueError(
                f"split_sizes must be a tuple or list of at least 2 block sizes, got {split_sizes!r}.")
        if any(isinstance(s, bool) or not isinstance(s, int) or s < 1 for s in split_sizes):
            raise ValueError(f"split_sizes entries must be positive integers, got {split_sizes!r}.")
        if self._resolve_num_heads(group) is not None:
            raise ValueError(
                "split_sizes is incompatible with num_heads > 1: use num_heads for uniform "
                "per-head splits or split_sizes for uneven row blocks, not both.")
        if group.get("flatten"):
            raise ValueError(
                "split_sizes is incompatible with flatten=True: split_sizes applies to 2D "
                "parameters only.")
        return tuple(split_sizes)

    def _validate_split_shape(self, split_sizes: Tuple[int, ...], params: List[Tensor]) -> None:
        shape = params[0].shape
        if len(shape) != 2:
            raise ValueError(
                f"split_sizes is only supported for 2D parameters, got shape {tuple(shape)}.")
        if sum(split_sizes) != shape[0]:
            raise ValueError(
                f"split_sizes {split_sizes} must sum to dim 0 of the parameter "
                f"(got shape {tuple(shape)}).")

    def _prepare_head_split(self, num_heads: int, params: List[Tensor], *extras: List[Tensor]):
        """Local 3-D views ``(heads_local, head_dim, ...)`` of 2-D parameters and of companion
        tensors with the same dim 0.  The views alias the storage, so in-place updates land in
        the parameters.  A dim-0 shard must hold whole heads."""
        first = params[0]
        if first.ndim != 2:
            raise ValueError(
                f"num_heads is only supported for 2D parameters, got shape {tuple(first.shape)}.")
        if first.shape[0] % num_heads != 0:
            raise ValueError(
                f"num_heads ({num_heads}) must divide dim 0 of the parameter "
                f"(got shape {tuple(first.shape)}).")
        head_dim = first.shape[0] // num_heads
        if isinstance(first, DTensor):
            sharded = [(i, pl) for i, pl in enumerate(first.placements)
                       if pl.is_shard() and first.device_mesh.size(i) > 1]
            if any(pl.dim != 0 for _, pl in sharded):
                raise NotImplementedError(
                    f"num_heads requires sharding on dim 0 (the heads dim) or no sharding; "
                    f"got placements {first.placements}.")
            if sharded:
                world = first.device_mesh.size(sharded[0][0])
                if num_heads % world != 0:
                    raise ValueError(
                        f"num_heads ({num_heads}) must be divisible by the sharding world_size "
                        f"({world}) so each rank holds whole heads.")

        def view3d(t: Tensor) -> Tensor:
            loc = to_local(t)
            if loc.shape[0] % head_dim != 0:
                raise RuntimeError(
                    f"Local shard dim 0 ({loc.shape[0]}) is not a multiple of head_dim "
                    f"({head_dim}); shard boundaries must align with heads.")
            return loc.view(loc.shape[0] // head_dim, head_dim, *loc.shape[1:])

        return tuple([view3d(t) for t in lst] for lst in (params,) + extras)

    def _get_shard_info(self, param: Tensor, group: dict):
        """-> (is_batch_sharded, is_matrix_sharded, sharded_tensor_dim)"""
        if not isinstance(param, DTensor):
            return False, False, None
        if not isinstance(self._distributed_mesh, DeviceMesh):
            raise RuntimeError("Must create optimizer with DeviceMesh if using DTensor parameters.")
        shards = [(i, pl) for i, pl in enumerate(param.placements)
                  if pl.is_shard() and param.device_mesh.size(i) > 1]
        batch_sharded = False
        if not group["flatten"]:
            matrix_dims = {param.ndim - 1, param.ndim - 2}
            batch_sharded = any(pl.dim not in matrix_dims for _, pl in shards)
            shards = [(i, pl) for i, pl in shards if pl.dim in matrix_dims]
        if len(shards) > 1:
            raise NotImplementedError(
                f"{self.__class__.__name__} does not support parameters with multiple sharded dimensions.")
        if not shards:
            return batch_sharded, False, None
        mesh_dim, placement = shards[0]
        if param.device_mesh.get_group(mesh_dim) != self._process_group:
            raise RuntimeError(
                f"Got DTensor sharded over mesh dimension {mesh_dim} different from the "
                f"optimizer's device mesh. DTensor has mesh: {param.device_mesh}, placements: "
                f"{param.placements}, but optimizer was created with mesh: {self._distributed_mesh}.")
        return batch_sharded, True, placement.dim

    def _bucket_layout(self, group: dict, params: List[Tensor], num_heads: Optional[int]):
        """-> (process_group or None, shard_dim or None) for one shape bucket."""
        if num_heads is not None:
            return None, None
        batch_sharded, matrix_sharded, dim = self._get_shard_info(params[0], group)
        if batch_sharded and not matrix_sharded:
            return None, dim
        return self._process_group, dim

    # ------------------------------------------------------------------ live hyperparams ----
    def _live_hyperparams(self, index: int) -> Tuple[str, ...]:
        """Hyper-parameters of group ``index`` that live in persistent device tensors.  ``lr``
        always; ``weight_decay`` once the caller has supplied a Tensor for it (the opt-in
        latches: later float assignments refill the tensor instead of replacing it)."""
        known = self._live_hyperparams_by_group.get(index, ())
        if "weight_decay" not in known and isinstance(
                self.param_groups[index].get("weight_decay"), Tensor):
            known = ("lr", "weight_decay")
        elif not known:
            known = ("lr",)
        self._live_hyperparams_by_group[index] = known
        return known

    def _ensure_hyperparam_tensor(self, index: int, name: str) -> Optional[Tensor]:
        """Make ``param_groups[index][name]`` the group's persistent 0-d fp32 device tensor.
        The tensor is allocated once and afterwards only filled, because a captured graph keeps
        reading the tensor it recorded."""
        group = self.param_groups[index]
        if len(group["params"]) == 0:
            return None
        slot = (index, name)
        held = self._hyperparam_tensors.get(slot)
        current = group[name]
        if current is held:          # already the persistent tensor (possibly refilled in place)
            return held
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                f"param group {index}: {name} is a {type(current).__name__}, not the group's "
                f"persistent device tensor, and it cannot be refreshed while a CUDA graph is "
                f"being captured.  Sync {name} before capturing (CudaGraphOptimizer does).")
        device = to_local(group["params"][0]).device
        if held is None or held.device != device:
            held = self._hyperparam_tensors[slot] = torch.empty((), dtype=torch.float32,
                                                               device=device)
        held.copy_(current) if isinstance(current, Tensor) else held.fill_(current)
        group[name] = held
        return held

    def _sync_hyperparam_tensors(self) -> None:
        for index, _ in enumerate(self.param_groups):
            for name in self._live_hyperparams(index):
                self._ensure_hyperparam_tensor(index, name)

    def _advance_host_step_counters(self) -> None:
        """Host ``group["step"]`` bookkeeping for a step that ran as a graph replay."""
        for group in self.param_groups:
            group["step"] = group["step"] + 1

    # ------------------------------------------------------------------ checkpointing -------
    def state_dict(self):
        """As ``Optimizer.state_dict`` with every 0-d tensor hyper-parameter (lr, a scheduler's
        initial_lr, tensor weight decay) written as a python number: checkpoints carry no device
        tensors in their param groups."""
        sd = super().state_dict()
        sd["param_groups"] = [
            {k: (v.item() if k != "params" and isinstance(v, Tensor) and v.ndim == 0 else v)
             for k, v in group.items()}
            for group in sd["param_groups"]]
        return sd

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._sync_hyperparam_tensors()
        adamw_params = [(p, g) for g in self.param_groups if g["algorithm"] == "adamw"
                        for p in g["params"]]
        for param, group in adamw_params:
            state = self.state.get(param)
            if state is not None:
                self._restore_step_tensor(state, param, group)

    def _restore_step_tensor(self, state: dict, param: Tensor, group: dict) -> None:
        """``Optimizer.load_state_dict`` casts state to the parameter dtype and device; put the
        AdamW counter back to fp32 on the parameter's device, or rebuild it from the host step
        for checkpoints that predate it."""
        device = to_local(param).device
        counter = state.get("step_dev")
        if counter is None:
            counter = torch.full((), float(group["step"]), dtype=torch.float32, device=device)
        elif counter.dtype != torch.float32 or counter.device != device:
            counter = counter.to(dtype=torch.float32, device=device)
        state["step_dev"] = counter


def _as_task(fn: Callable, *args, **kwargs) -> Generator[None, None, None]:
    """A one-leg task: run ``fn`` and yield once so the runtime can interleave it."""
    fn(*args, **kwargs)
    yield
