"""GPT training driver: CLI + YAML configuration, device-mesh set-up (DDP / FSDP2 / HSDP / TP),
optimizer factory, distributed checkpoints, trapezoid LR schedule, validation and timing.

Flags, defaults and behaviour follow the reference trainer (train.py:35-1096); differences:
``--synthetic`` trains on uniform-random tokens (no dataset needed), ``--device cpu`` runs the
whole loop on CPU ranks over gloo, step timing uses CUDA events and reports the maximum over
ranks, and wandb / tqdm are optional.
"""
from __future__ import annotations

import argparse
import os
import shutil
import time
from dataclasses import dataclass, fields
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.state_dict import get_state_dict, set_state_dict
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh
from torch.nn.parallel import DistributedDataParallel as DDP

from . import (Dion, Dion2, DionMixedPrecisionConfig, DionReference, DionSimple, Muon,
               MuonReference, NorDion2, NorMuon)
from .models.data import DistributedDataLoader, SyntheticDataLoader
from .models.gpt import GPT, GPTConfig, parallelize_gpt_model
from .utils.tensors import lm_head_lr_scale

VOCAB_SIZE = 50304  # GPT-2 vocabulary rounded up to a multiple of 128


@dataclass
class Hyperparameters:
    data_dir: str = "data/fineweb10B"
    batch_size: int = 8 * 64          # global batch size in sequences
    device_batch_size: int = 64       # sequences per device per micro-step
    sequence_length: int = 1024
    num_iterations: int = 5000
    warmup_ratio: float = 0.01
    warmdown_ratio: float = 0.2
    model_dim: int = 768
    n_layer: int = 12
    n_head: int = 6
    val_loss_every: int = 125
    val_tokens: int = 10485760
    checkpoint_freq: int = 0
    checkpoint_dir: Optional[str] = None
    wandb_project_name: str = "dion-test"
    optimizer: str = "dion"
    scalar_opt: str = "lion"
    lr: float = 0.02
    mu: float = 0.95
    weight_decay: float = 0.01
    ortho_fraction: float = 0.25
    qr_method: str = "rcqr"
    cqr_warmup: float = 0.05
    rcqr_oversample: float = 1.25
    replicate_mesh_grad_sync: bool = False
    mixed_precision: bool = False
    adjust_lr: str = "spectral_norm"
    verbose: bool = True


_MASTER = True


def print0(*args, **kwargs) -> None:
    if _MASTER:
        print(*args, **kwargs, flush=True)


def parse_cli_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Train a GPT model with an orthonormal optimizer")
    p.add_argument("--config", type=str, help="YAML file whose keys match these flags (flags win)")
    p.add_argument("--data_dir", type=str, default=None)
    p.add_argument("--checkpoint_dir", type=str, default=None)
    p.add_argument("--checkpoint_freq", type=int, default=None)
    p.add_argument("--optimizer", type=str, default=None)
    p.add_argument("--scalar_opt", type=str, default=None)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--adjust_lr", type=str, default=None,
                   choices=["spectral_norm", "rms_norm", "none"])
    p.add_argument("--qr_method", type=str, default=None, choices=["qr", "cqr", "rcqr"])
    p.add_argument("--mixed_precision", action="store_true")
    p.add_argument("--ortho_fraction", type=float, default=None)
    p.add_argument("--mu", type=float, default=None)
    p.add_argument("--weight_decay", type=float, default=None)
    p.add_argument("--time_optimizer", action="store_true",
                   help="time forward/backward and the optimizer step separately")
    p.add_argument("--model_dim", type=int, default=None)
    p.add_argument("--n_layer", type=int, default=None)
    p.add_argument("--n_head", type=int, default=None)
    p.add_argument("--num_iterations", type=int, default=None)
    p.add_argument("--batch_size", type=int, default=None)
    p.add_argument("--device_batch_size", type=int, default=None)
    p.add_argument("--sequence_length", type=int, default=None)
    p.add_argument("--warmup_ratio", type=float, default=None)
    p.add_argument("--warmdown_ratio", type=float, default=None)
    p.add_argument("--val_loss_every", type=int, default=None)
    p.add_argument("--val_tokens", type=int, default=None)
    p.add_argument("--no_wandb", action="store_true")
    p.add_argument("--wandb_project_name", type=str, default=None)
    p.add_argument("--wandb_job_name", type=str, default=None)
    p.add_argument("--dp_size", type=int, default=None)
    p.add_argument("--fs_size", type=int, default=None)
    p.add_argument("--tp_size", type=int, default=None)
    p.add_argument("--replicate_mesh_grad_sync", action="store_true")
    p.add_argument("--fast_fsdp", action="store_true",
                   help="keep parameters unsharded and skip gradient sync between micro-steps")
    p.add_argument("--debug", action="store_true")
    p.add_argument("--no_compile", action="store_true", help="accepted; nothing is traced here")
    p.add_argument("--no_triton", action="store_true", help="accepted; kernels are always CUDA")
    p.add_argument("--use_polar_express", action="store_true")
    p.add_argument("--use_gram_newton_schulz", action="store_true")
    p.add_argument("--profile_steps", type=int, default=0,
                   help="profile this many steps (after 10 warm-up steps) with torch.profiler, "
                        "with NVTX ranges on; rank 0 prints the kernel table")
    p.add_argument("--profile_trace", type=str, default=None,
                   help="write the Chrome trace of the profiled steps here (rank 0)")
    p.add_argument("--symm_all_gather", action="store_true",
                   help="FSDP2 parameter all-gather by this package's kernel over symmetric "
                        "memory (NVLS multimem / peer stores) instead of NCCL")
    p.add_argument("--graph_step", action="store_true",
                   help="Replay forward + backward + gradient all-reduce + optimizer as ONE CUDA "
                        "graph per step (single GPU or DDP, no gradient accumulation)")
    p.add_argument("--cuda_graph", action="store_true",
                   help="capture the optimizer step in a CUDA graph after warm-up")
    p.add_argument("--synthetic", action="store_true", help="uniform-random tokens, seed 0")
    p.add_argument("--device", type=str, default=None, choices=["cuda", "cpu"])
    p.add_argument("--seed", type=int, default=0)
    args = p.parse_args(argv)

    if args.config:
        import yaml

        with open(args.config) as f:
            cfg = flatten_config(yaml.safe_load(f) or {})
        store_true = {a.dest for a in p._actions if isinstance(a, argparse._StoreTrueAction)}
        for key, value in cfg.items():
            if not hasattr(args, key):
                continue
            if key in store_true:
                if value and not getattr(args, key):
                    setattr(args, key, True)
            elif getattr(args, key) is None:
                setattr(args, key, value)
    return args


def flatten_config(cfg: dict) -> dict:
    """Configuration files may group their keys in sections (``model: {...}``,
    ``optimizer: {...}``, ...); the section names carry no meaning, every leaf key is a flag of
    this script.  Flat files (one ``flag: value`` per line, the reference's layout) load the
    same way."""
    flat: dict = {}
    for key, value in cfg.items():
        if isinstance(value, dict):
            flat.update(flatten_config(value))
        else:
            flat[key] = value
    return flat


def override_args_from_cli(hp: Hyperparameters, args: argparse.Namespace) -> Hyperparameters:
    for f in fields(hp):
        val = getattr(args, f.name, None)
        if val is None:
            continue
        if isinstance(getattr(hp, f.name), bool):
            if val:
                setattr(hp, f.name, True)
        else:
            setattr(hp, f.name, val)
    if hp.adjust_lr == "none":
        hp.adjust_lr = None
    return hp


def init_distributed(dp_size, fs_size, tp_size, device_type: str = "cuda") -> Optional[DeviceMesh]:
    """Initialise the process group (plain DDP when no mesh size is given) or a 3-D
    ``("dp", "fs", "tp")`` device mesh.  Expects torchrun's RANK / LOCAL_RANK / WORLD_SIZE."""
    global _MASTER
    launcher_vars = ("RANK", "LOCAL_RANK", "WORLD_SIZE")
    if not any(v in os.environ for v in launcher_vars):
        # Started as a plain ``python train.py``: a one-process job on the local machine.
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
    elif not all(v in os.environ for v in launcher_vars):
        raise RuntimeError("This script must be launched using the 'torchrun' command.")
    rank, local_rank = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    _MASTER = rank == 0
    backend = "nccl" if device_type == "cuda" else "gloo"
    if device_type == "cuda":
        torch.cuda.set_device(local_rank)
    if all(d is None for d in (dp_size, fs_size, tp_size)):
        if not dist.is_initialized():
            dist.init_process_group(backend=backend)
        print0(f"Distributed training initialized with DDP, world size {world}")
        return None
    dp, fs, tp = (d if d is not None else 1 for d in (dp_size, fs_size, tp_size))
    if world != dp * fs * tp:
        raise AssertionError(
            f"World size {world} does not match expected size {dp * fs * tp} "
            f"(DP {dp}, FS {fs}, TP {tp})")
    if not dist.is_initialized():
        dist.init_process_group(backend=backend)
    mesh = init_device_mesh(device_type, (dp, fs, tp), mesh_dim_names=("dp", "fs", "tp"))
    print0(f"Distributed training initialized with DeviceMesh dp={dp} fs={fs} tp={tp}: {mesh}")
    return mesh


def init_optimizer(model: GPT, device_mesh: Optional[DeviceMesh], ddp_model, hp: Hyperparameters,
                   cli_args: argparse.Namespace) -> torch.optim.Optimizer:
    """Matrix parameters of the blocks go to the chosen optimizer; the embedding and the output
    head go to ``hp.scalar_opt`` (AdamW / Lion) without weight decay."""
    if hp.scalar_opt not in ("adamw", "lion"):
        raise ValueError(f"Unrecognized scalar optimizer: {hp.scalar_opt}")
    groups: List[Dict[str, Any]] = [dict(params=list(model.transformer.h.parameters()))]
    groups.append(dict(params=list(model.transformer.wte.parameters()), algorithm=hp.scalar_opt,
                       lr=hp.lr, betas=(0.95, 0.98), weight_decay=0))
    groups.append(dict(params=list(model.lm_head.parameters()), algorithm=hp.scalar_opt,
                       lr=hp.lr * lm_head_lr_scale(hp.scalar_opt, hp.model_dim),
                       betas=(0.95, 0.98), weight_decay=0))

    if device_mesh is not None:
        replicate_mesh, outer = device_mesh["dp"], device_mesh["fs"]
        inner = device_mesh["tp"] if device_mesh["tp"].size() > 1 else None
    else:
        replicate_mesh = ddp_model.process_group if ddp_model is not None else None
        outer = inner = None

    def megabatch_mesh(name: str):
        if device_mesh is None:
            return replicate_mesh
        if inner is not None and inner.size() > 1:
            raise ValueError(f"Tensor parallel is not supported by {name}.")
        return outer if outer.size() > 1 else replicate_mesh

    mp = (DionMixedPrecisionConfig(momentum_dtype=torch.bfloat16, variance_dtype=torch.bfloat16,
                                   Q_dtype=torch.bfloat16) if hp.mixed_precision else None)
    ns = dict(use_gram_newton_schulz=getattr(cli_args, "use_gram_newton_schulz", False),
              use_triton=not getattr(cli_args, "no_triton", False),
              use_polar_express=getattr(cli_args, "use_polar_express", False))
    name = hp.optimizer
    if name in ("dion", "dion_reference"):
        cls = Dion if name == "dion" else DionReference
        opt = cls(groups, replicate_mesh=replicate_mesh, outer_shard_mesh=outer,
                  inner_shard_mesh=inner, replicate_mesh_grad_sync=hp.replicate_mesh_grad_sync,
                  rank_fraction=hp.ortho_fraction, lr=hp.lr, mu=hp.mu,
                  weight_decay=hp.weight_decay, qr_method=hp.qr_method,
                  cqr_warmup_steps=round(hp.cqr_warmup * hp.num_iterations),
                  rcqr_oversample=hp.rcqr_oversample, mixed_precision_config=mp)
    elif name == "muon":
        opt = Muon(groups, distributed_mesh=megabatch_mesh("Muon"), lr=hp.lr, mu=hp.mu,
                   weight_decay=hp.weight_decay, nesterov=True, adjust_lr=hp.adjust_lr, **ns)
    elif name == "dion2":
        opt = Dion2(groups, distributed_mesh=megabatch_mesh("Dion2"), lr=hp.lr,
                    fraction=hp.ortho_fraction, ef_decay=hp.mu, weight_decay=hp.weight_decay,
                    adjust_lr=hp.adjust_lr, verbose=hp.verbose, **ns)
    elif name == "normuon":
        ns.pop("use_gram_newton_schulz")
        opt = NorMuon(groups, distributed_mesh=megabatch_mesh("NorMuon"), lr=hp.lr, mu=hp.mu,
                      muon_beta2=0.95, weight_decay=hp.weight_decay, nesterov=True,
                      adjust_lr=hp.adjust_lr, **ns)
    elif name in ("nordion2", "dion3"):
        opt = NorDion2(groups, distributed_mesh=megabatch_mesh("NorDion2"), lr=hp.lr,
                       fraction=hp.ortho_fraction, mu=hp.mu, muon_beta2=0.95,
                       weight_decay=hp.weight_decay, adjust_lr=hp.adjust_lr, **ns)
    elif name == "dion_simple":
        assert device_mesh is None, f"{name} does not support device mesh"
        opt = DionSimple(groups, lr=hp.lr, mu=hp.mu, weight_decay=hp.weight_decay,
                         rank=round(hp.ortho_fraction * hp.model_dim))
    elif name == "muon_reference":
        opt = MuonReference(groups, lr=hp.lr, mu=hp.mu, weight_decay=hp.weight_decay,
                            nesterov=True, adjust_lr=hp.adjust_lr)
    elif name == "adamw":
        for g in groups:
            g["lr"], g["betas"] = hp.lr, (0.9, 0.95)
            g.pop("algorithm", None)
        opt = torch.optim.AdamW(groups, lr=hp.lr, betas=(0.9, 0.95), weight_decay=hp.weight_decay)
    else:
        raise ValueError(f"Unsupported optimizer: {name}")
    if hp.replicate_mesh_grad_sync and name not in ("dion", "dion_reference"):
        raise ValueError("replicate_mesh_grad_sync is set for non-Dion optimizer")
    if hp.replicate_mesh_grad_sync and replicate_mesh is None and dist.is_initialized() \
            and dist.get_world_size() > 1:
        raise ValueError("replicate_mesh_grad_sync needs a replicate mesh or data-parallel "
                         "process group: nobody would average the gradients")
    return opt


class CheckpointManager:
    """Distributed checkpoints (``torch.distributed.checkpoint``) of model, optimizer, data
    loaders and step, written to a temporary directory and renamed into place."""

    def __init__(self, checkpoint_dir: str, model, optimizer, train_loader, val_loader,
                 wandb_id: Optional[str] = None, keep_last: int = 2):
        """``keep_last``: how many ``step_*`` directories survive a save (0 keeps all).  A
        directory written by the reference trainer (a single ``checkpoint`` folder that each
        save replaces, train.py:589-692 there) is recognised on load."""
        self.keep_last = keep_last
        self.checkpoint_dir = checkpoint_dir
        self.model, self.optimizer = model, optimizer
        self.train_loader, self.val_loader = train_loader, val_loader
        self.wandb_id = wandb_id
        # Position of the training loader before it prefetched the batch of the following step;
        # saved instead of the live position so that a resumed run reads the same batches as an
        # uninterrupted one.
        self.train_loader_state: Optional[dict] = None

    def _path(self, step: int) -> str:
        return os.path.join(self.checkpoint_dir, f"step_{step:08d}")

    def _steps(self) -> List[int]:
        if not os.path.isdir(self.checkpoint_dir):
            return []
        return sorted(int(d.split("_")[1]) for d in os.listdir(self.checkpoint_dir)
                      if d.startswith("step_") and d.split("_")[1].isdigit())

    def latest_step(self) -> Optional[int]:
        steps = self._steps()
        return steps[-1] if steps else None

    def _single_folder(self) -> Optional[str]:
        """The reference trainer's layout: one folder named ``checkpoint``."""
        path = os.path.join(self.checkpoint_dir, "checkpoint")
        return path if os.path.isdir(path) else None

    def exists(self) -> bool:
        return self.latest_step() is not None or self._single_folder() is not None

    def _state(self, step: int) -> Dict[str, Any]:
        model_sd, optim_sd = get_state_dict(self.model, self.optimizer)
        return {"model": model_sd, "optimizer": optim_sd,
                "train_loader": (self.train_loader_state if self.train_loader_state is not None
                                 else self.train_loader.state_dict() if self.train_loader else {}),
                "val_loader": self.val_loader.state_dict() if self.val_loader else {},
                "step": step, "wandb_id": self.wandb_id or ""}

    def save(self, step: int) -> None:
        # A kernel timeout (peer GPU that never delivered) must not end up in a checkpoint.
        check = getattr(self.optimizer, "check_device_status", None)
        if check is not None:
            check()
        final = self._path(step)
        tmp = final + ".tmp"
        rank = dist.get_rank() if dist.is_initialized() else 0
        if rank == 0:
            shutil.rmtree(tmp, ignore_errors=True)
            os.makedirs(tmp, exist_ok=True)
        if dist.is_initialized():
            dist.barrier()
        dcp.save(self._state(step), checkpoint_id=tmp)
        if dist.is_initialized():
            dist.barrier()
        if rank == 0:
            shutil.rmtree(final, ignore_errors=True)
            os.replace(tmp, final)
            if self.keep_last > 0:
                for old in self._steps()[:-self.keep_last]:
                    shutil.rmtree(self._path(old), ignore_errors=True)
        if dist.is_initialized():
            dist.barrier()

    def load(self, step: Optional[int] = None) -> int:
        step = self.latest_step() if step is None else step
        path = self._path(step) if step is not None else self._single_folder()
        if path is None:
            raise FileNotFoundError(f"no checkpoint under {self.checkpoint_dir}")
        state = self._state(0)
        dcp.load(state, checkpoint_id=path)
        set_state_dict(self.model, self.optimizer, model_state_dict=state["model"],
                       optim_state_dict=state["optimizer"])
        if self.train_loader and state["train_loader"]:
            self.train_loader.load_state_dict(state["train_loader"])
        if self.val_loader and state["val_loader"]:
            self.val_loader.load_state_dict(state["val_loader"])
        self.wandb_id = state.get("wandb_id") or None
        if dist.is_initialized():
            dist.barrier()
        return int(state["step"])


def lr_multiplier(step: int, num_iterations: int, warmup_ratio: float, warmdown_ratio: float) -> float:
    """Trapezoid: linear warm-up, flat, linear warm-down to zero."""
    warm = round(warmup_ratio * num_iterations)
    down = round(warmdown_ratio * num_iterations)
    if step < warm:
        return (step + 1) / warm
    if step < num_iterations - down:
        return 1.0
    return max(0.0, (num_iterations - step) / max(down, 1))


def build_model(hp: Hyperparameters, device_mesh: Optional[DeviceMesh], device: torch.device,
                fast_fsdp: bool = False, wrap_ddp: bool = True):
    """-> (model to call, raw GPT, DDP wrapper or None)"""
    config = GPTConfig(sequence_len=hp.sequence_length, vocab_size=VOCAB_SIZE, n_layer=hp.n_layer,
                       n_head=hp.n_head, n_embd=hp.model_dim)
    with torch.device("meta"):
        model = GPT(config)
    if device_mesh is not None:
        parallelize_gpt_model(model, device_mesh=device_mesh,
                              dp_name=(None if hp.replicate_mesh_grad_sync else "dp"),
                              fs_name="fs", tp_name="tp",
                              fsdp_reshard_after_forward=not fast_fsdp)
    model.to_empty(device=device)
    model.init_weights()
    ddp = None
    call = model
    if wrap_ddp and device_mesh is None and dist.is_initialized() and dist.get_world_size() > 1:
        if device.type == "cuda":
            ddp = DDP(model, device_ids=[device.index], output_device=device.index)
        else:
            ddp = DDP(model)
        call = ddp
    return call, model, ddp


def max_over_ranks(value: float, device: torch.device) -> float:
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class StepTimer:
    """Device-side (CUDA events) or host-side timer with the same interface."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self._t0 = None
        if self.cuda:
            self._a, self._b = torch.cuda.Event(True), torch.cuda.Event(True)

    def start(self):
        if self.cuda:
            self._a.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> float:
        """milliseconds since start()"""
        if self.cuda:
            self._b.record()
            self._b.synchronize()
            return self._a.elapsed_time(self._b)
        return 1000 * (time.perf_counter() - self._t0)


def main(argv: Optional[List[str]] = None) -> None:
    args = parse_cli_args(argv)
    hp = override_args_from_cli(Hyperparameters(), args)
    device_type = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    mesh = init_distributed(args.dp_size, args.fs_size, args.tp_size, device_type)
    rank = dist.get_rank()
    world = dist.get_world_size()
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if device_type == "cuda" \
        else torch.device("cpu")
    torch.manual_seed(args.seed)

    if mesh is not None:
        dp_mesh = mesh["dp", "fs"]._flatten() if hasattr(mesh["dp", "fs"], "_flatten") else None
        dp_rank = dp_mesh.get_local_rank() if dp_mesh is not None else rank
        dp_world = dp_mesh.size() if dp_mesh is not None else world
    else:
        dp_rank, dp_world = rank, world
    tokens_per_micro = hp.device_batch_size * dp_world
    if hp.batch_size % tokens_per_micro != 0:
        raise ValueError(f"batch_size {hp.batch_size} must be a multiple of "
                         f"device_batch_size*dp_world = {tokens_per_micro}")
    grad_accum = hp.batch_size // tokens_per_micro

    if args.synthetic:
        train_loader = SyntheticDataLoader(hp.device_batch_size, hp.sequence_length, VOCAB_SIZE,
                                           dp_rank, dp_world, seed=args.seed, device=device)
        val_loader = SyntheticDataLoader(hp.device_batch_size, hp.sequence_length, VOCAB_SIZE,
                                         dp_rank, dp_world, seed=args.seed + 1, device=device)
    else:
        train_loader = DistributedDataLoader(os.path.join(hp.data_dir, "fineweb_train_*.bin"),
                                             hp.device_batch_size, hp.sequence_length, dp_rank,
                                             dp_world, device=device)
        val_loader = DistributedDataLoader(os.path.join(hp.data_dir, "fineweb_val_*.bin"),
                                           hp.device_batch_size, hp.sequence_length, dp_rank,
                                           dp_world, device=device)

    graph_step = bool(args.graph_step) and device.type == "cuda"
    if graph_step and mesh is not None:
        raise ValueError("--graph_step needs plain data parallelism (no --dp_size/--fs_size/"
                         "--tp_size)")
    model, raw_model, ddp = build_model(hp, mesh, device, fast_fsdp=args.fast_fsdp,
                                        wrap_ddp=not graph_step)
    if graph_step and world > 1:
        # Without the DDP wrapper nothing has made the replicas identical yet.
        for t in list(raw_model.parameters()) + list(raw_model.buffers()):
            dist.broadcast(t.data, src=0)
    print0(f"Total parameters: {sum(p.numel() for p in raw_model.parameters())}")
    if args.symm_all_gather and mesh is not None and device.type == "cuda":
        from .parallel.fsdp_comm import use_symmetric_all_gather

        comm = use_symmetric_all_gather(raw_model, mesh["fs"].get_group(), device)
        print0("FSDP all-gather: " + ("symmetric-memory kernel" if comm is not None
                                      else "NCCL (symmetric memory unavailable)"))
    replicas = ddp
    if graph_step and world > 1:
        # No DDP wrapper on this path: the optimizer still has to know the data-parallel group,
        # to divide the orthogonalization work over the ranks (megabatch family).
        replicas = argparse.Namespace(process_group=dist.group.WORLD)
    optimizer = init_optimizer(raw_model, mesh, replicas, hp, args)
    if (graph_step or args.cuda_graph) and device.type == "cuda":
        from .optim.cuda_graph import require_graph_replay_support

        require_graph_replay_support(optimizer, "--graph_step / --cuda_graph")
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, lambda s: lr_multiplier(s, hp.num_iterations, hp.warmup_ratio, hp.warmdown_ratio))
    stepper = optimizer
    if args.cuda_graph and device.type == "cuda":
        from .optim.cuda_graph import CudaGraphOptimizer

        stepper = CudaGraphOptimizer(optimizer, warmup_steps=5)

    ckpt = None
    start_step = 0
    if hp.checkpoint_dir:
        ckpt = CheckpointManager(hp.checkpoint_dir, raw_model, optimizer, train_loader, val_loader)
        if ckpt.exists():
            done = ckpt.load()
            start_step = done + 1     # the checkpoint was written after step ``done`` completed
            scheduler.last_epoch = start_step
            for g, base in zip(optimizer.param_groups, scheduler.base_lrs):
                g["lr"] = base * lr_multiplier(start_step, hp.num_iterations, hp.warmup_ratio,
                                               hp.warmdown_ratio)
            print0(f"Resumed from step {done}")

    wandb = None
    if not args.no_wandb and not args.debug and rank == 0:
        try:
            import wandb as _wandb

            wandb = _wandb
            wandb.init(project=hp.wandb_project_name, name=args.wandb_job_name,
                       config=vars(hp), id=(ckpt.wandb_id if ckpt else None), resume="allow")
            if ckpt:
                ckpt.wandb_id = wandb.run.id
        except Exception as exc:  # wandb missing or offline
            print0(f"wandb disabled: {exc}")
            wandb = None

    from torch.distributed.fsdp import FSDPModule

    autocast = torch.autocast(device_type=device.type, dtype=torch.bfloat16)
    val_steps = max(1, hp.val_tokens // (hp.device_batch_size * hp.sequence_length * dp_world))
    timer_fb, timer_opt, timer_all = StepTimer(device), StepTimer(device), StepTimer(device)
    tot_fb = tot_opt = tot_all = 0.0
    timed = 0
    x, y = train_loader.next_batch()
    profiler = None
    profile_from = start_step + 10
    gstep = None
    if graph_step:
        from .parallel.graph_step import GraphedTrainStep

        sync_pg = dist.group.WORLD if (world > 1 and not hp.replicate_mesh_grad_sync) else None
        gstep = GraphedTrainStep(lambda a, b: raw_model(a, b), list(raw_model.parameters()),
                                 optimizer, [x, y], device=device, process_group=sync_pg,
                                 warmup=3, accumulation_steps=grad_accum)
    for step in range(start_step, hp.num_iterations + 1):
        last = step == hp.num_iterations
        if hp.val_loss_every > 0 and (last or step % hp.val_loss_every == 0):
            model.eval()
            val_loader.reset()
            vl = torch.zeros((), device=device)
            with torch.no_grad():
                for _ in range(val_steps):
                    vx, vy = val_loader.next_batch()
                    with autocast:
                        vl += model(vx, vy).detach().float()
            vl /= val_steps
            if world > 1:
                dist.all_reduce(vl, op=dist.ReduceOp.AVG if device.type == "cuda" else dist.ReduceOp.SUM)
                if device.type != "cuda":
                    vl /= world
            if hasattr(optimizer, "check_device_status"):
                optimizer.check_device_status()   # the host synchronizes here anyway
            msg = f"step:{step}/{hp.num_iterations} val_loss:{vl.item():.4f}"
            if timed:
                msg += (f" step_avg:{tot_all / timed:.2f}ms fwd_bwd_avg:{tot_fb / timed:.2f}ms "
                        f"opt_avg:{tot_opt / timed:.2f}ms")
            print0(msg)
            if wandb:
                wandb.log({"val/loss": vl.item(), "step": step})
        if last:
            break

        if args.profile_steps > 0:
            if step == profile_from:
                from torch.profiler import ProfilerActivity, profile
                from .utils import trace

                trace.enable(True)
                acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.type == "cuda" else [])
                profiler = profile(activities=acts)
                profiler.__enter__()
            elif profiler is not None and step == profile_from + args.profile_steps:
                if device.type == "cuda":
                    torch.cuda.synchronize()
                profiler.__exit__(None, None, None)
                if rank == 0:
                    key = "cuda_time_total" if device.type == "cuda" else "cpu_time_total"
                    print(profiler.key_averages().table(sort_by=key, row_limit=40))
                    if args.profile_trace:
                        profiler.export_chrome_trace(args.profile_trace)
                profiler = None
        model.train()
        if step == start_step + 10:  # discard warm-up steps from the averages
            tot_fb = tot_opt = tot_all = 0.0
            timed = 0
        if gstep is not None:
            timer_all.start()
            if grad_accum == 1:
                train_loss = gstep(x, y).clone()
            else:  # the graph holds all micro-batches of the step
                xs, ys = [x], [y]
                for _ in range(grad_accum - 1):
                    x, y = train_loader.next_batch()
                    xs.append(x)
                    ys.append(y)
                train_loss = gstep(torch.stack(xs), torch.stack(ys)).clone()
            scheduler.step()
            if ckpt:
                ckpt.train_loader_state = train_loader.state_dict()
            x, y = train_loader.next_batch()
            if args.time_optimizer:
                tot_all += max_over_ranks(timer_all.stop(), device)
                timed += 1
            if wandb:
                wandb.log({"train/loss": train_loss.item(), "step": step})
            if args.debug:
                print0(f"Step {step}: train_loss={train_loss.item():.4f}")
            if ckpt and hp.checkpoint_freq > 0 and step % hp.checkpoint_freq == 0 and step > 0:
                if hasattr(optimizer, "synchronize_for_checkpoint"):
                    optimizer.synchronize_for_checkpoint()
                ckpt.save(step)
            continue
        timer_all.start()
        timer_fb.start()
        for micro in range(1, grad_accum + 1):
            with autocast:
                loss = model(x, y)
            train_loss = loss.detach()
            loss = loss / grad_accum
            final = micro == grad_accum
            if final and ckpt:
                ckpt.train_loader_state = train_loader.state_dict()
            x, y = train_loader.next_batch()
            if ddp is not None and (not final or hp.replicate_mesh_grad_sync):
                with ddp.no_sync():
                    loss.backward()
            else:
                if isinstance(model, FSDPModule):
                    model.set_is_last_backward(final)
                    if args.fast_fsdp:
                        model.set_reshard_after_backward(final)
                        model.set_requires_gradient_sync(final)
                    else:
                        model.set_requires_gradient_sync(True)
                loss.backward()
        fb_ms = timer_fb.stop() if args.time_optimizer else 0.0
        timer_opt.start()
        grad_norm = torch.nn.utils.get_total_norm(
            [p.grad for p in model.parameters() if p.grad is not None])
        stepper.step()
        scheduler.step()
        if stepper is optimizer:
            model.zero_grad(set_to_none=True)
        else:
            stepper.zero_grad()
        opt_ms = timer_opt.stop() if args.time_optimizer else 0.0
        all_ms = timer_all.stop() if args.time_optimizer else 0.0
        if args.time_optimizer:
            tot_fb += max_over_ranks(fb_ms, device)
            tot_opt += max_over_ranks(opt_ms, device)
            tot_all += max_over_ranks(all_ms, device)
            timed += 1
        if wandb:
            wandb.log({"train/loss": train_loss.item(), "train/grad_norm": float(grad_norm),
                       "step": step})
        if args.debug:
            print0(f"Step {step}: train_loss={train_loss.item():.4f}, grad_norm={float(grad_norm):.4f}")
        if ckpt and hp.checkpoint_freq > 0 and step % hp.checkpoint_freq == 0 and step > 0:
            if hasattr(optimizer, "synchronize_for_checkpoint"):
                optimizer.synchronize_for_checkpoint()
            ckpt.save(step)

    if device.type == "cuda":
        print0(f"Peak memory consumption: {torch.cuda.max_memory_allocated() // 1024 // 1024} MiB")
    if hasattr(stepper, "release"):
        stepper.release()
    if gstep is not None:
        gstep.release()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
