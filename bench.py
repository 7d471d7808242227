#!/usr/bin/env python
"""Headline benchmark: GPT-160M (12 layers, d_model 768, 12 heads, vocab 50304, seq 1024) trained
with Dion2 (fraction 0.25, ef_decay 0.95, AdamW for embedding/head) under DDP, bf16 autocast with
fp32 master weights, 32x1024 uniform-random tokens per GPU per step, random init at seed 0.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints one JSON line.  ``value`` is whole-job tokens/s of the device-timed loop (inputs
already on the GPU); ``e2e.value`` is tokens/s of the loop a user runs: every step copies its
batch from pinned host memory, runs forward/backward/optimizer through the public API and reads
the loss back to the host.  ``--impl reference`` runs the unmodified reference package from
``baseline/_ref`` (its GPT model, its Dion2 with its Triton kernels, torch DDP) on the same
configuration and prints the same line with ``"impl": "reference"``.

After the headline both arms time a second block, printed under the key ``aux`` of the same line:
the optimizer step alone of GPT-1B (24 layers, d_model 2048) under Muon on the model's block
matrices (96 x 2048^2, 24 x 8192x2048, 24 x 2048x8192) held the way FSDP2 holds them: fp32
``Shard(0)`` DTensors over the N ranks (plain tensors for N = 1), with fixed random gradients.
Ours runs it twice, with the all-to-all carried by the compute kernels over peer memory
(``fused_ms``) and with NCCL ``all_to_all_single`` (``nccl_ms``); the reference runs its own
``dion.Muon`` (Triton Newton-Schulz, NCCL all-to-all).  ``aux.dion`` times the legacy Dion step
(rank 1/4) on the same matrices under data parallelism with compressed P/R synchronisation, and
``aux.newton_schulz`` five iterations on 16 matrices of 4096 x 4096 per GPU.  ``--no-aux`` skips
the block.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

MODEL = dict(n_layer=12, n_embd=768, n_head=12, vocab_size=50304, sequence_len=1024)
DEVICE_BATCH = 32
SEQ = 1024
PRIME_STEPS = 3   # untimed steps both arms take before the warm-up (compile / capture)
LR, FRACTION, MU, WD = 0.02, 0.25, 0.95, 0.01


def parse() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--optimizer", type=str, default="dion2",
                   choices=["dion2", "muon", "normuon", "nordion2", "dion"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-aux", action="store_true",
                   help="skip the GPT-1B Muon optimizer-step block")
    p.add_argument("--aux-steps", type=int, default=20)
    p.add_argument("--aux-warmup", type=int, default=5)
    p.add_argument("--eager", action="store_true",
                   help="ours: launch every kernel from Python (torch DDP for N>1) instead of "
                        "replaying the whole step as one CUDA graph")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def setup_dist(n_gpus: int):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return rank, local_rank, world


def time_loop(step_fn, steps: int, warmup: int, world: int, device, sampler=None,
              on_start=None):
    """Runs ``warmup`` untimed and ``steps`` timed calls of ``step_fn`` bracketed by
    barrier + synchronize; returns the device time in ms (max over ranks)."""
    import torch
    import torch.distributed as dist

    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    if on_start is not None:
        on_start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else None
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, clocks


def synthetic_batches(n: int, rank: int, device):
    """``n`` (x, y) batches of uniform-random token ids in pinned host memory."""
    import numpy as np
    import torch

    out = []
    for i in range(n):
        rng = np.random.default_rng([0, rank, i])
        w = torch.from_numpy(rng.integers(0, MODEL["vocab_size"], size=DEVICE_BATCH * SEQ + 1,
                                          dtype=np.int64))
        host = torch.empty((2, DEVICE_BATCH, SEQ), dtype=torch.int64).pin_memory()
        host[0].copy_(w[:-1].view(DEVICE_BATCH, SEQ))
        host[1].copy_(w[1:].view(DEVICE_BATCH, SEQ))
        out.append(host)
    return out


def emit(args, impl, ms, e2e_ms, clocks, launches, world, extra=None):
    tokens = world * DEVICE_BATCH * SEQ * args.steps
    value = tokens / (ms / 1e3)
    line = {
        "metric": "training throughput, GPT-160M Dion2 DDP (tokens/sec, whole job)",
        "impl": impl,
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random token ids, random-init weights (seed 0)",
        "config": {"model": "GPT-160M (12L, d768, 12 heads, vocab 50304)",
                   "optimizer": f"{args.optimizer} fraction={FRACTION} ef_decay={MU} lr={LR} "
                                f"wd={WD} + AdamW(embedding, head)",
                   "global_batch": world * DEVICE_BATCH, "seq_len": SEQ,
                   "parallelism": f"ddp{world}",
                   "precision": "bf16 autocast, fp32 master weights and optimizer state",
                   "l2": "working set per step (weights, activations, logits) is several GB, "
                         "far larger than the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s",
                       "ms_per_step": e2e_ms / args.steps,
                       "h2d_bytes_per_step": 2 * DEVICE_BATCH * SEQ * 8,
                       "d2h_bytes_per_step": 4}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# second block: GPT-1B Muon optimizer step on FSDP-style shards
# ------------------------------------------------------------------------------------------------
AUX_D, AUX_LAYERS = 2048, 24
NVLINK_BYTES_PER_S = 770e9     # measured peer copy per direction per GPU on this kind of box


def aux_shapes():
    d, n = AUX_D, AUX_LAYERS
    return [(d, d)] * (4 * n) + [(4 * d, d)] * n + [(d, 4 * d)] * n


def measured_peak_tflops() -> float:
    """Sustained cuBLAS bf16 rate of this pool's GPUs when a measurement file lies beside this
    script, else a typical sustained figure for a B200 under its power cap."""
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
                     ["bf16_tflops_sustained"])
    except Exception:  # noqa: BLE001
        return 1400.0


def aux_bounds(world: int) -> dict:
    """Work of one Muon step on ``aux_shapes()`` per rank: Newton-Schulz FLOPs by the reference's
    cost model (5 x (4 m^2 n + 2 m^3), benchmark/benchmark_newton_shultz.py:40-45), the
    multiply-adds actually needed when the two symmetric products are computed as half
    (5 x (3 m^2 n + m^3)), and the bf16 bytes each rank sends (shards out, results back)."""
    nominal = real = elems = 0.0
    for r, c in aux_shapes():
        m, n = min(r, c), max(r, c)
        nominal += 5 * (4.0 * m * m * n + 2.0 * m ** 3)
        real += 5 * (3.0 * m * m * n + 1.0 * m ** 3)
        elems += r * c
    sent = 2 * (elems * 2 / world) * (world - 1) / world if world > 1 else 0.0
    peak = measured_peak_tflops() * 1e12
    compute_ms = real / world / peak * 1e3
    link_ms = sent / NVLINK_BYTES_PER_S * 1e3
    return {"ns_tflop_nominal_per_gpu": nominal / world / 1e12,
            "ns_tflop_needed_per_gpu": real / world / 1e12,
            "nvlink_mb_sent_per_gpu": sent / 1e6,
            "compute_bound_ms": compute_ms, "nvlink_bound_ms": link_ms,
            "roofline_ms": max(compute_ms, link_ms), "peak_tflops_used": peak / 1e12}


def aux_tensors(world: int, rank: int, device):
    """Parameters and gradients of the block matrices: fp32 (as FSDP2 keeps sharded parameters
    under its bf16 mixed-precision policy), gradient values representable in bf16, seed 0.
    -> (params, grads, mesh)"""
    import torch

    gen = torch.Generator(device=device).manual_seed(0)

    def make(shape, scale):
        t = torch.randn(*shape, device=device, dtype=torch.float32, generator=gen) * scale
        return t.bfloat16().float()

    if world == 1:
        params = [torch.nn.Parameter(make(s, 0.02)) for s in aux_shapes()]
        grads = [make(s, 1.0) for s in aux_shapes()]
        return params, grads, None
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard

    mesh = init_device_mesh("cuda", (world,))

    def shard(shape, scale):
        return DTensor.from_local(make((shape[0] // world, shape[1]), scale), mesh, [Shard(0)],
                                  run_check=False)

    params = [torch.nn.Parameter(shard(s, 0.02)) for s in aux_shapes()]
    grads = [shard(s, 1.0) for s in aux_shapes()]
    return params, grads, mesh


def aux_time(opt, params, grads, steps: int, warmup: int, world: int, device) -> float:
    """ms per optimizer step, CUDA events, max over ranks."""
    def step():
        for p, g in zip(params, grads):
            p.grad = g
        opt.step()

    ms, _ = time_loop(step, steps, warmup, world, device)
    return ms / steps


def run_aux_ours(args, rank: int, world: int, device) -> dict:
    import torch

    import dion_b200
    from dion_b200.ops.gemm import check_status

    out = {"what": "GPT-1B Muon optimizer step on the block matrices (96x2048^2, 24x8192x2048, "
                   "24x2048x8192), fp32 Shard(0) over N ranks, nesterov, quintic Newton-Schulz",
           "steps": args.aux_steps, "warmup": args.aux_warmup, "n_gpus": world}
    out.update(aux_bounds(world))
    params, grads, mesh = aux_tensors(world, rank, device)
    variants = [("fused", "1"), ("nccl", "0")] if world > 1 else [("single", "1")]
    old = os.environ.get("DION_B200_FUSED_EXCHANGE")
    try:
        for label, env in variants:
            os.environ["DION_B200_FUSED_EXCHANGE"] = env
            opt = dion_b200.Muon([dict(params=params)], distributed_mesh=mesh, lr=LR, mu=MU,
                                 weight_decay=WD, nesterov=True, use_polar_express=False)
            ms = aux_time(opt, params, grads, args.aux_steps, args.aux_warmup, world, device)
            out[f"{label}_ms"] = ms
            out[f"{label}_fraction_of_roofline"] = out["roofline_ms"] / ms
            if label == "fused":
                out["n_fused_exchanges"] = len(opt._fused_exchanges)
            try:
                check_status()
                out[f"{label}_status"] = "ok"
            except RuntimeError as exc:
                out[f"{label}_status"] = str(exc)
            del opt
            torch.cuda.empty_cache()
    finally:
        if old is None:
            os.environ.pop("DION_B200_FUSED_EXCHANGE", None)
        else:
            os.environ["DION_B200_FUSED_EXCHANGE"] = old
    return out


def aux_dion_tensors(world: int, device):
    """GPT-1B block matrices held the way DDP holds them (every rank a full fp32 copy, equal on
    all ranks) with gradients that differ per rank; seed 0."""
    import torch

    gen = torch.Generator(device=device).manual_seed(0)
    params = [torch.nn.Parameter((torch.randn(*s, device=device, generator=gen) * 0.02)
                                 .bfloat16().float()) for s in aux_shapes()]
    rank_gen = torch.Generator(device=device).manual_seed(1 + int(os.environ.get("RANK", "0")))
    grads = [torch.randn(*s, device=device, generator=rank_gen).bfloat16().float()
             for s in aux_shapes()]
    return params, grads


def run_aux_dion_ours(args, rank: int, world: int, device) -> dict:
    """Legacy Dion (rank fraction 1/4) optimizer step on the GPT-1B block matrices under data
    parallelism with compressed synchronisation (P and R travel instead of the gradients): with
    the reduce-scatter inside the GEMM epilogue over peer memory, and with NCCL collectives."""
    import torch
    import torch.distributed as dist

    import dion_b200
    from dion_b200.ops.gemm import check_status

    out = {"what": "legacy Dion (rank 1/4, rcQR) optimizer step, GPT-1B block matrices, fp32, "
                   "data parallel with compressed P/R synchronisation",
           "steps": args.aux_steps, "warmup": args.aux_warmup, "n_gpus": world}
    params, grads = aux_dion_tensors(world, device)
    pg = dist.group.WORLD if world > 1 else None
    variants = [("fused", "1"), ("nccl", "0")] if world > 1 else [("single", "1")]
    old = os.environ.get("DION_B200_FUSED_LOWRANK")
    try:
        for label, env in variants:
            os.environ["DION_B200_FUSED_LOWRANK"] = env
            opt = dion_b200.Dion([dict(params=params)], replicate_mesh=pg,
                                 replicate_mesh_grad_sync=world > 1, rank_fraction=FRACTION,
                                 lr=LR, mu=MU, weight_decay=WD)
            out[f"{label}_ms"] = aux_time(opt, params, grads, args.aux_steps, args.aux_warmup,
                                          world, device)
            if label == "fused":
                out["n_fused_workspaces"] = len(opt._lowrank_sync)
            try:
                check_status()
                out[f"{label}_status"] = "ok"
            except RuntimeError as exc:
                out[f"{label}_status"] = str(exc)
            del opt
            torch.cuda.empty_cache()
    finally:
        if old is None:
            os.environ.pop("DION_B200_FUSED_LOWRANK", None)
        else:
            os.environ["DION_B200_FUSED_LOWRANK"] = old
    return out


def run_aux_dion_reference(args, ref_dion, rank: int, world: int, device) -> dict:
    import torch.distributed as dist

    out = {"what": "legacy Dion optimizer step, unmodified reference dion.Dion on the same "
                   "tensors (cuBLAS / cuSOLVER, NCCL)",
           "steps": args.aux_steps, "warmup": args.aux_warmup, "n_gpus": world}
    params, grads = aux_dion_tensors(world, device)
    pg = dist.group.WORLD if world > 1 else None
    opt = ref_dion.Dion([dict(params=params)], replicate_mesh=pg,
                        replicate_mesh_grad_sync=world > 1, rank_fraction=FRACTION, lr=LR, mu=MU,
                        weight_decay=WD)
    out["reference_ms"] = aux_time(opt, params, grads, min(args.aux_steps, 10), 3, world, device)
    return out


NS_BATCH, NS_DIM = 16, 4096


def run_aux_ns(fn, device) -> dict:
    """Five Newton-Schulz iterations on 16 bf16 matrices of 4096 x 4096 (entries N(0,1)), one
    GPU's worth of work; ms per call and TFLOP/s by the reference's cost model."""
    import torch

    gen = torch.Generator(device=device).manual_seed(0)
    X = torch.randn(NS_BATCH, NS_DIM, NS_DIM, device=device, generator=gen).bfloat16()
    ms, _ = time_loop(lambda: fn(X), 10, 3, 1, device)
    ms /= 10
    flops = NS_BATCH * 5 * 6.0 * NS_DIM ** 3
    return {"what": "Newton-Schulz, 5 quintic iterations, 16 x 4096 x 4096 bf16, per GPU",
            "ms": ms, "tflops_reference_cost_model": flops / ms / 1e9,
            "fraction_of_measured_cublas_sustained": flops / ms / 1e9 / measured_peak_tflops()}


def run_aux_reference(args, ref_dion, rank: int, world: int, device) -> dict:
    out = {"what": "GPT-1B Muon optimizer step, unmodified reference dion.Muon (Triton "
                   "Newton-Schulz, NCCL all-to-all) on the same tensors",
           "steps": args.aux_steps, "warmup": args.aux_warmup, "n_gpus": world}
    out.update(aux_bounds(world))
    params, grads, mesh = aux_tensors(world, rank, device)
    # Arguments as the reference trainer builds them (train.py:421-446).
    opt = ref_dion.Muon([dict(params=params)], distributed_mesh=mesh, lr=LR, mu=MU,
                        weight_decay=WD, nesterov=True, adjust_lr="spectral_norm",
                        use_triton=True, use_polar_express=False)
    ms = aux_time(opt, params, grads, args.aux_steps, args.aux_warmup, world, device)
    out["reference_ms"] = ms
    out["reference_fraction_of_roofline"] = out["roofline_ms"] / ms
    return out


def guarded_aux(fn, *a) -> dict:
    """The second block must never cost the headline: report its failure instead."""
    try:
        return fn(*a)
    except Exception as exc:  # noqa: BLE001
        return {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    sys.path.insert(0, ROOT)
    import dion_b200
    from dion_b200.models.gpt import GPT, GPTConfig
    from dion_b200.ops import _backend

    rank, local_rank, world = setup_dist(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.manual_seed(0)
    model = GPT(GPTConfig(**MODEL)).to(device)
    model.init_weights()
    # Legacy Dion hands its learning rate to the kernels as a host number: no graph replay.
    graphed = not args.eager and args.optimizer != "dion"
    if graphed:
        # Same seed on every rank, so the replicas start identical; gradients are averaged by
        # the step object's own bucketed all-reduce.
        call = model
        pg = dist.group.WORLD if world > 1 else None
    else:
        call = DDP(model, device_ids=[local_rank]) if world > 1 else model
        pg = call.process_group if world > 1 else None

    groups = [dict(params=list(model.transformer.h.parameters())),
              dict(params=list(model.transformer.wte.parameters()), algorithm="adamw", lr=LR,
                   betas=(0.95, 0.98), weight_decay=0),
              dict(params=list(model.lm_head.parameters()), algorithm="adamw", lr=LR,
                   betas=(0.95, 0.98), weight_decay=0)]
    name = args.optimizer
    if name == "dion2":
        opt = dion_b200.Dion2(groups, distributed_mesh=pg, lr=LR, fraction=FRACTION, ef_decay=MU,
                              weight_decay=WD, use_polar_express=False)
    elif name == "muon":
        opt = dion_b200.Muon(groups, distributed_mesh=pg, lr=LR, mu=MU, weight_decay=WD,
                             nesterov=True, use_polar_express=False)
    elif name == "normuon":
        opt = dion_b200.NorMuon(groups, distributed_mesh=pg, lr=LR, mu=MU, weight_decay=WD,
                                nesterov=True, use_polar_express=False)
    elif name == "nordion2":
        opt = dion_b200.NorDion2(groups, distributed_mesh=pg, lr=LR, fraction=FRACTION, mu=MU,
                                 weight_decay=WD, use_polar_express=False)
    else:
        opt = dion_b200.Dion(groups, replicate_mesh=pg, replicate_mesh_grad_sync=False,
                             rank_fraction=FRACTION, lr=LR, mu=MU, weight_decay=WD)

    autocast = torch.autocast(device_type="cuda", dtype=torch.bfloat16)
    host = synthetic_batches(4, rank, device)
    dev_batches = [h.to(device) for h in host]
    state = {"i": 0, "loss": None}

    if graphed:
        from dion_b200.parallel.graph_step import GraphedTrainStep

        gstep = GraphedTrainStep(lambda x, y: model(x, y), list(model.parameters()), opt,
                                 [dev_batches[0][0], dev_batches[0][1]], device=device,
                                 process_group=pg, warmup=2)
        # Prime (PRIME_STEPS calls): two eager steps, then the capture; count the kernels one
        # replay launches.
        for i in range(2):
            gstep(dev_batches[i][0], dev_batches[i][1])
        _backend.reset_launch_count()
        gstep(dev_batches[2][0], dev_batches[2][1])
        launches_per_step = _backend.launch_count()
        torch.cuda.synchronize()
        state["i"] = PRIME_STEPS

        def step_device():
            xy = dev_batches[state["i"] % len(dev_batches)]
            state["i"] += 1
            state["loss"] = gstep(xy[0], xy[1])

        def step_e2e():
            xy = host[state["i"] % len(host)]
            state["i"] += 1
            state["loss_host"] = gstep(xy[0], xy[1]).item()
    else:
        launches_per_step = None

        def step_device():
            xy = dev_batches[state["i"] % len(dev_batches)]
            state["i"] += 1
            with autocast:
                loss = call(xy[0], xy[1])
            loss.backward()
            opt.step()
            call.zero_grad(set_to_none=True)
            state["loss"] = loss.detach()

        for _ in range(PRIME_STEPS):
            step_device()

        def step_e2e():
            xy = host[state["i"] % len(host)].to(device, non_blocking=True)
            state["i"] += 1
            with autocast:
                loss = call(xy[0], xy[1])
            loss.backward()
            opt.step()
            call.zero_grad(set_to_none=True)
            state["loss_host"] = loss.item()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms, clocks = time_loop(step_device, args.steps, args.warmup, world, device, sampler,
                           on_start=_backend.reset_launch_count)
    launches = (_backend.launch_count() if launches_per_step is None
                else launches_per_step * args.steps)
    from dion_b200.ops.gemm import check_status

    check_status()
    # Loss of the last device-timed step: the same step index, on the same batches, in both arms.
    loss_after = float(state["loss"].item())
    e2e_ms = None
    if not args.no_e2e:
        e2e_ms, _ = time_loop(step_e2e, args.steps, 2, world, device, None)
    if graphed:
        gstep.release()
    torch.cuda.empty_cache()
    aux = None
    if not args.no_aux:
        from dion_b200.ops.newton_schulz import newton_schulz_quintic

        aux = guarded_aux(run_aux_ours, args, rank, world, device)
        torch.cuda.empty_cache()
        aux["dion"] = guarded_aux(run_aux_dion_ours, args, rank, world, device)
        torch.cuda.empty_cache()
        aux["newton_schulz"] = guarded_aux(run_aux_ns, newton_schulz_quintic, device)
    if rank == 0:
        emit(args, "ours", ms, e2e_ms, clocks, launches, world,
             {"final_loss": loss_after,
              "final_loss_after_steps": PRIME_STEPS + args.warmup + args.steps,
              "aux": aux,
              "launch_mode": "one CUDA graph per step (forward, backward, gradient all-reduce, "
                             "optimizer); gpu_launches counts the kernels of this package "
                             "recorded in the graph x steps" if graphed else "eager"})
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------
def run_reference(args) -> None:
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "dion")):
        print(json.dumps({"impl": "reference",
                          "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return
    sys.path.insert(0, ref_root)
    # The image's default g++ (/opt/gcc) cannot link OpenMP (no libgomp.spec), which breaks every
    # torch.compile call of the reference; the system compiler works.
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    try:
        import torch
        import torch.distributed as dist
        from torch.nn.parallel import DistributedDataParallel as DDP

        import dion as ref_dion                      # the reference package
        from models.gpt_model import GPT, GPTConfig  # the reference model (baseline/_ref/models)
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference",
                          "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"}))
        return
    if not ref_dion.__file__.startswith(ref_root):
        print(json.dumps({"impl": "reference",
                          "unavailable": "import dion did not resolve to baseline/_ref"}))
        return

    rank, local_rank, world = setup_dist(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.manual_seed(0)
    model = GPT(GPTConfig(**MODEL)).to(device)
    model.init_weights()
    compiled = True
    try:
        model.compile()  # the reference trainer's stock path (train.py:815-816)
    except Exception:  # noqa: BLE001
        compiled = False
    call = DDP(model, device_ids=[local_rank]) if world > 1 else model
    pg = call.process_group if world > 1 else None
    groups = [dict(params=list(model.transformer.h.parameters())),
              dict(params=list(model.transformer.wte.parameters()), algorithm="adamw", lr=LR,
                   betas=(0.95, 0.98), weight_decay=0),
              dict(params=list(model.lm_head.parameters()), algorithm="adamw", lr=LR,
                   betas=(0.95, 0.98), weight_decay=0)]
    # Arguments as the reference trainer builds them (train.py:448-470): Triton Newton-Schulz and
    # the Triton post-update on, Polar-Express off.
    name = args.optimizer
    if name == "dion2":
        opt = ref_dion.Dion2(groups, distributed_mesh=pg, lr=LR, fraction=FRACTION, ef_decay=MU,
                             weight_decay=WD, adjust_lr="spectral_norm", use_triton=True,
                             use_polar_express=False, verbose=False, triton_post_ortho=True)
    elif name == "muon":
        opt = ref_dion.Muon(groups, distributed_mesh=pg, lr=LR, mu=MU, weight_decay=WD,
                            nesterov=True, use_triton=True, use_polar_express=False)
    elif name == "normuon":
        opt = ref_dion.NorMuon(groups, distributed_mesh=pg, lr=LR, mu=MU, weight_decay=WD,
                               nesterov=True, use_triton=True, use_polar_express=False)
    elif name == "nordion2":
        opt = ref_dion.NorDion2(groups, distributed_mesh=pg, lr=LR, fraction=FRACTION, mu=MU,
                                weight_decay=WD, use_triton=True, use_polar_express=False,
                                triton_post_ortho=True)
    else:
        opt = ref_dion.Dion(groups, replicate_mesh=pg, replicate_mesh_grad_sync=False,
                            rank_fraction=FRACTION, lr=LR, mu=MU, weight_decay=WD)

    autocast = torch.autocast(device_type="cuda", dtype=torch.bfloat16)
    host = synthetic_batches(4, rank, device)
    dev_batches = [h.to(device) for h in host]
    state = {"i": 0, "loss": None}

    # The reference runs through its own public API only: its model (compiled as its trainer
    # does), its optimizer, torch DDP; nothing of dion_b200 is on this path.
    def step_device():
        xy = dev_batches[state["i"] % len(dev_batches)]
        state["i"] += 1
        with autocast:
            loss = call(xy[0], xy[1])
        loss.backward()
        opt.step()
        call.zero_grad(set_to_none=True)
        state["loss"] = loss.detach()

    def step_e2e():
        xy = host[state["i"] % len(host)].to(device, non_blocking=True)
        state["i"] += 1
        with autocast:
            loss = call(xy[0], xy[1])
        loss.backward()
        opt.step()
        call.zero_grad(set_to_none=True)
        state["loss_host"] = loss.item()

    try:
        for _ in range(PRIME_STEPS):
            step_device()  # the first call compiles / autotunes
    except Exception as exc:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": f"reference step failed: {type(exc).__name__}: "
                                             f"{str(exc)[:300]}"}))
        if world > 1:
            dist.destroy_process_group()
        return
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms, clocks = time_loop(step_device, args.steps, args.warmup, world, device, sampler)
    loss_after = float(state["loss"].item())
    e2e_ms = None
    if not args.no_e2e:
        e2e_ms, _ = time_loop(step_e2e, args.steps, 2, world, device, None)
    torch.cuda.empty_cache()
    aux = None
    if not args.no_aux:
        aux = guarded_aux(run_aux_reference, args, ref_dion, rank, world, device)
        torch.cuda.empty_cache()
        aux["dion"] = guarded_aux(run_aux_dion_reference, args, ref_dion, rank, world, device)
        torch.cuda.empty_cache()

        def ref_ns(X):   # the reference's Triton driver, as its trainer selects it
            from dion.newton_schulz_triton import newton_schulz_triton

            return newton_schulz_triton(X, epsilon=1e-7)

        aux["newton_schulz"] = guarded_aux(run_aux_ns, ref_ns, device)
    if rank == 0:
        emit(args, "reference", ms, e2e_ms, clocks, 0, world,
             {"final_loss": loss_after,
              "final_loss_after_steps": PRIME_STEPS + args.warmup + args.steps,
              "aux": aux, "model_compiled": compiled})
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
