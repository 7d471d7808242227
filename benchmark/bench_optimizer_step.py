#!/usr/bin/env python
"""Optimizer-step time on the matrix parameters of a GPT of a given size, sharded like FSDP2
(``Shard(0)`` DTensors over all ranks) or replicated like DDP, with random gradients.

    python -m torch.distributed.run --nproc-per-node N benchmark/bench_optimizer_step.py \
        --model 1b --optimizer muon --mode fsdp --impl ours

``--impl``: ``ours`` (fused peer-memory exchange where eligible), ``ours_nccl`` (this package
with the collective exchange), ``reference`` (the unmodified reference package from
``baseline/_ref`` with its Triton kernels).  Prints one JSON line on rank 0: milliseconds per step
(CUDA events, max over ranks) and the Newton-Schulz TFLOP/s it implies.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MODELS = {  # (d_model, n_layer)
    "160m": (768, 12),
    "1b": (2048, 24),
    "3b": (3072, 32),
}


def matrix_shapes(model: str):
    d, L = MODELS[model]
    return [(d, d)] * (4 * L) + [(4 * d, d)] * L + [(d, 4 * d)] * L


def ns_flops(shapes, fraction=1.0, iters=5) -> float:
    total = 0.0
    for m, n in shapes:
        a, b = min(m, n), max(m, n)
        a = a * fraction if fraction < 1 else a
        total += iters * (4 * a * a * b + 2 * a ** 3)
    return total


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1b", choices=list(MODELS))
    ap.add_argument("--optimizer", default="muon", choices=["muon", "normuon", "dion2", "nordion2", "dion"])
    ap.add_argument("--mode", default="fsdp", choices=["fsdp", "ddp", "single"])
    ap.add_argument("--impl", default="ours", choices=["ours", "ours_nccl", "reference"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    args = ap.parse_args()

    if args.impl == "reference":
        if os.path.exists("/usr/bin/g++"):
            os.environ["CXX"], os.environ["CC"] = "/usr/bin/g++", "/usr/bin/gcc"
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import dion as pkg
    else:
        os.environ["DION_B200_FUSED_EXCHANGE"] = "1" if args.impl == "ours" else "0"
        sys.path.insert(0, ROOT)
        import dion_b200 as pkg

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mesh = None
    pg = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    shapes = matrix_shapes(args.model)
    gen = torch.Generator(device=dev).manual_seed(0)

    def make(shape):
        return torch.randn(*shape, device=dev, dtype=torch.float32, generator=gen).to(dtype)

    if args.mode == "fsdp" and world > 1:
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.tensor import DTensor, Shard

        mesh = init_device_mesh("cuda", (world,))

        def shard(shape):
            rows = shape[0] // world
            return DTensor.from_local(make((rows, shape[1])), mesh, [Shard(0)], run_check=False)

        params = [torch.nn.Parameter(shard(s)) for s in shapes]
        grads = [shard(s) for s in shapes]
        dmesh = mesh
    else:
        params = [torch.nn.Parameter(make(s)) for s in shapes]
        grads = [make(s) for s in shapes]
        dmesh = pg if args.mode == "ddp" else None

    ref = args.impl == "reference"
    kw = dict(use_polar_express=False)
    if ref:
        kw["use_triton"] = True
    name = args.optimizer
    fraction = 1.0
    if name == "muon":
        opt = pkg.Muon([dict(params=params)], distributed_mesh=dmesh, lr=0.02, nesterov=True, **kw)
    elif name == "normuon":
        opt = pkg.NorMuon([dict(params=params)], distributed_mesh=dmesh, lr=0.02, nesterov=True, **kw)
    elif name == "dion2":
        fraction = 0.25
        if ref:
            kw["triton_post_ortho"] = True
        opt = pkg.Dion2([dict(params=params)], distributed_mesh=dmesh, lr=0.02, fraction=0.25, **kw)
    elif name == "dion":
        # Legacy low-rank Dion (rank fraction 0.25); replicated over the ranks in ddp mode.
        fraction = 0.0
        dkw = dict(replicate_mesh=pg, replicate_mesh_grad_sync=False) if world > 1 else {}
        opt = pkg.Dion([dict(params=params)], lr=0.02, rank_fraction=0.25, **dkw)
    else:
        fraction = 0.25
        if ref:
            kw["triton_post_ortho"] = True
        opt = pkg.NorDion2([dict(params=params)], distributed_mesh=dmesh, lr=0.02, fraction=0.25, **kw)

    def step():
        for p, g in zip(params, grads):
            p.grad = g
        opt.step()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if not ref:
        from dion_b200.ops.gemm import check_status

        check_status()
    if rank == 0:
        flops = ns_flops(shapes, fraction)
        print(json.dumps({
            "bench": "optimizer_step", "impl": args.impl, "model": args.model,
            "optimizer": name, "mode": args.mode if world > 1 else "single", "n_gpus": world,
            "param_dtype": args.dtype, "ms_per_step": ms,
            "ns_tflops_per_gpu": flops / world / (ms * 1e-3) / 1e12,
            "matrices": len(shapes)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
