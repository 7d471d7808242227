#!/usr/bin/env python
"""All-reduce inside symmetric memory (NVLS multimem or plain peer access) against NCCL.

    python -m torch.distributed.run --nproc-per-node N benchmark/bench_allreduce.py

Prints one JSON line per size on rank 0: microseconds per call (CUDA events, max over ranks) and
bus bandwidth ``2 (N-1)/N * bytes / time``.  The symmetric numbers are for the zero-copy form
(data already in the buffer), NCCL's for an in-place all-reduce of an ordinary tensor.
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def timed(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e3  # us


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from dion_b200.ops.gemm import check_status
    from dion_b200.parallel import symm

    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = [1 << 16, 1 << 20, 1 << 24, 1 << 26, 1 << 28]
    modes = {}
    for name, env in (("multimem", "1"), ("peer", "0")):
        os.environ["DION_B200_NVLS"] = env
        modes[name] = symm.SymmetricAllReduce(dist.group.WORLD, max(sizes), dev)
    for nbytes in sizes:
        n = nbytes // 4
        x = torch.randn(n, device=dev)
        row = {"bytes": nbytes, "n_gpus": world}
        us = timed(lambda: dist.all_reduce(x))
        row["nccl_us"] = round(us, 1)
        row["nccl_busbw_gbs"] = round(2 * (world - 1) / world * nbytes / us / 1e3, 1)
        for name, red in modes.items():
            if name == "multimem" and not red.uses_multimem:
                row["multimem"] = "no multicast support"
                continue
            us = timed(lambda: red.all_reduce_(n, torch.float32, "sum"))
            row[f"{name}_us"] = round(us, 1)
            row[f"{name}_busbw_gbs"] = round(2 * (world - 1) / world * nbytes / us / 1e3, 1)
        check_status()
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
