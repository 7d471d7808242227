"""Helpers to run a function on several ranks as child processes (gloo on CPU, NCCL on GPUs)."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        if result_dir is not None and out is not None:
            torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
        dist.barrier()
    except Exception:
        traceback.print_exc()
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world, backend="gloo", args=(), result_dir=None):
    """Runs ``fn(rank, world, *args)`` on ``world`` processes; results are saved per rank."""
    mp.spawn(_entry, args=(world, free_port(), backend, fn, args, result_dir), nprocs=world,
             join=True)
    if result_dir is None:
        return None
    return [torch.load(os.path.join(result_dir, f"rank{r}.pt")) for r in range(world)
            if os.path.exists(os.path.join(result_dir, f"rank{r}.pt"))]
