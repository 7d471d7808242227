"""Build and load the hand-written sm_100a kernels.

Each ``csrc/*.cu`` file becomes one shared object under ``dion_b200/_lib`` with a plain C ABI,
loaded through ``ctypes``.  The kernels take raw device pointers and a stream handle, so the
libraries have no dependency on the PyTorch headers and compile in seconds.

``build()`` compiles everything with ``nvcc -gencode arch=compute_100a,code=sm_100a``; it works
on a machine without a GPU.  ``lib(name)`` loads a library and raises if it is missing, so that
a GPU run never silently falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import fcntl
import os
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List, Optional

_PKG = Path(__file__).resolve().parent.parent
CSRC = _PKG / "csrc"
LIBDIR = _PKG / "_lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]

# source stem -> library stem
SOURCES = {
    "ns_gemm_sm100": "libdion_ns_gemm.so",
    "ns_gemm2_sm100": "libdion_ns_gemm2.so",
    "ns_persistent_sm100": "libdion_ns_persistent.so",
    "foreach_ops": "libdion_foreach.so",
    "select_ops": "libdion_select.so",
    "model_ops": "libdion_model.so",
    "embedding_ops": "libdion_embedding.so",
    "comm_ops": "libdion_comm.so",
    "lowrank_ops": "libdion_lowrank.so",
    "lowrank_gemm_sm100": "libdion_lowrank_gemm.so",
    "no_alloc": "libdion_noalloc.so",
}

_loaded: Dict[str, "_CountingLib"] = {}
_lock = threading.Lock()


def nvcc_path() -> Optional[str]:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def _needs_build(src: Path, out: Path) -> bool:
    if not out.exists():
        return True
    newest = max([src.stat().st_mtime] + [h.stat().st_mtime for pat in ("*.cuh", "*.h") for h in CSRC.glob(pat)])
    return out.stat().st_mtime < newest


def _compile(stem: str, force: bool, verbose: bool) -> Optional[str]:
    """Compile one library.  Several processes may get here at once (every rank of a multi-GPU
    launch sees a missing or stale library on the first run after a checkout or a header edit),
    so the build happens under an exclusive file lock, the need to build is re-checked once the
    lock is held, and the result is written beside its final place and renamed into it: nobody
    can load a half-written library."""
    src = CSRC / f"{stem}.cu"
    if not src.exists():
        return None
    out = LIBDIR / SOURCES[stem]
    if not force and not _needs_build(src, out):
        return None
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build dion_b200 kernels")
    LIBDIR.mkdir(exist_ok=True)
    with open(LIBDIR / f".{stem}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _needs_build(src, out):
                return None  # another process built it while this one waited
            tmp = LIBDIR / f".{SOURCES[stem]}.{os.getpid()}.tmp"
            cmd = ([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
                   + ["-o", str(tmp), str(src)])
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, out)
            return res.stderr
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build(force: bool = False, verbose: bool = False) -> List[str]:
    """Compile every kernel library that is missing or older than its source."""
    LIBDIR.mkdir(exist_ok=True)
    logs: List[str] = []
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        for log in ex.map(lambda s: _compile(s, force, verbose), list(SOURCES)):
            if log:
                logs.append(log)
    return logs


# Kernels launched per exported entry point (default 1); used for the launch counter.
_KERNELS_PER_CALL = {"dion_adamw": 2, "dion_dion2_post_masked": 2, "dion_aol_rescale": 2,
                     "dion_embedding_bwd": 3, "dion_embedding_sort_bytes": 0,  # own kernels only
                     "dion_ns_iterate2": 0}  # the last one counts itself
_launches = 0


class _CountingLib:
    """Proxy over a ``ctypes.CDLL`` that counts kernel launches made through it."""

    def __init__(self, dll: ctypes.CDLL):
        self._dll = dll
        self._cache = {}

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._dll, name)
            per_call = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=per_call):
                global _launches
                _launches += _n
                return _raw(*args)

            self._cache[name] = fn
        return fn


def add_launches(n: int) -> None:
    """For entry points that launch a data-dependent number of kernels."""
    global _launches
    _launches += n


def launch_count() -> int:
    """Kernel launches issued through this package since the last reset."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def lib(stem: str) -> "_CountingLib":
    """Load (building first if a compiler is present and the source is newer) one library."""
    with _lock:
        h = _loaded.get(stem)
        if h is not None:
            return h
        out = LIBDIR / SOURCES[stem]
        src = CSRC / f"{stem}.cu"
        if src.exists() and nvcc_path() is not None and _needs_build(src, out):
            LIBDIR.mkdir(exist_ok=True)
            _compile(stem, False, False)
        if not out.exists():
            raise RuntimeError(
                f"kernel library {out} is missing; build it with "
                f"`python -c 'from dion_b200.ops import _backend; _backend.build()'` (needs nvcc)"
            )
        dll = ctypes.CDLL(str(out))
        _apply_wait_budget(dll)
        h = _CountingLib(dll)
        _loaded[stem] = h
        return h


_wait_budget_ms: Optional[float] = None


def _apply_wait_budget(dll: ctypes.CDLL) -> None:
    ms = _wait_budget_ms
    if ms is None:
        env = os.environ.get("DION_B200_WAIT_BUDGET_MS")
        ms = float(env) if env else None
    if ms is None:
        return
    setter = getattr(dll, "dion_set_wait_budget_ns", None)
    if setter is None:
        return
    try:
        import torch

        if not torch.cuda.is_available():
            return
        torch.cuda.current_device()  # makes sure the context exists
    except Exception:  # noqa: BLE001
        return
    setter.argtypes = [ctypes.c_ulonglong]
    if setter(ctypes.c_ulonglong(int(ms * 1e6))) != 0:
        raise RuntimeError("could not set the kernels' wait budget")


def set_wait_budget_ms(ms: float) -> None:
    """How long a kernel may wait for a peer GPU (or for one of its own pipeline stages) before
    it records a timeout and unwinds; 2000 by default, ``DION_B200_WAIT_BUDGET_MS`` at start-up.
    The value is written into each library's device variable on the GPU that is current at the
    time (one process drives one GPU) and applies to libraries loaded later as well."""
    global _wait_budget_ms
    _wait_budget_ms = float(ms)
    with _lock:
        for h in _loaded.values():
            _apply_wait_budget(h._dll)


def available(stem: str) -> bool:
    try:
        lib(stem)
        return True
    except Exception:
        return False
