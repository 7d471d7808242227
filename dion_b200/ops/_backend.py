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
    "foreach_ops": "libdion_foreach.so",
    "select_ops": "libdion_select.so",
    "model_ops": "libdion_model.so",
    "comm_ops": "libdion_comm.so",
    "lowrank_ops": "libdion_lowrank.so",
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
    src = CSRC / f"{stem}.cu"
    if not src.exists():
        return None
    out = LIBDIR / SOURCES[stem]
    if not force and not _needs_build(src, out):
        return None
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build dion_b200 kernels")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", str(out), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


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
_KERNELS_PER_CALL = {"dion_adamw": 2, "dion_ns_iterate2": 0}  # the latter counts itself
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
                f"kernel library {out} is missing; run `python -c 'import __graft_entry__ as g; "
                f"g.build()'` (needs nvcc)"
            )
        h = _CountingLib(ctypes.CDLL(str(out)))
        _loaded[stem] = h
        return h


def available(stem: str) -> bool:
    try:
        lib(stem)
        return True
    except Exception:
        return False
