"""The allocation-free entry point, called through its exported C symbol.

For callers that cannot request device memory at call time (frozen memory pools, real-time loops,
plugins inside a runtime that owns the allocator) the library keeps its scratch in an array that
is part of the module.  This test loads the shared object with ``ctypes``, runs the entry point
twice in a row (the second call on a smaller batch, so stale scratch contents would show) and
compares with the regular path, which takes its accumulator from PyTorch's allocator.
Collected last on purpose: a failure here cannot hide other tests under ``-x``."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_MATRICES = 16384


def _load():
    from dion_b200.ops import _backend
    _backend.lib("no_alloc")  # builds it if needed and fails loudly if it cannot
    dll = ctypes.CDLL(str(_backend.LIBDIR / _backend.SOURCES["no_alloc"]))
    fn = dll.dion_frobenius_scale_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float,
                   ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _regular(X, mult, eps):
    from dion_b200.ops import foreach as F
    ss = F.sumsq(X)
    return F.finalize_scale(ss, mult, eps)


def test_no_alloc_entry_point_matches_regular_path_twice():
    fn = _load()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for n, shape in ((48, (192, 768)), (5, (64, 40))):   # second call: fewer, smaller matrices
        X = torch.randn(n, *shape, device="cuda").bfloat16()
        out = torch.full((n,), float("nan"), device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(X.data_ptr(), n, X[0].numel(), 1.02, 1e-7, out.data_ptr(), stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before  # nothing came from the torch allocator
        torch.cuda.synchronize()
        ref = _regular(X, 1.02, 1e-7)
        exact = 1.0 / (X.float().flatten(1).norm(dim=1) * 1.02 + 1e-7)
        assert torch.allclose(out, ref, rtol=1e-5, atol=0)
        assert torch.allclose(out, exact, rtol=1e-4, atol=0)


def test_no_alloc_entry_point_rejects_oversized_batches():
    fn = _load()
    x = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(1, device="cuda")
    rc = fn(x.data_ptr(), MAX_MATRICES + 1, 8, 1.0, 0.0, out.data_ptr(), 0)
    assert rc == -2
    assert fn(None, 1, 8, 1.0, 0.0, out.data_ptr(), 0) == -3
