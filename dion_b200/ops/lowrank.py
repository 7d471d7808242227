"""Low-rank building blocks of the Dion optimizer: power-iteration GEMMs, randomized
Cholesky-QR orthogonalization, column normalization and the rank-r in-place updates
(reference: dion/dion.py:1197-1558).

All functions work on local (already un-wrapped) tensors; the callers own the collectives.
Batched operands are ``[B, rows, cols]``.
"""
from __future__ import annotations

import ctypes
import os
import math
from typing import List, Optional, Tuple

import torch
from torch import Tensor

from . import _backend

_MAX_FACTOR_DIM = 1024  # row limit of the batched factorization kernels (csrc/lowrank_ops.cu)


def _ptr(t: Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


class _LrOperand(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("ld", ctypes.c_longlong), ("stride", ctypes.c_longlong)]


class _LrExtra(ctypes.Structure):
    _fields_ = [("c_table", ctypes.c_void_p), ("d_table", ctypes.c_void_p),
                ("out_mode", ctypes.c_int), ("targets", ctypes.c_longlong * 8),
                ("n_targets", ctypes.c_int), ("slot0", ctypes.c_int),
                ("colsq", ctypes.c_void_p), ("sched", ctypes.c_void_p)]


_sched_pairs: dict = {}


def dynamic_tiles_enabled() -> bool:
    """``DION_B200_DYNAMIC_TILES`` (default on): the low-rank GEMM's CTAs draw tile numbers from a
    device counter instead of taking a fixed share, so a launch that shares the GPU with another
    stream's kernels is not held up by the CTAs that start late."""
    return os.environ.get("DION_B200_DYNAMIC_TILES", "1") != "0"


def _sched_pair(device: torch.device) -> Tensor:
    """Two zeroed ints per (device, stream): launches on one stream follow one another, and the
    kernel rewinds the pair when its last CTA leaves."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    t = _sched_pairs.get(key)
    if t is None:
        t = _sched_pairs[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return t


_pointer_tables: dict = {}


def _address_table(addresses: tuple, device: torch.device) -> Tensor:
    """int64 device tensor holding ``addresses``; cached by value, because building one is a
    blocking host-to-device copy and the state tensors keep their addresses from step to step."""
    key = (addresses, device.index)
    tab = _pointer_tables.get(key)
    if tab is None:
        if len(_pointer_tables) > 512:
            _pointer_tables.clear()
        tab = torch.tensor(addresses, dtype=torch.int64).to(device)
        _pointer_tables[key] = tab
    return tab


def _pointer_table(tensors: List[Tensor]) -> Tensor:
    """int64 device tensor of the data pointers of ``tensors`` (cached by those pointers)."""
    return _address_table(tuple(t.data_ptr() for t in tensors), tensors[0].device)


def _ld_stride3(t: Tensor) -> Tuple[int, int]:
    ld = t.stride(1) if t.size(1) > 1 else max(t.stride(1), t.size(2))
    bs = t.stride(0) if t.size(0) > 1 else t.size(1) * ld
    return ld, bs


def lr_gemm_ok(*ts: Tensor) -> bool:
    """Operands the tensor-core kernel can read in place: CUDA, fp32 or bf16 (all alike), 3-D,
    innermost dimension contiguous, 16-byte aligned base / leading dimension / batch stride."""
    from ..utils.tensors import is_plain_tensor

    dt = ts[0].dtype
    if dt not in (torch.float32, torch.bfloat16):
        return False
    per16 = 16 // ts[0].element_size()
    for t in ts:
        if not (t.is_cuda and t.dtype == dt and t.ndim == 3 and is_plain_tensor(t)):
            return False
        if t.numel() == 0 or t.stride(2) != 1 or t.data_ptr() % 16:
            return False
        ld, bs = _ld_stride3(t)
        if ld % per16 or bs % per16:
            return False
    return True


def split_lo(x: Tensor) -> Tensor:
    """``x - tf32(x)``: the part of an fp32 tensor that a tf32 instruction does not see.  A 3-D
    strided view (a block of rows and columns of every matrix of a batch) is read in place; the
    result is contiguous."""
    if (x.ndim == 3 and not x.is_contiguous() and x.stride(2) == 1 and x.size(2) % 4 == 0
            and x.stride(1) % 4 == 0 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0):
        lo = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        rc = _backend.lib("lowrank_gemm_sm100").dion_split_lo_view(
            _ptr(x), ctypes.c_longlong(x.stride(1)), ctypes.c_longlong(x.stride(0)), _ptr(lo),
            ctypes.c_longlong(x.size(0)), x.size(1), x.size(2), _stream(x.device))
        if rc != 0:
            raise RuntimeError(f"dion_split_lo_view launch failed (code {rc})")
        return lo
    x = x.contiguous()
    lo = torch.empty_like(x)
    rc = _backend.lib("lowrank_gemm_sm100").dion_split_lo(
        _ptr(x), _ptr(lo), ctypes.c_longlong(x.numel()), _stream(x.device))
    if rc != 0:
        raise RuntimeError(f"dion_split_lo launch failed (code {rc})")
    return lo


def lr_gemm(A: Tensor, B: Tensor, *, a_mn: bool = False, b_mn: bool = False,
            out: Optional[Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            out_list: Optional[List[Tensor]] = None, D: Optional[Tensor] = None,
            d_list: Optional[List[Tensor]] = None, alpha: float = 1.0, beta: float = 0.0,
            precise: bool = False, colsq: Optional[Tensor] = None,
            reduce_into: Optional[Tensor] = None, reduce_ld: int = 0,
            broadcast_to: Optional[List[int]] = None, slot0: int = 0, out_ld: int = 0,
            out_stride: int = 0, bn: Optional[int] = None,
            a_lo: Optional[Tensor] = None, b_lo: Optional[Tensor] = None) -> Optional[Tensor]:
    """``out[b] = alpha * A[b] @ op(B[b]) + beta * D[b]`` on the tensor cores (tf32 for fp32
    operands, bf16 otherwise; fp32 accumulation), see csrc/lowrank_gemm_sm100.cu.

    ``A`` is ``[batch, M, K]`` (``a_mn``: ``[batch, K, M]``), ``B`` is ``[batch, N, K]``
    (``b_mn``: ``[batch, K, N]``).  ``out`` / ``D`` are strided batches, ``out_list`` / ``d_list``
    lists of per-matrix tensors (separately allocated weights); ``D`` may be ``out``.
    ``precise`` (fp32 operands): three tf32 products recover fp32-level accuracy (``a_lo``,
    ``b_lo``: the tf32 remainders of ``A`` / ``B`` if the caller has them already; computed once
    when ``B`` is ``A``).
    ``colsq [batch, N]`` (fp32, zeroed by the caller) receives the column sums of squares of the
    result.

    Two ways for the result to leave over NVLink instead of being stored locally (fp32):
    ``reduce_into``: int64 device tensor of one address per matrix (row length ``reduce_ld``);
    the result is added there with ``red.add`` - with each address inside the buffer of the rank
    that owns the matrix, the launches of all ranks together perform a reduce-scatter.
    ``broadcast_to``: raw base addresses of buffers ``[slots, M, N]`` (``out_ld``,
    ``out_stride``) on every rank; matrix ``b`` is stored into slot ``slot0 + b`` of each - an
    all-gather."""
    from . import gemm

    assert lr_gemm_ok(A, B), "operands violate the kernel's layout rules; see lr_gemm_ok()"
    batch = A.size(0)
    M, K = (A.size(2), A.size(1)) if a_mn else (A.size(1), A.size(2))
    N, Kb = (B.size(2), B.size(1)) if b_mn else (B.size(1), B.size(2))
    assert K == Kb and B.size(0) == batch
    dev = A.device
    eb = A.element_size()
    segs = [(A, B)]
    if precise and eb == 4:
        if a_lo is None:
            a_lo = split_lo(A)
        if b_lo is None:
            same = (B.data_ptr() == A.data_ptr() and B.shape == A.shape
                    and B.stride() == A.stride())
            b_lo = a_lo if same else split_lo(B)
        segs = [(A, B), (a_lo, B), (A, b_lo)]
    a_ops = (_LrOperand * 3)()
    b_ops = (_LrOperand * 3)()
    for i, (a, b) in enumerate(segs):
        lda, sa = _ld_stride3(a)
        ldb, sb = _ld_stride3(b)
        a_ops[i] = _LrOperand(a.data_ptr(), lda, sa)
        b_ops[i] = _LrOperand(b.data_ptr(), ldb, sb)
    ex = _LrExtra()
    use_ex = False
    c_ptr, ldc, sc, c_dt = 0, N, M * N, 0
    if reduce_into is not None:
        assert reduce_into.dtype == torch.int64 and reduce_into.numel() >= batch
        ex.c_table = reduce_into.data_ptr()
        ex.out_mode = 1
        ldc = reduce_ld or N
        use_ex = True
    elif broadcast_to is not None:
        for i, addr in enumerate(broadcast_to):
            ex.targets[i] = addr
        ex.n_targets, ex.slot0, ex.out_mode = len(broadcast_to), slot0, 2
        ldc, sc = out_ld or N, out_stride or M * N
        use_ex = True
    elif out_list is not None:
        assert len(out_list) == batch
        ex.c_table = _pointer_table(out_list).data_ptr()
        ldc = out_list[0].stride(0)
        c_dt = 0 if out_list[0].dtype == torch.float32 else 1
        use_ex = True
    else:
        if out is None:
            out = torch.empty((batch, M, N), dtype=out_dtype or A.dtype, device=dev)
        assert out.ndim == 3 and out.stride(2) == 1
        ldc, sc = _ld_stride3(out)
        c_ptr, c_dt = out.data_ptr(), (0 if out.dtype == torch.float32 else 1)
    d_ptr, ldd, sd, d_dt = 0, 0, 0, 0
    if d_list is not None:
        ex.d_table = _pointer_table(d_list).data_ptr()
        ldd = d_list[0].stride(0)
        d_dt = 0 if d_list[0].dtype == torch.float32 else 1
        d_ptr = d_list[0].data_ptr()
        use_ex = True
    elif D is not None:
        ldd, sd = _ld_stride3(D)
        d_ptr, d_dt = D.data_ptr(), (0 if D.dtype == torch.float32 else 1)
    if colsq is not None:
        assert colsq.dtype == torch.float32 and colsq.numel() >= batch * N
        ex.colsq = colsq.data_ptr()
        use_ex = True
    if bn is None:
        bn = 256 if N > 128 else 128
    if dynamic_tiles_enabled() and not torch.cuda.is_current_stream_capturing():
        ex.sched = _sched_pair(dev).data_ptr()
        use_ex = True
    st = gemm.status_tensor(dev)
    rc = _backend.lib("lowrank_gemm_sm100").dion_lr_gemm(
        eb, len(segs), a_ops, b_ops, int(a_mn), int(b_mn),
        ctypes.c_void_p(c_ptr), ctypes.c_longlong(ldc), ctypes.c_longlong(sc), c_dt,
        ctypes.c_void_p(d_ptr), ctypes.c_longlong(ldd), ctypes.c_longlong(sd), d_dt,
        batch, M, N, K, ctypes.c_float(alpha), ctypes.c_float(beta), bn, gemm.sm_count(dev),
        _ptr(st), _stream(dev), ctypes.byref(ex) if use_ex else None)
    if rc != 0:
        raise RuntimeError(f"dion_lr_gemm launch failed (code {rc})")
    return out


def triu_inverse(U: Tensor) -> Tensor:
    """Inverse of every upper-triangular ``U[b]`` (``[B, r, r]`` fp32).  The kernel works on
    32 x 32 blocks; other sizes are padded with the identity."""
    r = U.size(-1)
    if U.is_cuda and U.dtype == torch.float32 and U.ndim == 3 and r <= _MAX_FACTOR_DIM:
        rp = (r + 31) // 32 * 32
        if rp != r:
            Uc = torch.eye(rp, dtype=U.dtype, device=U.device).repeat(U.size(0), 1, 1)
            Uc[:, :r, :r] = U
        else:
            Uc = U.contiguous()
        X = torch.empty_like(Uc)
        rc = _backend.lib("lowrank_ops").dion_triu_inverse(
            _ptr(Uc), _ptr(X), Uc.size(0), rp, _stream(Uc.device))
        if rc != 0:
            raise RuntimeError(f"dion_triu_inverse launch failed (code {rc})")
        return X if rp == r else X[:, :r, :r].contiguous()
    eye = torch.eye(r, dtype=U.dtype, device=U.device).expand_as(U)
    return torch.linalg.solve_triangular(U, eye, upper=True)


def sketch_rows(r: int, oversample: float) -> int:
    """Number of sketch rows: ``oversample * r`` rounded up to a multiple of 128."""
    return int(math.ceil(oversample * r / 128.0) * 128)


_sketch_calls = 0


def random_sketch(batch: int, k: int, m: int, dtype: torch.dtype, device: torch.device,
                  generator: Optional[torch.Generator] = None) -> Tensor:
    """Gaussian sketch ``S ~ N(0, 1/k)`` of shape ``[batch, k, m]``.  On a GPU the values are a
    pure function of the generator's seed and the element index (Philox counter kernel of this
    package): replicas that derive the same seed draw the same sketch.  Without a generator the
    seed is the framework's default seed combined with a call counter."""
    S = torch.empty((batch, k, m), dtype=dtype, device=device)
    std = math.sqrt(1.0 / k)
    if S.is_cuda and dtype in (torch.float32, torch.bfloat16) and S.numel():
        global _sketch_calls
        if generator is not None:
            seed = generator.initial_seed()
        else:
            _sketch_calls += 1
            seed = (torch.initial_seed() * 1000003 + _sketch_calls) % (1 << 63)
        rc = _backend.lib("lowrank_ops").dion_philox_normal(
            _ptr(S), ctypes.c_longlong(S.numel()), ctypes.c_ulonglong(seed & ((1 << 64) - 1)),
            ctypes.c_float(std), 0 if dtype == torch.float32 else 1, _stream(device))
        if rc != 0:
            raise RuntimeError(f"dion_philox_normal launch failed (code {rc})")
        return S
    S.normal_(std=std, generator=generator)
    return S


def householder_q(P: Tensor) -> Tensor:
    """Orthonormal factor of a reduced QR in fp32 (used when rows <= cols)."""
    Q, _ = torch.linalg.qr(P.to(torch.float32), mode="reduced")
    return Q


_QR_PANEL = 32
_QR_PANEL_MAX_ROWS = 1580      # shared memory of the panel kernel: (rows * 33 + ...) * 4 bytes
_QR_BLOCKED_MIN_COLS = 256     # below this the single-kernel form wins (five launches per panel)


def blocked_qr_enabled() -> bool:
    return os.environ.get("DION_B200_BLOCKED_QR", "1") != "0"


def _qr_r_blocked(A32: Tensor) -> Tensor:
    """Blocked Householder QR of a private fp32 batch ``[B, k, r]`` (overwritten): per 32-column
    panel one kernel factors the panel in shared memory (one CTA per matrix) and emits the
    reflectors ``V`` and ``V T^T`` of the compact WY form; the columns to the right are then
    updated by two tensor-core products over the whole batch, ``W = V^T A_right`` and
    ``A_right -= (V T^T) W`` (split operands: the factor is only as good as these)."""
    B, k, r = A32.shape
    dev = A32.device
    V, VT, Vlo, VTlo = torch.empty((4, B, k, _QR_PANEL), dtype=torch.float32, device=dev).unbind(0)
    W = torch.empty((B, _QR_PANEL, r), dtype=torch.float32, device=dev)
    lib = _backend.lib("lowrank_ops")
    for j in range(0, r, _QR_PANEL):
        rc = lib.dion_qr_panel(_ptr(A32), ctypes.c_longlong(k * r), r, B, k, j, _ptr(V), _ptr(VT),
                               _ptr(Vlo), _ptr(VTlo), _stream(dev))
        if rc != 0:
            raise RuntimeError(f"dion_qr_panel launch failed (code {rc})")
        nt = r - j - _QR_PANEL
        if nt <= 0:
            break
        right = A32[:, j:, j + _QR_PANEL:]
        Wv = W[:, :, :nt]
        lr_gemm(V[:, j:, :], right, a_mn=True, b_mn=True, out=Wv, precise=True,
                a_lo=Vlo[:, j:, :])
        lr_gemm(VT[:, j:, :], Wv, b_mn=True, D=right, out=right, alpha=-1.0, beta=1.0,
                precise=True, a_lo=VTlo[:, j:, :])
    return torch.triu(A32[:, :r, :r])


def qr_r_factor(A: Tensor, overwrite: bool = False) -> Tensor:
    """Upper-triangular factor of every ``A[b]`` (``[B, k, r]``, ``k >= r``) in fp32.  On a GPU
    all matrices of the batch are factored together: blocked Householder with the trailing
    updates on the tensor cores when ``r`` is a multiple of 32 (at least 256), else one kernel
    with one CTA per matrix (up to 1024 rows).  The sign of a row of ``R`` may differ from
    LAPACK's.  ``overwrite``: ``A`` is a temporary of the caller and may be destroyed."""
    A32 = A.to(torch.float32)
    if A32.is_cuda and A32.ndim == 3 and A32.size(-1) <= A32.size(-2):
        B, k, r = A32.shape
        if (blocked_qr_enabled() and r % _QR_PANEL == 0 and r >= _QR_BLOCKED_MIN_COLS
                and k <= _QR_PANEL_MAX_ROWS and k % 4 == 0 and B > 0):
            if not A32.is_contiguous():
                A32 = A32.contiguous()
            elif A32.data_ptr() == A.data_ptr() and not overwrite:
                A32 = A32.clone()
            return _qr_r_blocked(A32)
        if k <= _MAX_FACTOR_DIM:
            A32 = A32.contiguous()
            V = torch.empty((B, r, k), dtype=torch.float32, device=A32.device)
            tau = torch.empty((B, r), dtype=torch.float32, device=A32.device)
            R = torch.empty((B, r, r), dtype=torch.float32, device=A32.device)
            rc = _backend.lib("lowrank_ops").dion_qr_r_factor(
                _ptr(A32), _ptr(V), _ptr(tau), _ptr(R), B, k, r, _stream(A32.device))
            if rc != 0:
                raise RuntimeError(f"dion_qr_r_factor launch failed (code {rc})")
            return R
    return torch.linalg.qr(A32, mode="r")[1]


def cholesky_upper(G: Tensor) -> Tensor:
    """Upper Cholesky factor without raising on failure (NaNs propagate and are handled by
    :func:`fix_all_zero_or_nan`).  GPU batches of fp32 matrices go to one kernel."""
    if (G.is_cuda and G.dtype == torch.float32 and G.ndim == 3
            and G.size(-1) == G.size(-2) <= _MAX_FACTOR_DIM):
        Gc = G.contiguous()
        U = torch.empty_like(Gc)
        rc = _backend.lib("lowrank_ops").dion_cholesky_upper(
            _ptr(Gc), _ptr(U), Gc.size(0), Gc.size(-1), _stream(Gc.device))
        if rc != 0:
            raise RuntimeError(f"dion_cholesky_upper launch failed (code {rc})")
        return U
    return torch.linalg.cholesky_ex(G, upper=True)[0]


def _solve_on_kernel(R: Tensor, P: Tensor) -> bool:
    return (P.is_cuda and P.dtype == torch.float32 and R.dtype == torch.float32 and P.ndim == 3
            and R.size(-1) <= _MAX_FACTOR_DIM and lr_gemm_ok(P, R.contiguous()))


def right_solve_upper(R: Tensor, P: Tensor, p_lo: Optional[Tensor] = None,
                      out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """``P @ R^-1`` for upper-triangular ``R`` (``[B, r, r]`` fp32) and ``P [B, m, r]`` fp32.  On
    a GPU: ``R^-1`` from the batched inversion kernel, then a tensor-core product with split
    operands (fp32-level accuracy; ``p_lo``: the tf32 remainder of ``P`` if already known; the
    epilogue rounds to ``out_dtype``); elsewhere a triangular solve."""
    if _solve_on_kernel(R, P):
        return lr_gemm(P, triu_inverse(R), b_mn=True, precise=True, a_lo=p_lo,
                       out_dtype=out_dtype)
    X = torch.linalg.solve_triangular(R, P, upper=True, left=False)
    return X if out_dtype is None else X.to(out_dtype)


def gram(P: Tensor, p_lo: Optional[Tensor] = None) -> Tensor:
    """``P^T P`` in fp32 for ``P [B, m, r]`` fp32 (tensor cores with split operands on a GPU)."""
    if P.is_cuda and P.dtype == torch.float32 and P.ndim == 3 and lr_gemm_ok(P):
        return lr_gemm(P, P, a_mn=True, b_mn=True, precise=True, a_lo=p_lo, b_lo=p_lo)
    return P.mT @ P


def sketch_product(S: Tensor, P: Tensor) -> Tensor:
    """``S P`` for the sketch ``S [B, k, m]`` and ``P [B, m, r]`` (same dtype), fp32 result."""
    if lr_gemm_ok(S, P):
        return lr_gemm(S, P, b_mn=True, out_dtype=torch.float32)
    return (S @ P).to(torch.float32)


def orthogonalize(P: Tensor, oversample: float = 1.25,
                  generator: Optional[torch.Generator] = None,
                  sketch: Optional[Tensor] = None) -> Tensor:
    """Orthonormalize the columns of every ``P[b]`` (``[B, m, r]``), result in ``P.dtype``.

    ``m <= r``: Householder QR.  Otherwise randomized Cholesky-QR: ``R1 = qr(S P).R``,
    ``P <- P R1^-1`` (well conditioned), then ``R2 = chol(P^T P)``, ``P <- P R2^-1``
    (reference: dion/dion.py:1265-1305).  On a GPU every product runs on this package's
    tensor-core kernel and the triangular solves are products with explicitly inverted
    factors."""
    assert P.ndim >= 3, "expected a batch dimension"
    dtype = P.dtype
    m, r = P.shape[-2], P.shape[-1]
    if m <= r:
        return householder_q(P).to(dtype).contiguous()
    if sketch is None:
        sketch = random_sketch(P.size(0), sketch_rows(r, oversample), m, dtype, P.device, generator)
    R1 = qr_r_factor(sketch_product(sketch, P), overwrite=True)
    P32 = right_solve_upper(R1, P.to(torch.float32))
    # the tf32 remainder of the preconditioned P serves the Gram product and the second solve
    lo = split_lo(P32) if (P32.is_cuda and lr_gemm_ok(P32)) else None
    R2 = cholesky_upper(gram(P32, lo))
    return right_solve_upper(R2, P32, lo, out_dtype=dtype).contiguous()


def fix_all_zero_or_nan(P: Tensor, R: Tensor, Q_init: Tensor, B: Optional[Tensor],
                        sum_sq: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Branch-free guard: where the (local) momentum ``B[b]`` is entirely zero, return ``P = 0``
    and ``R = Q_init``; elsewhere replace NaNs by zero.  Shards are judged independently so no
    communication is needed.  "Entirely zero" is read off the max-norm (one pass over ``B`` with
    no full-size temporary; a NaN in ``B`` makes the norm NaN, which is not zero, exactly as an
    element-wise comparison would decide).  ``sum_sq`` (one value per matrix, e.g. the sum of
    squares the momentum kernel accumulates anyway) replaces the pass over ``B``: it is zero, NaN
    or positive exactly when the max-norm is."""
    if sum_sq is not None:
        zero = (sum_sq.reshape(-1, 1, 1) == 0)
    else:
        zero = (torch.linalg.vector_norm(B, ord=float("inf"), dim=(-2, -1), keepdim=True) == 0)
    keep = ~zero
    return P.nan_to_num() * keep, R.nan_to_num() * keep + Q_init * zero


def _factor_kernel_ok(*ts: Tensor) -> bool:
    from ..utils.tensors import is_plain_tensor

    dt = ts[0].dtype
    return dt in (torch.float32, torch.bfloat16) and all(
        t.is_cuda and t.dtype == dt and t.ndim == 3 and t.is_contiguous() and is_plain_tensor(t)
        and t.numel() for t in ts)


def fix_factors_(P: Tensor, R: Tensor, Q_init: Tensor, sum_sq: Tensor) -> Tensor:
    """In-place form of :func:`fix_all_zero_or_nan` for GPU batches, one launch per factor:
    where ``sum_sq[b] == 0`` (all-zero momentum) ``P[b] = 0`` and ``R[b] = Q_init[b]``, elsewhere
    NaN / infinities are replaced as ``nan_to_num`` does.  Returns the column sums of squares of
    the cleaned ``R`` (``[B, 1, r]`` fp32), which the second launch accumulates on the way."""
    assert _factor_kernel_ok(P, R, Q_init) and sum_sq.dtype == torch.float32
    lib = _backend.lib("lowrank_ops")
    dt = 0 if P.dtype == torch.float32 else 1
    B = P.size(0)
    rc = lib.dion_fix_factor(_ptr(P), ctypes.c_void_p(0), _ptr(sum_sq), B, P.size(1), P.size(2),
                             ctypes.c_void_p(0), dt, _stream(P.device))
    colsq = torch.zeros((B, 1, R.size(2)), dtype=torch.float32, device=R.device)
    rc |= lib.dion_fix_factor(_ptr(R), _ptr(Q_init), _ptr(sum_sq), B, R.size(1), R.size(2),
                              _ptr(colsq), dt, _stream(R.device))
    if rc != 0:
        raise RuntimeError("dion_fix_factor launch failed")
    return colsq


def normalize_columns_into(R: Tensor, colsq: Tensor, epsilon: float,
                           q_states: Optional[List[Tensor]] = None) -> Tensor:
    """``Q = R / (sqrt(colsq) + eps)`` in one launch; returns the stack ``Q`` (dtype of ``R``)
    and, when ``q_states`` is given (one contiguous ``[rows, r]`` tensor per matrix, or None to
    skip), also writes each matrix into its state tensor (fp32 or bf16)."""
    assert _factor_kernel_ok(R) and colsq.dtype == torch.float32
    B, rows, cols = R.shape
    Q = torch.empty_like(R)
    q_ptrs, q_dt = 0, 0
    if q_states is not None:
        live = [q for q in q_states if q is not None]
        q_dt = 0 if (live and live[0].dtype == torch.float32) else 1
        addrs = tuple([q.data_ptr() if q is not None else 0 for q in q_states]
                      + [0] * (B - len(q_states)))
        q_ptrs = _address_table(addrs, R.device).data_ptr()
    rc = _backend.lib("lowrank_ops").dion_normalize_q(
        _ptr(R), _ptr(colsq), ctypes.c_float(float(epsilon)), _ptr(Q), ctypes.c_void_p(q_ptrs),
        q_dt, B, rows, cols, 0 if R.dtype == torch.float32 else 1, _stream(R.device))
    if rc != 0:
        raise RuntimeError("dion_normalize_q launch failed")
    return Q


def local_column_sum_sq(X: Tensor) -> Tensor:
    """Per-column sum of squares in fp32, shape ``[..., 1, cols]``."""
    return X.to(torch.float32).square().sum(dim=-2, keepdim=True)


def column_normalize(X: Tensor, full_column_sum_sq: Optional[Tensor] = None,
                     epsilon: float = 1e-8) -> Tensor:
    """``X / (||X||_col + eps)`` computed in fp32; a row-sharded ``X`` passes the all-reduced
    column sums of squares."""
    X32 = X.to(torch.float32)
    ss = X32.square().sum(dim=-2, keepdim=True) if full_column_sum_sq is None \
        else full_column_sum_sq.to(torch.float32)
    return (X32 / (ss.sqrt() + epsilon)).to(X.dtype)


def foreach_baddbmm_(X: List[Tensor], A: Tensor, B: Tensor, alpha=1.0, beta=1.0,
                     transpose: bool = False) -> None:
    """``X[i] = beta*X[i] + alpha*(A[i] @ B[i]^T)`` (or ``B[i] @ A[i]^T`` when ``transpose``).
    One fused GEMM-with-epilogue launch for all matrices on a GPU (the rank-r product is never
    materialized at full size and every ``X[i]`` is read and written once, in place, by the
    epilogue of the tensor-core kernel); one ``addmm`` per matrix elsewhere."""
    assert A.size(0) == B.size(0) == len(X)
    if isinstance(alpha, Tensor) or isinstance(beta, Tensor):
        # Device-resident scalars (no host read): scale with multi-tensor ops instead.
        upd = (B @ A.mT) if transpose else (A @ B.mT)
        upd = torch._foreach_mul(list(upd.unbind(0)), alpha)
        torch._foreach_mul_(X, beta)
        torch._foreach_add_(X, [u.to(x.dtype) for u, x in zip(upd, X)])
        return
    alpha, beta = float(alpha), float(beta)
    a3, b3 = (B, A) if transpose else (A, B)
    if _rank_update_ok(X, a3, b3):
        lr_gemm(a3, b3, out_list=X, d_list=X, alpha=alpha, beta=beta)
        return
    for i, x in enumerate(X):
        a, b = a3[i], b3[i]
        if a.dtype != x.dtype:
            a, b = a.to(x.dtype), b.to(x.dtype)
        torch.addmm(x, a, b.mT, beta=beta, alpha=alpha, out=x)


def _rank_update_ok(X: List[Tensor], a3: Tensor, b3: Tensor) -> bool:
    from ..utils.tensors import is_plain_tensor

    if not (a3.dtype == b3.dtype and lr_gemm_ok(a3, b3)):
        return False
    x0 = X[0]
    if x0.dtype not in (torch.float32, torch.bfloat16) or x0.ndim != 2:
        return False
    for x in X:
        if not (is_plain_tensor(x) and x.is_cuda and x.dtype == x0.dtype and x.stride(1) == 1
                and x.stride(0) == x0.stride(0) and x.shape == x0.shape):
            return False
    return True


def rank_update_stack_(X3: Tensor, A: Tensor, B: Tensor, alpha: float, beta: float,
                       transpose: bool = False) -> None:
    """As :func:`foreach_baddbmm_` for matrices stored as one stack ``X3 [B, m, n]``."""
    a3, b3 = (B, A) if transpose else (A, B)
    if a3.dtype == b3.dtype and lr_gemm_ok(a3, b3) and X3.is_cuda and X3.stride(2) == 1 \
            and X3.dtype in (torch.float32, torch.bfloat16):
        lr_gemm(a3, b3, out=X3, D=X3, alpha=float(alpha), beta=float(beta))
        return
    foreach_baddbmm_(list(X3.unbind(0)), A, B, alpha=alpha, beta=beta, transpose=transpose)


def power_iteration_p(M3: Tensor, Q3: Tensor, transposed: bool = False,
                      reduce_into: Optional[Tensor] = None, alpha: float = 1.0
                      ) -> Optional[Tensor]:
    """``P = Mt Q`` with ``Mt = M^T`` when ``transposed`` else ``M``, for the stack ``M3
    [B, m, n]`` in its row-major storage and ``Q3 [B, n or m, r]`` (reference:
    dion/dion.py:797-798).  On a GPU both operands are read in place by the tensor-core kernel
    (``M^T`` as an MN-major operand, ``Q`` as a ``[K, N]`` operand): no transposed copy.
    ``reduce_into`` / ``alpha``: the product (scaled) leaves through ``red.add`` instead of being
    returned, see :func:`lr_gemm`."""
    if Q3.dtype != M3.dtype:
        Q3 = Q3.to(M3.dtype)
    if reduce_into is not None:
        lr_gemm(M3, Q3, a_mn=transposed, b_mn=True, reduce_into=reduce_into, alpha=alpha)
        return None
    if lr_gemm_ok(M3, Q3):
        return lr_gemm(M3, Q3, a_mn=transposed, b_mn=True, alpha=alpha)
    return ((M3.mT if transposed else M3) @ Q3) * alpha if alpha != 1.0 else \
        (M3.mT if transposed else M3) @ Q3


def power_iteration_r(M3: Tensor, P: Tensor, transposed: bool = False,
                      colsq: Optional[Tensor] = None, reduce_into: Optional[Tensor] = None,
                      alpha: float = 1.0) -> Optional[Tensor]:
    """``R = Mt^T P`` (reference: dion/dion.py:836); ``colsq``, ``reduce_into`` and ``alpha`` as
    in :func:`lr_gemm`."""
    if P.dtype != M3.dtype:
        P = P.to(M3.dtype)
    if reduce_into is not None:
        lr_gemm(M3, P, a_mn=not transposed, b_mn=True, reduce_into=reduce_into, alpha=alpha)
        return None
    if lr_gemm_ok(M3, P):
        return lr_gemm(M3, P, a_mn=not transposed, b_mn=True, colsq=colsq)
    R = (M3 if transposed else M3.mT) @ P
    if colsq is not None:
        colsq.view(R.size(0), R.size(-1)).add_(R.to(torch.float32).square().sum(dim=-2))
    return R


def stack_for_power_iteration(M: List[Tensor], Q: List[Tensor], transposed: bool):
    """``(M_batch, Q_batch)`` with ``M_batch[i] = M[i]^T`` when ``transposed``; ``Q`` is cast to
    the momentum dtype.  (List form kept for callers that hold separate tensors; the optimizer
    keeps its momentum as one stack and passes ``transposed`` to the functions above.)"""
    Mb = torch.stack([m.mT for m in M]) if transposed else torch.stack(M)
    return Mb, torch.stack(Q).to(Mb.dtype)
