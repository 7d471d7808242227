"""Low-rank building blocks of the Dion optimizer: power-iteration GEMMs, randomized
Cholesky-QR orthogonalization, column normalization and the rank-r in-place updates
(reference: dion/dion.py:1197-1558).

All functions work on local (already un-wrapped) tensors; the callers own the collectives.
Batched operands are ``[B, rows, cols]``.
"""
from __future__ import annotations

import ctypes
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


def sketch_rows(r: int, oversample: float) -> int:
    """Number of sketch rows: ``oversample * r`` rounded up to a multiple of 128."""
    return int(math.ceil(oversample * r / 128.0) * 128)


def random_sketch(batch: int, k: int, m: int, dtype: torch.dtype, device: torch.device,
                  generator: Optional[torch.Generator] = None) -> Tensor:
    """Gaussian sketch ``S ~ N(0, 1/k)`` of shape ``[batch, k, m]``."""
    S = torch.empty((batch, k, m), dtype=dtype, device=device)
    S.normal_(std=math.sqrt(1.0 / k), generator=generator)
    return S


def householder_q(P: Tensor) -> Tensor:
    """Orthonormal factor of a reduced QR in fp32 (used when rows <= cols)."""
    Q, _ = torch.linalg.qr(P.to(torch.float32), mode="reduced")
    return Q


def qr_r_factor(A: Tensor) -> Tensor:
    """Upper-triangular factor of every ``A[b]`` (``[B, k, r]``, ``k >= r``) in fp32.  On a GPU
    all matrices of the batch are factored at once by one kernel (Householder reflections, one
    CTA per matrix); the sign of a row of ``R`` may differ from LAPACK's."""
    A32 = A.to(torch.float32)
    if A32.is_cuda and A32.ndim == 3 and A32.size(-1) <= A32.size(-2) <= _MAX_FACTOR_DIM:
        A32 = A32.contiguous()
        B, k, r = A32.shape
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


def right_solve_upper(R: Tensor, P: Tensor) -> Tensor:
    """``P @ R^-1`` for upper-triangular ``R``."""
    return torch.linalg.solve_triangular(R, P, upper=True, left=False)


def orthogonalize(P: Tensor, oversample: float = 1.25,
                  generator: Optional[torch.Generator] = None,
                  sketch: Optional[Tensor] = None) -> Tensor:
    """Orthonormalize the columns of every ``P[b]`` (``[B, m, r]``), result in ``P.dtype``.

    ``m <= r``: Householder QR.  Otherwise randomized Cholesky-QR: ``R1 = qr(S P).R``,
    ``P <- P R1^-1`` (well conditioned), then ``R2 = chol(P^T P)``, ``P <- P R2^-1``."""
    assert P.ndim >= 3, "expected a batch dimension"
    dtype = P.dtype
    m, r = P.shape[-2], P.shape[-1]
    if m <= r:
        return householder_q(P).to(dtype).contiguous()
    if sketch is None:
        sketch = random_sketch(P.size(0), sketch_rows(r, oversample), m, dtype, P.device, generator)
    R1 = qr_r_factor(sketch @ P)
    P32 = right_solve_upper(R1, P.to(torch.float32))
    R2 = cholesky_upper(P32.mT @ P32)
    return right_solve_upper(R2, P32).to(dtype).contiguous()


def fix_all_zero_or_nan(P: Tensor, R: Tensor, Q_init: Tensor, B: Tensor) -> Tuple[Tensor, Tensor]:
    """Branch-free guard: where the (local) momentum ``B[b]`` is entirely zero, return ``P = 0``
    and ``R = Q_init``; elsewhere replace NaNs by zero.  Shards are judged independently so no
    communication is needed.  "Entirely zero" is read off the max-norm (one pass over ``B`` with
    no full-size temporary; a NaN in ``B`` makes the norm NaN, which is not zero, exactly as an
    element-wise comparison would decide)."""
    zero = (torch.linalg.vector_norm(B, ord=float("inf"), dim=(-2, -1), keepdim=True) == 0)
    keep = ~zero
    return P.nan_to_num() * keep, R.nan_to_num() * keep + Q_init * zero


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
    One fused GEMM-with-epilogue per matrix: the rank-r product is never materialized at full
    size and every ``X[i]`` is read and written once."""
    assert A.size(0) == B.size(0) == len(X)
    if isinstance(alpha, Tensor) or isinstance(beta, Tensor):
        # Device-resident scalars (no host read): scale with multi-tensor ops instead.
        upd = (B @ A.mT) if transpose else (A @ B.mT)
        upd = torch._foreach_mul(list(upd.unbind(0)), alpha)
        torch._foreach_mul_(X, beta)
        torch._foreach_add_(X, [u.to(x.dtype) for u, x in zip(upd, X)])
        return
    alpha, beta = float(alpha), float(beta)
    for i, x in enumerate(X):
        a, b = (B[i], A[i]) if transpose else (A[i], B[i])
        if a.dtype != x.dtype:
            a, b = a.to(x.dtype), b.to(x.dtype)
        torch.addmm(x, a, b.mT, beta=beta, alpha=alpha, out=x)


def _tcgen05_ok(A: Tensor, B: Tensor) -> bool:
    from . import gemm
    from ..utils.tensors import is_plain_tensor

    return (A.is_cuda and A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16
            and A.ndim == 3 and B.ndim == 3 and is_plain_tensor(A) and is_plain_tensor(B)
            and A.is_contiguous() and B.is_contiguous() and gemm.supported(A, B)
            and B.size(-1) % 8 == 0 and min(A.shape[-2:]) >= 64 and B.size(-1) >= 64)


def power_iteration_p(Mb: Tensor, Qb: Tensor) -> Tensor:
    """``P = M Q`` for batches ``Mb [B, m, n]``, ``Qb [B, n, r]`` (reference: dion/dion.py:798).
    bf16 batches on a GPU run on this package's tcgen05 GEMM (``Q`` read as a [K, N] operand),
    anything else through ``torch.bmm``."""
    if _tcgen05_ok(Mb, Qb):
        from . import gemm
        return gemm.ns_gemm(Mb, Qb, b_is_kn=True)
    return Mb @ Qb


def power_iteration_r(Mb: Tensor, P: Tensor) -> Tensor:
    """``R = M^T P`` for ``Mb [B, m, n]``, ``P [B, m, r]`` (reference: dion/dion.py:836) without
    a transposed copy of ``M``: both operands are read K-outermost."""
    if _tcgen05_ok(Mb, P):
        from . import gemm
        return gemm.ns_gemm(Mb, P, a_is_km=True, b_is_kn=True)
    return Mb.mT @ P


def stack_for_power_iteration(M: List[Tensor], Q: List[Tensor], transposed: bool):
    """``(M_batch, Q_batch)`` with ``M_batch[i] = M[i]^T`` when ``transposed``; ``Q`` is cast to
    the momentum dtype."""
    Mb = torch.stack([m.mT for m in M]) if transposed else torch.stack(M)
    return Mb, torch.stack(Q).to(Mb.dtype)
