"""Newton-Schulz style orthogonalization: coefficient tables and drivers.

Every driver has the signature ``func(G, epsilon) -> Tensor`` used throughout the optimizers
(reference contract: dion/muon.py:47-48).  Inputs may be ``[m, n]`` or batched ``[B, m, n]``;
the result is bf16 with the input's shape.

On CUDA the iterations run on the tcgen05 GEMM kernel (``ops/gemm.py``): the Gram matrix
``A = X X^T`` and the polynomial ``B = b*A + c*A^2`` are computed as symmetric half-work GEMMs
and ``X' = a*X + B X`` reads ``X`` as an MN-major operand, so no transposed copies are made.  The
Frobenius normalization is folded into the first iteration's epilogue scalars instead of being a
separate pass over ``X``.  On CPU (tests, gloo runs) the same math runs in plain PyTorch.

Variants (reference: dion/muon.py:351-378, dion/muon_reference.py:11-27,
dion/polar_express.py:10-85, dion/newton_schulz_triton.py:495-628, and the optional external
Gram-NS package selected at dion/megabatch_base.py:77-94):
  * ``newton_schulz_quintic``   five tuned quintic steps
  * ``newton_schulz_classic``   fixed (3.4445, -4.7750, 2.0315) repeated ``steps`` times
  * ``polar_express``           five Polar-Express steps, input scaled by 1/(1.02*||X||)
  * ``newton_schulz_aol``       four steps after AOL rescaling
  * ``gram_newton_schulz``      iterates on the small Gram matrix, re-materializing X at resets
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import torch
from torch import Tensor

from ..utils import trace
from ..utils.tensors import unwrap
from . import foreach as F
from . import gemm

Coeffs = Sequence[Tuple[float, float, float]]

QUINTIC_COEFFS: Coeffs = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)
CLASSIC_COEFF = (3.4445, -4.7750, 2.0315)
POLAR_EXPRESS_COEFFS: Coeffs = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)
AOL_COEFFS: Coeffs = (
    (4.6051, -9.6552, 5.6769),
    (4.7505, -6.0861, 2.1790),
    (2.7763, -2.3190, 0.5523),
    (2.4231, -2.2861, 0.8193),
)


def _eps(epsilon) -> float:
    if epsilon is None:
        return 1e-7
    return float(epsilon)


# ------------------------------------------------------------------------------------------------
# PyTorch implementations (CPU path and oracle)
# ------------------------------------------------------------------------------------------------
def _iterate_torch(X: Tensor, coeffs: Coeffs) -> Tensor:
    for a, b, c in coeffs:
        A = X @ X.mT
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X


def _ns_torch(G: Tensor, coeffs: Coeffs, norm_mult: float, epsilon: float) -> Tensor:
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * norm_mult + epsilon)
    X = _iterate_torch(X, coeffs)
    if tall:
        X = X.mT
    return X


def _aol_torch(G: Tensor, epsilon: float) -> Tensor:
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    A = X @ X.mT
    s = torch.rsqrt(A.abs().sum(dim=-1).clamp_min(epsilon))
    X = X * s.unsqueeze(-1)
    A = A * s.unsqueeze(-1) * s.unsqueeze(-2)
    a, b, c = AOL_COEFFS[0]
    B = b * A + c * (A @ A)
    X = a * X + B @ X
    X = _iterate_torch(X, AOL_COEFFS[1:])
    if tall:
        X = X.mT
    return X


def _gram_torch(G: Tensor, coeffs: Coeffs, norm_mult: float, epsilon: float,
                resets: Sequence[int]) -> Tensor:
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * norm_mult + epsilon)
    m = X.size(-2)
    eye = torch.eye(m, dtype=X.dtype, device=X.device)
    R = X @ X.mT
    Q: Optional[Tensor] = None
    for it, (a, b, c) in enumerate(coeffs):
        if it in resets and Q is not None:
            X = Q @ X
            R = X @ X.mT
            Q = None
        Z = a * eye + b * R + c * (R @ R)
        Q = Z if Q is None else Z @ Q
        R = (Z @ R) @ Z
    X = Q @ X
    if tall:
        X = X.mT
    return X


# ------------------------------------------------------------------------------------------------
# CUDA implementations on the tcgen05 GEMM
# ------------------------------------------------------------------------------------------------
def _prepare_cuda(G: Tensor, allow_tall: bool = False):
    """-> (X [B, m, n] bf16 contiguous with m, n multiples of 8, restore).  Tall inputs are
    transposed to wide unless ``allow_tall`` (the caller then iterates in right-multiply form)."""
    G = unwrap(G)  # a pending functional collective must complete before its address is used
    shape = G.shape
    X = G.to(torch.bfloat16)
    if X.ndim == 2:
        X = X.unsqueeze(0)
    elif X.ndim > 3:
        X = X.reshape(-1, shape[-2], shape[-1])
    tall = X.size(-2) > X.size(-1) and not allow_tall
    if tall:
        X = X.mT
    m, n = X.size(-2), X.size(-1)
    mp, np_ = (m + 7) // 8 * 8, (n + 7) // 8 * 8
    padded = (mp, np_) != (m, n)
    if padded:
        Xp = torch.zeros((X.size(0), mp, np_), dtype=torch.bfloat16, device=X.device)
        Xp[:, :m, :n] = X
        X = Xp
    elif not X.is_contiguous() or X.data_ptr() % 16:
        X = X.contiguous()
    elif X.data_ptr() == G.data_ptr():
        X = X.clone()  # the iteration ping-pongs into its input buffer

    def restore(Y: Tensor) -> Tensor:
        if padded:
            Y = Y[:, :m, :n]
        if tall:
            Y = Y.mT
        return Y.reshape(shape)

    return X, restore


def _norm_scale(X: Tensor, norm_mult: float, epsilon: float) -> Tensor:
    ss = F.sumsq(X)
    return F.finalize_scale(ss, norm_mult, epsilon, out=ss)


def _iterate_cuda(X: Tensor, coeffs: Coeffs, scale: Optional[Tensor], hooks=None) -> Tensor:
    """Newton-Schulz iterations on ``X [B, m, n]``.  Wide or square matrices use the left form
    ``A = X X^T, X' = aX + (bA + cA^2) X``; tall ones the right form ``A = X^T X,
    X' = aX + X (bA + cA^2)``, reading ``X`` as an MN-major operand so that neither needs a
    transposed copy.  ``hooks`` (fused exchange) may supply per-launch coupling to other GPUs:
    ``hooks.first_gram()``, ``hooks.after_first_iteration()``, ``hooks.last_update()``."""
    B_, m, n = X.shape
    tall = m > n
    g = n if tall else m
    A = torch.empty((B_, g, g), dtype=torch.bfloat16, device=X.device)
    Bm = torch.empty_like(A)
    C = torch.empty_like(X)
    if hooks is None and gemm.persistent_fits(X, B_, m, n, len(coeffs)):
        done = gemm.ns_persistent(X, C, A, Bm, coeffs, scale)
        if done is not None:
            return done
    if hooks is None and gemm.iterate_in_one_call(X, B_, m, n):
        return gemm.ns_iterate(X, C, A, Bm, coeffs, scale)
    last = len(coeffs) - 1
    for it, (a, b, c) in enumerate(coeffs):
        sc = scale if it == 0 else None
        ex_first = hooks.first_gram(tall) if (hooks is not None and it == 0) else None
        if ex_first is not None:
            gemm.ns_gemm(X, X, out=A, sym=True, a_is_km=tall, b_is_kn=tall, alpha_pow=2,
                         extra=ex_first)
            sc = hooks.scale_after_first_gram()
        else:
            gemm.ns_gemm(X, X, out=A, sym=True, a_is_km=tall, b_is_kn=tall, scale=sc,
                         alpha_pow=2 if sc is not None else 0)
        gemm.ns_gemm(A, A, out=Bm, sym=True, D=A, alpha=c, beta=b)
        pw = 1 if sc is not None else 0
        ex_last = hooks.last_update() if (hooks is not None and it == last) else None
        out = None if ex_last is not None else C
        if tall:   # X' = a X + X B   (B symmetric: its rows are its columns)
            gemm.ns_gemm(X, Bm, out=out, D=X, alpha=1.0, beta=a, scale=sc, alpha_pow=pw,
                         beta_pow=pw, extra=ex_last)
        else:      # X' = a X + B X
            gemm.ns_gemm(Bm, X, out=out, b_is_kn=True, D=X, alpha=1.0, beta=a, scale=sc,
                         alpha_pow=pw, beta_pow=pw, extra=ex_last)
        if hooks is not None and it == 0:
            hooks.after_first_iteration()
            # the input belongs to the exchange and is handed back to the peers: from here on
            # ping-pong between private buffers only
            X, C = C, torch.empty_like(C)
        else:
            X, C = C, X
    return None if (hooks is not None) else X


def _ns_cuda(G: Tensor, coeffs: Coeffs, norm_mult: float, epsilon: float) -> Tensor:
    with trace.span("newton_schulz"):
        X, restore = _prepare_cuda(G, allow_tall=True)
        scale = _norm_scale(X, norm_mult, epsilon)
        return restore(_iterate_cuda(X, coeffs, scale))


def _aol_cuda(G: Tensor, epsilon: float) -> Tensor:
    X, restore = _prepare_cuda(G)
    B_, m, n = X.shape
    A = torch.empty((B_, m, m), dtype=torch.bfloat16, device=X.device)
    gemm.ns_gemm(X, X, out=A, sym=True)
    # X is private to this call (see _prepare_cuda), so the rescale may work in place: two
    # launches, the row scales and then X and A rescaled together.
    F.aol_rescale_(X, A, epsilon)
    a, b, c = AOL_COEFFS[0]
    Bm = torch.empty_like(A)
    C = torch.empty_like(X)
    gemm.ns_gemm(A, A, out=Bm, sym=True, D=A, alpha=c, beta=b)
    gemm.ns_gemm(Bm, X, out=C, b_is_kn=True, D=X, alpha=1.0, beta=a)
    return restore(_iterate_cuda(C, AOL_COEFFS[1:], None))


def _gram_cuda(G: Tensor, coeffs: Coeffs, norm_mult: float, epsilon: float,
               resets: Sequence[int]) -> Tensor:
    X, restore = _prepare_cuda(G)
    scale = _norm_scale(X, norm_mult, epsilon)
    B_, m, n = X.shape
    dev = X.device
    R = torch.empty((B_, m, m), dtype=torch.bfloat16, device=dev)
    gemm.ns_gemm(X, X, out=R, sym=True, scale=scale, alpha_pow=2)
    x_scale: Optional[Tensor] = scale  # X itself is still unnormalized until re-materialized
    Q: Optional[Tensor] = None
    Z = torch.empty_like(R)
    T = torch.empty_like(R)
    for it, (a, b, c) in enumerate(coeffs):
        if it in resets and Q is not None:
            Xn = torch.empty_like(X)
            gemm.ns_gemm(Q, X, out=Xn, b_is_kn=True, scale=x_scale,
                         alpha_pow=1 if x_scale is not None else 0)
            X, x_scale, Q = Xn, None, None
            gemm.ns_gemm(X, X, out=R, sym=True)
        gemm.ns_gemm(R, R, out=Z, sym=True, D=R, alpha=c, beta=b)
        Z.diagonal(dim1=-2, dim2=-1).add_(a)
        if Q is None:
            Q = Z.clone()
        else:
            Qn = torch.empty_like(Q)
            gemm.ns_gemm(Z, Q, out=Qn, b_is_kn=True)
            Q = Qn
        gemm.ns_gemm(Z, R, out=T)            # Z R   (R symmetric, so R^T = R)
        Rn = torch.empty_like(R)
        gemm.ns_gemm(T, Z, out=Rn, sym=True)  # (Z R) Z  (Z symmetric)
        R = Rn
    out = torch.empty_like(X)
    gemm.ns_gemm(Q, X, out=out, b_is_kn=True, scale=x_scale,
                 alpha_pow=1 if x_scale is not None else 0)
    return restore(out)


def _use_cuda(G: Tensor) -> bool:
    return G.is_cuda and G.numel() > 0


# ------------------------------------------------------------------------------------------------
# Public drivers
# ------------------------------------------------------------------------------------------------
@torch.no_grad()
def newton_schulz_quintic(G: Tensor, epsilon=1e-7) -> Tensor:
    eps = _eps(epsilon)
    return _ns_cuda(G, QUINTIC_COEFFS, 1.0, eps) if _use_cuda(G) else _ns_torch(G, QUINTIC_COEFFS, 1.0, eps)


@torch.no_grad()
def newton_schulz_classic(G: Tensor, epsilon=1e-7, steps: int = 5) -> Tensor:
    eps = _eps(epsilon)
    coeffs = (CLASSIC_COEFF,) * steps
    return _ns_cuda(G, coeffs, 1.0, eps) if _use_cuda(G) else _ns_torch(G, coeffs, 1.0, eps)


@torch.no_grad()
def polar_express(G: Tensor, epsilon=1e-6) -> Tensor:
    eps = _eps(epsilon)
    if _use_cuda(G):
        return _ns_cuda(G, POLAR_EXPRESS_COEFFS, 1.02, eps)
    return _ns_torch(G, POLAR_EXPRESS_COEFFS, 1.02, eps)


@torch.no_grad()
def newton_schulz_aol(G: Tensor, epsilon=1e-7) -> Tensor:
    eps = _eps(epsilon)
    return _aol_cuda(G, eps) if _use_cuda(G) else _aol_torch(G, eps)


@torch.no_grad()
def gram_newton_schulz(G: Tensor, epsilon=1e-6, reset_iterations: Sequence[int] = (2,),
                       coeffs: Coeffs = POLAR_EXPRESS_COEFFS, norm_mult: float = 1.02) -> Tensor:
    eps = _eps(epsilon)
    if _use_cuda(G):
        return _gram_cuda(G, coeffs, norm_mult, eps, tuple(reset_iterations))
    return _gram_torch(G, coeffs, norm_mult, eps, tuple(reset_iterations))


# (coefficients, norm multiplier) of the drivers whose iteration the fused exchange can run itself
newton_schulz_quintic.ns_spec = (QUINTIC_COEFFS, 1.0)
polar_express.ns_spec = (POLAR_EXPRESS_COEFFS, 1.02)
newton_schulz_classic.ns_spec = ((CLASSIC_COEFF,) * 5, 1.0)


def iterate_with_exchange(X: Tensor, ns_func: Callable, epsilon, hooks) -> None:
    """Run ``ns_func``'s iteration on the exchange's receive buffer ``X`` with the cross-GPU
    hooks attached (see ``parallel/fused_exchange.py``); results leave through the hooks."""
    coeffs, mult = ns_func.ns_spec
    hooks.norm_mult, hooks.eps = float(mult), _eps(epsilon)
    _iterate_cuda(X, coeffs, None, hooks=hooks)


def torch_reference(name: str) -> Callable:
    """Plain-PyTorch version of a driver (used as the oracle in tests and benchmarks)."""
    table = {
        "quintic": lambda G, epsilon=1e-7: _ns_torch(G, QUINTIC_COEFFS, 1.0, _eps(epsilon)),
        "classic": lambda G, epsilon=1e-7: _ns_torch(G, (CLASSIC_COEFF,) * 5, 1.0, _eps(epsilon)),
        "polar_express": lambda G, epsilon=1e-6: _ns_torch(G, POLAR_EXPRESS_COEFFS, 1.02, _eps(epsilon)),
        "aol": lambda G, epsilon=1e-7: _aol_torch(G, _eps(epsilon)),
        "gram": lambda G, epsilon=1e-6: _gram_torch(G, POLAR_EXPRESS_COEFFS, 1.02, _eps(epsilon), (2,)),
    }
    return table[name]


# Names under which the reference exposes the same functionality.
zeropower_via_newtonschulz5 = newton_schulz_quintic
newton_schulz_triton = newton_schulz_quintic
polar_express_triton = polar_express
newton_schulz_triton_fast = newton_schulz_aol


def ns_line_1(X: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``X @ X^T`` with symmetric half-work (reference: newton_schulz_triton.py:160-198)."""
    if X.is_cuda:
        return gemm.ns_gemm(X, X, out=out, sym=True)
    r = X @ X.mT
    return r if out is None else out.copy_(r)


def ns_line_2(A: Tensor, alpha: float, beta: float, out: Optional[Tensor] = None) -> Tensor:
    """``alpha * A @ A^T + beta * A`` for symmetric ``A`` (reference: :290-333)."""
    if A.is_cuda:
        return gemm.ns_gemm(A, A, out=out, sym=True, D=A, alpha=alpha, beta=beta)
    r = alpha * (A @ A.mT) + beta * A
    return r if out is None else out.copy_(r)


def ns_line_3(B: Tensor, X: Tensor, a: float, out: Optional[Tensor] = None) -> Tensor:
    """``a * X + B @ X`` (reference: :450-491)."""
    if B.is_cuda:
        return gemm.ns_gemm(B, X, out=out, b_is_kn=True, D=X, alpha=1.0, beta=a)
    r = a * X + B @ X
    return r if out is None else out.copy_(r)
