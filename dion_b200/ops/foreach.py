"""Element-wise optimizer updates over lists of tensors.

Every function has two implementations with the same semantics:

* CUDA tensors run one multi-tensor kernel launch from ``csrc/foreach_ops.cu``;
* anything else (CPU tensors in tests and in ``gloo`` runs, dtypes the kernels do not cover)
  runs the plain PyTorch code in this file, which is also the numerical oracle of the kernels.

The math follows the reference's compiled helpers: Muon pre/post-orthogonalize
(dion/muon.py:283-347), AdamW and Lion (dion/scalar_opts.py:121-308), Dion2 post-update
(dion/dion2.py:666-740, dion/dion2_triton.py:57-144) and NorMuon normalization
(dion/normuon.py:344-399).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor

from . import _backend
from ..utils.tensors import is_plain_tensor
from .tables import RawPointer, build_table

Scalar = Union[float, Tensor]
_DT = {torch.float32: 0, torch.bfloat16: 1}


def _c(p):
    return ctypes.c_void_p(p)


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _kernel_ok(*lists: Sequence[Tensor]) -> bool:
    """CUDA kernels cover contiguous fp32/bf16 tensors."""
    first = lists[0][0]
    if not first.is_cuda:
        return False
    for lst in lists:
        for t in lst:
            if t is None or isinstance(t, RawPointer):
                continue
            if not is_plain_tensor(t) or t.dtype not in _DT or not t.is_contiguous():
                return False
    return True


def _same_dtype(lst: Sequence[Tensor]) -> bool:
    return all(t.dtype == lst[0].dtype for t in lst)


def device_scalar(value: Scalar, device: torch.device) -> Tensor:
    """0-d fp32 tensor on ``device``; an existing device tensor is passed through untouched so
    that a captured graph keeps reading the live value."""
    if isinstance(value, Tensor):
        if value.device == device and value.dtype == torch.float32:
            return value
        return value.detach().to(device=device, dtype=torch.float32)
    return torch.full((), float(value), dtype=torch.float32, device=device)


def _wd_args(wd: Scalar, device):
    """(pointer-tensor or None, float) - a device tensor is read live, anything else is baked."""
    if isinstance(wd, Tensor) and wd.is_cuda:
        t = device_scalar(wd, device)
        return t, 0.0
    return None, float(wd)


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} launch failed (code {rc})")


# ------------------------------------------------------------------------------------------------
# Muon pre-orthogonalize
# ------------------------------------------------------------------------------------------------
def muon_pre(
    G: List[Tensor],
    M: List[Tensor],
    mu: float,
    nesterov: bool,
    out: Optional[List[Tensor]] = None,
    sumsq: Optional[Tensor] = None,
    add_only: bool = False,
    sumsq_targets: Optional[List[int]] = None,
    out_block: Optional[Tuple[int, int]] = None,
) -> List[Tensor]:
    """``M = mu*M + G`` (or ``M += G`` with ``add_only``); returns the bf16 orthogonalization
    input ``U`` (``mu*M + G`` with Nesterov, else ``M``), written into ``out`` when given.
    ``out=False`` skips the bf16 output altogether.
    ``sumsq[i]`` (optional, fp32, pre-zeroed) receives ``sum(U_i**2)``.  ``out`` entries may be
    :class:`RawPointer` addresses of peer-GPU memory; ``sumsq_targets[i]`` (raw addresses of fp32
    accumulators, possibly on a peer) then receive the sums instead of ``sumsq``.
    ``out_block=(cols, pitch)``: every ``M`` is a ``[rows, cols]`` matrix and its ``out`` entry
    points at a column block of a wider row-major matrix with row pitch ``pitch`` elements
    (kernel path with raw pointers only)."""
    if not G:
        return []
    if out is False:      # momentum update only: no bf16 copy is wanted
        out = [None] * len(M)
    if out is None:
        out = [torch.empty_like(m, dtype=torch.bfloat16) for m in M]
    if _kernel_ok(G, M, out) and _same_dtype(G) and _same_dtype(M) and M[0].numel():
        dev = M[0].device
        lists = [G, M, out]
        if sumsq_targets is not None:
            lists.append([RawPointer(a) for a in sumsq_targets])
        tb = build_table(lists, [m.numel() for m in M], tag="pre")
        _check(
            _backend.lib("foreach_ops").dion_muon_pre(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks),
                _DT[G[0].dtype], _DT[M[0].dtype], ctypes.c_float(float(mu)),
                int(bool(nesterov)), int(bool(add_only)),
                _c(sumsq.data_ptr() if sumsq is not None else 0),
                int(sumsq_targets is not None),
                ctypes.c_longlong(out_block[0] if out_block else 0),
                ctypes.c_longlong(out_block[1] if out_block else 0), _stream(dev)),
            "dion_muon_pre")
        return out
    if out_block is not None:
        raise RuntimeError("muon_pre(out_block=...) needs the CUDA kernel path")
    # PyTorch path
    dtype = M[0].dtype
    Gc = [g.to(dtype) for g in G]
    if add_only:
        torch._foreach_add_(M, Gc)
        U = M
    else:
        torch._foreach_mul_(M, float(mu))
        torch._foreach_add_(M, Gc)
        if nesterov:
            U = torch._foreach_mul(M, float(mu))
            torch._foreach_add_(U, Gc)
        else:
            U = M
    for o, u in zip(out, U):
        if o is not None and o.numel():
            o.copy_(u)
    if sumsq is not None:
        sumsq.add_(torch.stack([u.to(torch.bfloat16).float().square().sum() for u in U]))
    return out


# ------------------------------------------------------------------------------------------------
# Muon post-orthogonalize
# ------------------------------------------------------------------------------------------------
def muon_post(
    X: List[Tensor],
    U: List[Tensor],
    lr: Scalar,
    weight_decay: Scalar,
    ratio: float,
    cautious_wd: bool = False,
    rowscale: Optional[List[Tensor]] = None,
    normU2: Optional[Tensor] = None,
    normNew2: Optional[Tensor] = None,
    wait: Optional[tuple] = None,
) -> None:
    """``X = X*(1 - lr*wd) - lr*ratio*U`` (cautious: decay only where ``X*U >= 0``).

    ``wait = (flags, seq, per_rank, status)`` makes every block first wait (bounded) until the
    rank that produced its ``U`` has raised its flag to the current sequence number.

    ``rowscale[i]`` (fp32, one value per row of ``U[i]``) and the pair ``normU2/normNew2``
    (per-tensor squared Frobenius norms before/after the row scaling) carry NorMuon's
    normalization so that it is applied while the update is read."""
    if not X:
        return
    if _kernel_ok(X, U) and _same_dtype(X) and all(u.dtype == torch.bfloat16 for u in U):
        dev = X[0].device
        lr_t = device_scalar(lr, dev)
        wd_t, wd_f = _wd_args(weight_decay, dev)
        cols = X[0].size(-1) if rowscale is not None else 0
        lists = [X, U, rowscale if rowscale is not None else [None] * len(X)]
        tb = build_table(lists, [x.numel() for x in X], tag="post")
        _check(
            _backend.lib("foreach_ops").dion_muon_post(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks),
                _c(lr_t.data_ptr()), _c(wd_t.data_ptr() if wd_t is not None else 0),
                ctypes.c_float(wd_f), ctypes.c_float(float(ratio)), int(bool(cautious_wd)),
                _DT[X[0].dtype], int(cols),
                _c(normU2.data_ptr() if normU2 is not None else 0),
                _c(normNew2.data_ptr() if normNew2 is not None else 0),
                _c(wait[0].data_ptr() if wait else 0), _c(wait[1].data_ptr() if wait else 0),
                int(wait[2]) if wait else 1, _c(wait[3].data_ptr() if wait else 0),
                _stream(dev)),
            "dion_muon_post")
        return
    # PyTorch path
    step = lr * ratio
    Uf = []
    for i, (x, u) in enumerate(zip(X, U)):
        uf = u.to(torch.float32)
        if rowscale is not None:
            uf = uf * rowscale[i].reshape(*uf.shape[:-1], 1)
        if normU2 is not None:
            uf = uf * (normU2[i].sqrt() / normNew2[i].sqrt().clamp(min=1e-8))
        Uf.append(uf.to(x.dtype) if rowscale is None and normU2 is None else uf)
    if cautious_wd:
        coeff = lr * weight_decay
        for x, u in zip(X, Uf):
            mask = (x * u.to(x.dtype) >= 0).to(x.dtype)
            x.sub_(x * mask * coeff)
    else:
        torch._foreach_mul_(X, 1 - lr * weight_decay)
    for x, u in zip(X, Uf):
        x.sub_((u * step).to(x.dtype))


# ------------------------------------------------------------------------------------------------
# AdamW
# ------------------------------------------------------------------------------------------------
def adamw(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    V: List[Tensor],
    lr: Scalar,
    beta1: float,
    beta2: float,
    weight_decay: Scalar,
    epsilon: float,
    step: Optional[int] = None,
    state_steps: Optional[List[Tensor]] = None,
    cautious_wd: bool = False,
) -> None:
    """Decoupled-weight-decay Adam over a list of tensors.

    Exactly one of ``step`` (host integer, baked) and ``state_steps`` (per-tensor fp32 device
    counters, advanced here on the device) selects the bias-correction source."""
    if (step is None) == (state_steps is None):
        raise ValueError("adamw takes exactly one of step (host int) or state_steps (device counters)")
    if state_steps is not None and not isinstance(lr, Tensor):
        raise TypeError("the state_steps form requires lr as a tensor so that it stays live under graph replay")
    if not X:
        return
    n = len(X)
    assert n == len(G) == len(M) == len(V)
    beta1, beta2, epsilon = float(beta1), float(beta2), float(epsilon)
    if (_kernel_ok(X, G, M, V) and _same_dtype(X) and _same_dtype(G) and _same_dtype(M)
            and _same_dtype(V)
            and (state_steps is None or all(s.is_cuda and s.dtype == torch.float32 for s in state_steps))):
        dev = X[0].device
        lr_t = device_scalar(lr, dev)
        wd_t, wd_f = _wd_args(weight_decay, dev)
        lists = [X, G, M, V]
        if state_steps is not None:
            lists.append(state_steps)
        tb = build_table(lists, [x.numel() for x in X], tag="adamw")
        _check(
            _backend.lib("foreach_ops").dion_adamw(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks), n,
                _c(lr_t.data_ptr()), _c(wd_t.data_ptr() if wd_t is not None else 0),
                ctypes.c_float(wd_f), ctypes.c_float(beta1), ctypes.c_float(beta2),
                ctypes.c_float(epsilon), int(bool(cautious_wd)),
                _DT[X[0].dtype], _DT[G[0].dtype], _DT[M[0].dtype], _DT[V[0].dtype],
                int(state_steps is not None), ctypes.c_float(float(step or 0)), _stream(dev)),
            "dion_adamw")
        return
    # PyTorch path
    if state_steps is not None:
        seen = set()
        for s in state_steps:
            if id(s) not in seen:
                seen.add(id(s))
                s.add_(1)
    for i in range(n):
        x, g, m, v = X[i], G[i], M[i], V[i]
        dev = x.device
        if state_steps is not None:
            st = state_steps[i].detach().to(device=dev, dtype=torch.float64)
        else:
            st = torch.tensor(float(step), dtype=torch.float64, device=dev)
        lr64 = (lr.detach().to(device=dev, dtype=torch.float64) if isinstance(lr, Tensor)
                else torch.tensor(float(lr), dtype=torch.float64, device=dev))
        wd32 = (weight_decay.detach().to(device=dev, dtype=torch.float32)
                if isinstance(weight_decay, Tensor) else float(weight_decay))
        m.lerp_(g.to(m.dtype), 1 - beta1)
        gv = g.to(v.dtype)
        v.mul_(beta2).addcmul_(gv, gv, value=1 - beta2)
        step_size = (lr64 / (1 - beta1 ** st)).to(torch.float32)
        bc2_sqrt = (1 - beta2 ** st).sqrt().to(torch.float32)
        denom = v.to(torch.float32).sqrt() / bc2_sqrt + epsilon
        coeff = lr64.to(torch.float32) * wd32
        if cautious_wd:
            mask = (m.to(torch.float32) * x.to(torch.float32) >= 0).to(x.dtype)
            x.sub_((x * mask * coeff).to(x.dtype))
        else:
            x.sub_((x * coeff).to(x.dtype))
        x.sub_((step_size * m.to(torch.float32) / denom).to(x.dtype))


# ------------------------------------------------------------------------------------------------
# Lion
# ------------------------------------------------------------------------------------------------
def lion(
    X: List[Tensor],
    G: List[Tensor],
    M: List[Tensor],
    lr: Scalar,
    beta1: float,
    beta2: float,
    weight_decay: Scalar,
    cautious_wd: bool = False,
) -> None:
    """``U = sign(lerp(M, G, 1-beta1)); M = lerp(M, G, 1-beta2); X = X*(1-lr*wd) - lr*U``."""
    if not X:
        return
    beta1, beta2 = float(beta1), float(beta2)
    if _kernel_ok(X, G, M) and _same_dtype(X) and _same_dtype(G) and _same_dtype(M):
        dev = X[0].device
        lr_t = device_scalar(lr, dev)
        wd_t, wd_f = _wd_args(weight_decay, dev)
        tb = build_table([X, G, M], [x.numel() for x in X], tag="lion")
        _check(
            _backend.lib("foreach_ops").dion_lion(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks),
                _c(lr_t.data_ptr()), _c(wd_t.data_ptr() if wd_t is not None else 0),
                ctypes.c_float(wd_f), ctypes.c_float(beta1), ctypes.c_float(beta2),
                int(bool(cautious_wd)), _DT[X[0].dtype], _DT[G[0].dtype], _DT[M[0].dtype],
                _stream(dev)),
            "dion_lion")
        return
    Gc = [g.to(m.dtype) for g, m in zip(G, M)]
    U = [torch.lerp(m, g, 1 - beta1).sign_() for m, g in zip(M, Gc)]
    for m, g in zip(M, Gc):
        m.lerp_(g, 1 - beta2)
    coeff = lr * weight_decay
    if cautious_wd:
        for x, u in zip(X, U):
            mask = (u.to(x.dtype) * x >= 0).to(x.dtype)
            x.sub_(x * mask * coeff)
    else:
        torch._foreach_mul_(X, 1 - coeff)
    for x, u in zip(X, U):
        x.sub_((u * lr).to(x.dtype))


# ------------------------------------------------------------------------------------------------
# Dion2 post-update
# ------------------------------------------------------------------------------------------------
def dion2_post(
    X: List[Tensor],
    U: List[Tensor],
    indices: List[Tensor],
    maps: Optional[List[Tensor]],
    lr: Scalar,
    weight_decay: Scalar,
    ratio: float,
    select_dim: int,
    rowscale: Optional[List[Tensor]] = None,
    normU2: Optional[Tensor] = None,
    normNew2: Optional[Tensor] = None,
    wait: Optional[tuple] = None,
) -> None:
    """``x = (1 - lr*wd)*x - lr*ratio*u`` on the selected rows/columns and plain decay elsewhere,
    rounded once.  ``indices[i]`` lists the selected slices of ``X[i]`` in the order of ``U[i]``;
    ``maps[i]`` (int32, slice -> position or -1) is the inverse the kernel reads.  ``wait`` as
    in :func:`muon_post` (kernel path only)."""
    if not X:
        return
    k = U[0].size(select_dim) if U[0].numel() else 0
    if (maps is not None and X[0].ndim == 2 and _kernel_ok(X, U) and _same_dtype(X)
            and all(u.dtype == torch.bfloat16 for u in U)):
        dev = X[0].device
        lr_t = device_scalar(lr, dev)
        wd_t, wd_f = _wd_args(weight_decay, dev)
        lists = [X, U, maps, rowscale if rowscale is not None else [None] * len(X)]
        tb = build_table(lists, [x.numel() for x in X], tag="d2post")
        _check(
            _backend.lib("foreach_ops").dion_dion2_post(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks),
                _c(lr_t.data_ptr()), _c(wd_t.data_ptr() if wd_t is not None else 0),
                ctypes.c_float(wd_f), ctypes.c_float(float(ratio)), _DT[X[0].dtype],
                int(X[0].size(-1)), int(k), int(select_dim == -2),
                _c(normU2.data_ptr() if normU2 is not None else 0),
                _c(normNew2.data_ptr() if normNew2 is not None else 0),
                _c(wait[0].data_ptr() if wait else 0), _c(wait[1].data_ptr() if wait else 0),
                int(wait[2]) if wait else 1, _c(wait[3].data_ptr() if wait else 0),
                _stream(dev)),
            "dion_dion2_post")
        return
    if wait is not None:
        raise RuntimeError("dion2_post(wait=...) needs the CUDA kernel path (2-D bf16 updates "
                           "with an index map)")
    # PyTorch path: decay in place, then overwrite the selected slices with the fused value.
    a = 1 - lr * weight_decay
    b = lr * ratio
    for i, (x, u, idx) in enumerate(zip(X, U, indices)):
        if idx.numel() == 0:
            x.mul_(a)
            continue
        uf = u.to(torch.float32)
        if rowscale is not None:
            uf = uf * rowscale[i].reshape(*uf.shape[:-1], 1)
        if normU2 is not None:
            uf = uf * (normU2[i].sqrt() / normNew2[i].sqrt().clamp(min=1e-8))
        idx_exp = idx.unsqueeze(-1).expand_as(uf) if select_dim == -2 else idx.unsqueeze(-2).expand_as(uf)
        sel = a * torch.gather(x, select_dim, idx_exp).to(torch.float32) - b * uf
        x.mul_(a)
        x.scatter_(select_dim, idx_exp, sel.to(x.dtype))


def dion2_post_masked(X: List[Tensor], M: List[Tensor], U: List[Tensor], lr: Scalar,
                      weight_decay: Scalar, ratio: float, ef_decay: float, select_dim: int) -> None:
    """Post step of Dion2's global selection scope (reference: dion/dion2.py:621-659): ``U[i]``
    is full-size and zero off the selected slices, which are recognised by holding a non-zero.
    ``X = (1 - lr*wd)*X - lr*ratio*U`` and the selected slices of ``M`` are scaled by
    ``ef_decay``; on a GPU two launches cover every parameter."""
    if not X:
        return
    if (X[0].ndim == 2 and _kernel_ok(X, M, U) and _same_dtype(X) and _same_dtype(M)
            and all(u.dtype == torch.bfloat16 for u in U)
            and all(x.shape == X[0].shape for x in X)):
        dev = X[0].device
        lr_t = device_scalar(lr, dev)
        wd_t, wd_f = _wd_args(weight_decay, dev)
        num_select = X[0].size(select_dim)
        flags = torch.empty((len(X), num_select), dtype=torch.int32, device=dev)
        tb = build_table([X, M, U], [x.numel() for x in X], tag="d2mask")
        _check(
            _backend.lib("foreach_ops").dion_dion2_post_masked(
                _c(tb.device_tensor.data_ptr()), ctypes.c_longlong(tb.n_chunks), len(X),
                _c(lr_t.data_ptr()), _c(wd_t.data_ptr() if wd_t is not None else 0),
                ctypes.c_float(wd_f), ctypes.c_float(float(ratio)), ctypes.c_float(float(ef_decay)),
                _DT[X[0].dtype], _DT[M[0].dtype], int(X[0].size(-1)), int(select_dim == -2),
                int(num_select), _c(flags.data_ptr()), _stream(dev)),
            "dion_dion2_post_masked")
        return
    norm_dim = -1 if select_dim == -2 else -2
    torch._foreach_mul_(X, 1 - lr * weight_decay)
    step = lr * ratio
    for x, m, u in zip(X, M, U):
        sel = u.to(torch.float32).abs().sum(dim=norm_dim, keepdim=True) > 0
        m.mul_(torch.where(sel, ef_decay, 1.0).to(m.dtype))
        x.sub_((step * u).to(x.dtype))


# ------------------------------------------------------------------------------------------------
# NorMuon statistics
# ------------------------------------------------------------------------------------------------
def normuon_rowstats(
    U: Tensor,
    V: List[Tensor],
    beta2: float,
    vmaps: Optional[List[Tensor]] = None,
    guard: Optional[Tensor] = None,
):
    """Per-row second-moment update for a stacked update ``U`` of shape ``[N, rows, cols]``.

    ``V[i]`` (shape ``[R, 1]``) is updated in place as ``lerp(V, mean(U_i**2, -1), 1-beta2)`` at
    rows ``vmaps[i]`` (all rows when ``vmaps`` is None).  Returns ``(rinv, normU2, normNew2)``:
    ``rinv[N, rows] = 1/(sqrt(V)+1e-8)``, and the squared Frobenius norms of ``U_i`` and of
    ``U_i * rinv_i``.  ``guard`` (the device status word) makes the kernel leave ``V`` untouched
    when an earlier kernel reported that ``U`` may be incomplete."""
    N, rows, cols = U.shape
    dev = U.device
    rinv = torch.empty((N, rows), dtype=torch.float32, device=dev)
    normU2 = torch.zeros(N, dtype=torch.float32, device=dev)
    normNew2 = torch.zeros(N, dtype=torch.float32, device=dev)
    if N == 0 or rows == 0:
        return rinv, normU2, normNew2
    if (U.is_cuda and U.dtype == torch.bfloat16 and U.is_contiguous() and _kernel_ok(V)
            and _same_dtype(V)):
        lists = [V, vmaps if vmaps is not None else [None] * N]
        tb = build_table(lists, [rows] * N, tag="nmu")
        _check(
            _backend.lib("foreach_ops").dion_normuon_rowstats(
                _c(tb.device_tensor.data_ptr()), _c(U.data_ptr()), N, rows, cols,
                _DT[V[0].dtype], ctypes.c_float(float(beta2)), _c(rinv.data_ptr()),
                _c(normU2.data_ptr()), _c(normNew2.data_ptr()),
                _c(guard.data_ptr() if guard is not None else 0), _stream(dev)),
            "dion_normuon_rowstats")
        return rinv, normU2, normNew2
    Uf = U.to(torch.float32)
    rowsq = Uf.square().sum(dim=-1)  # [N, rows]
    ms = rowsq / cols
    for i in range(N):
        v = V[i].reshape(-1)
        vf = v.to(torch.float32)
        if vmaps is not None:
            cur = vf[vmaps[i]]
            new = torch.lerp(cur, ms[i], 1 - beta2)
            v[vmaps[i]] = new.to(v.dtype)
        else:
            new = torch.lerp(vf, ms[i], 1 - beta2)
            v.copy_(new.to(v.dtype))
        rinv[i] = 1.0 / (new.sqrt() + 1e-8)
    normU2.copy_(rowsq.sum(dim=-1))
    normNew2.copy_((rowsq * rinv * rinv).sum(dim=-1))
    return rinv, normU2, normNew2


def sumsq(X: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """Squared Frobenius norm of every matrix of a bf16 batch ``[N, ...]`` (fp32 result)."""
    N = X.size(0)
    if out is None:
        out = torch.zeros(N, dtype=torch.float32, device=X.device)
    if X.is_cuda and X.dtype == torch.bfloat16 and X.is_contiguous():
        numel = X[0].numel() if N else 0
        _check(
            _backend.lib("foreach_ops").dion_sumsq(
                _c(X.data_ptr()), N, ctypes.c_longlong(numel), _c(out.data_ptr()), _stream(X.device)),
            "dion_sumsq")
        return out
    out.add_(X.to(torch.float32).reshape(N, -1).square().sum(dim=-1))
    return out


def aol_rescale_(X: Tensor, A: Tensor, eps: float) -> None:
    """AOL rescaling in place: with ``s_i = rsqrt(max(sum_j |A_ij|, eps))`` of the Gram matrix
    ``A = X X^T`` (``[B, m, m]``), ``X <- diag(s) X`` and ``A <- diag(s) A diag(s)``
    (reference: dion/newton_schulz_triton.py:601-612)."""
    B, m, n = X.shape
    if (X.is_cuda and X.dtype == A.dtype == torch.bfloat16 and X.is_contiguous()
            and A.is_contiguous() and m % 8 == 0 and n % 8 == 0):
        s = torch.empty(B * m, dtype=torch.float32, device=X.device)
        _check(
            _backend.lib("foreach_ops").dion_aol_rescale(
                _c(X.data_ptr()), _c(A.data_ptr()), _c(s.data_ptr()), ctypes.c_longlong(B), m, n,
                ctypes.c_float(float(eps)), _stream(X.device)),
            "dion_aol_rescale")
        return
    s = torch.rsqrt(A.abs().sum(dim=-1, dtype=torch.float32).clamp_min(eps))
    X.copy_((X * s.unsqueeze(-1)).to(X.dtype))
    A.copy_((A * s.unsqueeze(-1) * s.unsqueeze(-2)).to(A.dtype))


def finalize_scale(sumsq_t: Tensor, mult: float, eps: float, out: Optional[Tensor] = None) -> Tensor:
    """``1 / (sqrt(sumsq)*mult + eps)``: the Newton-Schulz input normalization factor."""
    if out is None:
        out = torch.empty_like(sumsq_t)
    if sumsq_t.is_cuda:
        _check(
            _backend.lib("foreach_ops").dion_finalize_scale(
                _c(sumsq_t.data_ptr()), _c(out.data_ptr()), sumsq_t.numel(),
                ctypes.c_float(float(mult)), ctypes.c_float(float(eps)), _stream(sumsq_t.device)),
            "dion_finalize_scale")
        return out
    out.copy_(1.0 / (sumsq_t.sqrt() * mult + eps))
    return out
