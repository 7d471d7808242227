"""Dion2 sub-matrix selection: momentum accumulate, slice L1 norms, exact top-k, gather and
error-feedback write-back (reference: dion/dion2.py:437-547 and the ``_select_ns`` wrapper at
:565-617).  CUDA tensors use ``csrc/select_ops.cu``; other tensors use the PyTorch code below.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
from torch import Tensor

from . import _backend
from .tables import RawPointer, build_ptr_array

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _c(p):
    return ctypes.c_void_p(p)


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _check(rc, name):
    if rc != 0:
        raise RuntimeError(f"{name} launch failed (code {rc})")


def _as_matrices(ts: List[Tensor]) -> List[Tensor]:
    """Expand tensors with batch dimensions into lists of 2-D views."""
    out: List[Tensor] = []
    for t in ts:
        if t.ndim == 2:
            out.append(t)
        else:
            out.extend(t.reshape(-1, t.size(-2), t.size(-1)).unbind(0))
    return out


def dion2_select(
    G: Optional[List[Tensor]],
    M: List[Tensor],
    k: int,
    select_dim: int,
    ef_decay: float,
    apply_ef: bool = True,
    out_addresses: Optional[List[int]] = None,
    sumsq_addresses: Optional[List[int]] = None,
) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """``M += G`` (skipped when ``G`` is None), pick the ``k`` rows (``select_dim=-2``) or columns
    (``-1``) of each matrix with the largest L1 norm, return them as a dense bf16 stack and scale
    them by ``ef_decay`` inside ``M``.

    Returns ``(U, indices, maps)``: ``U`` is ``[N, k, cols]`` or ``[N, rows, k]``; ``indices`` is
    ``[N, k]`` int64 (unordered); ``maps`` is ``[N, num_slices]`` int32 giving each slice's
    position in ``U`` or -1 (None on the PyTorch path).  ``N`` counts 2-D matrices, so a
    parameter with batch dimensions contributes several."""
    Mm = _as_matrices(M)
    Gm = _as_matrices(G) if G is not None else None
    N = len(Mm)
    rows, cols = Mm[0].shape
    num = rows if select_dim == -2 else cols
    dev = Mm[0].device
    out_shape = (N, k, cols) if select_dim == -2 else (N, rows, k)
    use_kernel = (
        dev.type == "cuda" and k > 0 and num > 0
        and all(m.dtype in _DT and m.is_contiguous() and m.dtype == Mm[0].dtype for m in Mm)
        and (Gm is None or all(g.dtype in _DT and g.is_contiguous() and g.dtype == Gm[0].dtype for g in Gm))
    )
    if use_kernel:
        lib = _backend.lib("select_ops")
        ptrs = build_ptr_array([Gm if Gm is not None else [None] * N, Mm], tag="sel")
        norms = (torch.empty if select_dim == -2 else torch.zeros)(
            (N, num), dtype=torch.float32, device=dev)
        g_dt = _DT[Gm[0].dtype] if Gm is not None else 0
        m_dt = _DT[Mm[0].dtype]
        _check(lib.dion_slice_norms(_c(ptrs.data_ptr()), N, rows, cols, g_dt, m_dt,
                                    int(select_dim == -2), _c(norms.data_ptr()), _stream(dev)),
               "dion_slice_norms")
        idx = torch.empty((N, k), dtype=torch.int64, device=dev)
        maps = torch.empty((N, num), dtype=torch.int32, device=dev)
        _check(lib.dion_topk_select(_c(norms.data_ptr()), N, num, k, _c(idx.data_ptr()),
                                    _c(maps.data_ptr()), _stream(dev)), "dion_topk_select")
        if out_addresses is not None:
            # Selected rows go straight to the given addresses (peer-mapped buffers of the ranks
            # that own the matrices); their sums of squares are added at sumsq_addresses.
            assert select_dim == -2 and len(out_addresses) == N
            dst = build_ptr_array([[RawPointer(a) for a in out_addresses],
                                   [RawPointer(a) for a in (sumsq_addresses or [0] * N)]],
                                  tag="sel_dst")
            _check(lib.dion_gather_ef(_c(ptrs.data_ptr()), N, rows, cols, m_dt,
                                      _c(idx.data_ptr()), k, 1, _c(0), ctypes.c_longlong(0),
                                      ctypes.c_float(float(ef_decay)), int(bool(apply_ef)),
                                      _c(dst[0].data_ptr()),
                                      _c(dst[1].data_ptr() if sumsq_addresses else 0),
                                      _stream(dev)), "dion_gather_ef")
            return None, idx, maps
        U = torch.empty(out_shape, dtype=torch.bfloat16, device=dev)
        _check(lib.dion_gather_ef(_c(ptrs.data_ptr()), N, rows, cols, m_dt, _c(idx.data_ptr()), k,
                                  int(select_dim == -2), _c(U.data_ptr()),
                                  ctypes.c_longlong(U[0].numel()), ctypes.c_float(float(ef_decay)),
                                  int(bool(apply_ef)), _c(0), _c(0), _stream(dev)),
               "dion_gather_ef")
        return U, idx, maps

    # PyTorch path
    if Gm is not None:
        torch._foreach_add_(Mm, [g.to(Mm[0].dtype) for g in Gm])
    if k == 0 or num == 0:
        U = torch.zeros(out_shape, dtype=torch.bfloat16, device=dev)
        return U, torch.empty((N, 0), dtype=torch.int64, device=dev), None
    stacked = torch.stack(Mm)
    norm_dim = -1 if select_dim == -2 else -2
    norms = stacked.abs().sum(dim=norm_dim, dtype=torch.float32)
    idx = torch.topk(norms, k, dim=-1, sorted=False).indices
    if select_dim == -2:
        idx_exp = idx.unsqueeze(-1).expand(N, k, cols)
    else:
        idx_exp = idx.unsqueeze(-2).expand(N, rows, k)
    sel = torch.gather(stacked, select_dim, idx_exp)
    if apply_ef:
        for m, ie, s in zip(Mm, idx_exp.unbind(0), sel.unbind(0)):
            m.scatter_(select_dim, ie, s * ef_decay)
    return sel.to(torch.bfloat16), idx, None


def scatter_selected(src: Tensor, idx: Tensor, num: int, select_dim: int) -> Tensor:
    """Place the selected slices ``src`` back into a zero matrix with ``num`` slices along
    ``select_dim`` (the layout the "global" selection scope hands to the masked post-update)."""
    N = src.size(0)
    if select_dim == -2:
        out = torch.zeros((N, num, src.size(-1)), dtype=src.dtype, device=src.device)
        if src.is_cuda and src.dtype == torch.bfloat16 and src.is_contiguous() and idx.numel():
            _check(_backend.lib("select_ops").dion_scatter_rows(
                _c(src.data_ptr()), _c(idx.data_ptr()), N, idx.size(-1), src.size(-1),
                _c(out.data_ptr()), num, _stream(src.device)), "dion_scatter_rows")
            return out
        out.scatter_(-2, idx.unsqueeze(-1).expand_as(src), src)
        return out
    out = torch.zeros((N, src.size(-2), num), dtype=src.dtype, device=src.device)
    out.scatter_(-1, idx.unsqueeze(-2).expand_as(src), src)
    return out
