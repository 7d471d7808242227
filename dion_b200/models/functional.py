"""Fused element-wise pieces of the GPT block and the loss.

Each function is an autograd ``Function`` whose forward and backward are single CUDA kernels from
``csrc/model_ops.cu`` when the input lives on a GPU, and the equivalent PyTorch expression
otherwise (CPU tests, unsupported dtypes).  They replace what the reference obtains by tracing
its model with ``torch.compile`` (models/gpt_model.py:195-200).

* ``rms_norm(x)``            RMS normalisation over the last dim, no weight; under bf16 autocast
                             the result is emitted in bf16 for the GEMM that consumes it.
* ``rope_qknorm(q, k, ...)`` rotary embedding followed by RMS-norm over ``head_dim`` for q and k.
* ``relu2(x)``               ``relu(x)**2``.
* ``cross_entropy(...)``     mean token loss from bf16/fp32 logits with fp32 softmax arithmetic;
                             the backward pass is computed together with the forward and stored
                             in place of the logits.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn.functional as tF
from torch import Tensor

from ..ops import _backend
from ..utils.tensors import is_plain_tensor, materialize, unwrap

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _c(t: Optional[Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    ptr = t.data_ptr()
    if ptr == 0 and t.numel():
        # e.g. a wrapper tensor subclass without storage of its own: never give a kernel address 0
        raise RuntimeError(f"{type(t).__name__} has no device storage to hand to a kernel")
    return ctypes.c_void_p(ptr)


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _lib():
    return _backend.lib("model_ops")


def _check(rc, name):
    if rc != 0:
        raise RuntimeError(f"{name} launch failed (code {rc})")


def _autocast_bf16(x: Tensor) -> bool:
    return (x.is_cuda and torch.is_autocast_enabled("cuda")
            and torch.get_autocast_dtype("cuda") == torch.bfloat16)


def _eps_for(dtype: torch.dtype) -> float:
    return float(torch.finfo(dtype).eps)


# ------------------------------------------------------------------------------------------------
# RMS norm (optionally fused with the residual add that precedes it)
# ------------------------------------------------------------------------------------------------
def _rows(x: Tensor) -> Tensor:
    x2 = x.reshape(-1, x.size(-1))
    return x2 if x2.is_contiguous() else x2.contiguous()


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, eps: float, out_dtype: torch.dtype):
        x2 = _rows(x)
        rows, D = x2.shape
        y = torch.empty((rows, D), dtype=out_dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(_lib().dion_rmsnorm_fwd(_c(x2), _DT[x2.dtype], _c(None), 0, _c(None), _c(y),
                                       _DT[out_dtype], _c(rstd), ctypes.c_longlong(rows), D,
                                       ctypes.c_float(eps), _stream(x.device)), "dion_rmsnorm_fwd")
        ctx.save_for_backward(x2, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy: Tensor):
        dy = unwrap(dy)
        x2, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = _rows(dy)
        dx = torch.empty_like(x2)
        _check(_lib().dion_rmsnorm_bwd(_c(x2), _DT[x2.dtype], _c(dy2), _DT[dy2.dtype], _c(rstd),
                                       _c(None), _c(dx), _c(None), ctypes.c_longlong(rows), D,
                                       _stream(x2.device)), "dion_rmsnorm_bwd")
        return dx.view(ctx.shape), None, None


class _AddRMSNorm(torch.autograd.Function):
    """``x_new = x + delta; h = rms_norm(x_new)`` in one pass; the backward pass adds the
    gradient that reaches ``x_new`` through the residual path to the norm's gradient and emits
    it twice: in ``x``'s dtype for the residual stream and in bf16 for the branch behind
    ``delta``."""

    @staticmethod
    def forward(ctx, x: Tensor, delta: Tensor, eps: float, out_dtype: torch.dtype):
        x2, d2 = _rows(x), _rows(delta)
        rows, D = x2.shape
        x_new = torch.empty_like(x2)
        h = torch.empty((rows, D), dtype=out_dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(_lib().dion_rmsnorm_fwd(_c(x2), _DT[x2.dtype], _c(d2), _DT[d2.dtype], _c(x_new),
                                       _c(h), _DT[out_dtype], _c(rstd), ctypes.c_longlong(rows),
                                       D, ctypes.c_float(eps), _stream(x.device)),
               "dion_rmsnorm_fwd")
        ctx.save_for_backward(x_new, rstd)
        ctx.shape = x.shape
        ctx.delta_dtype = delta.dtype
        return x_new.view(x.shape), h.view(x.shape)

    @staticmethod
    def backward(ctx, g_x: Tensor, g_h: Tensor):
        g_x, g_h = unwrap(g_x), unwrap(g_h)
        x_new, rstd = ctx.saved_tensors
        rows, D = x_new.shape
        gx2 = _rows(g_x) if g_x is not None else None
        gh2 = _rows(g_h)
        dx = torch.empty_like(x_new)
        want_bf16 = ctx.delta_dtype == torch.bfloat16 and x_new.dtype != torch.bfloat16
        dx2 = torch.empty((rows, D), dtype=torch.bfloat16, device=x_new.device) if want_bf16 else None
        _check(_lib().dion_rmsnorm_bwd(_c(x_new), _DT[x_new.dtype], _c(gh2), _DT[gh2.dtype],
                                       _c(rstd), _c(gx2), _c(dx), _c(dx2),
                                       ctypes.c_longlong(rows), D, _stream(x_new.device)),
               "dion_rmsnorm_bwd")
        dx = dx.view(ctx.shape)
        ddelta = dx2.view(ctx.shape) if want_bf16 else dx.to(ctx.delta_dtype)
        return dx, ddelta, None, None


def _norm_kernel_ok(x: Tensor) -> bool:
    return (is_plain_tensor(x) and x.is_cuda and x.dtype in _DT and x.size(-1) % 8 == 0
            and x.size(-1) <= 4096)


def rms_norm(x: Tensor, eps: Optional[float] = None) -> Tensor:
    """``x * rsqrt(mean(x**2, -1) + eps)``; ``eps`` defaults to the machine epsilon of ``x``'s
    dtype, as in ``torch.nn.functional.rms_norm``."""
    x = materialize(x)
    if _norm_kernel_ok(x):
        out_dtype = torch.bfloat16 if _autocast_bf16(x) else x.dtype
        return _RMSNorm.apply(x, _eps_for(x.dtype) if eps is None else eps, out_dtype)
    return tF.rms_norm(x, (x.size(-1),), eps=eps)


def add_rms_norm(x: Tensor, delta: Tensor, eps: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """``(x + delta, rms_norm(x + delta))``: the residual update of a transformer block together
    with the normalisation that feeds the next sub-layer."""
    x, delta = materialize(x), materialize(delta)
    if (_norm_kernel_ok(x) and is_plain_tensor(delta) and delta.is_cuda and delta.dtype in _DT
            and delta.shape == x.shape):
        out_dtype = torch.bfloat16 if _autocast_bf16(x) else x.dtype
        return _AddRMSNorm.apply(x, delta, _eps_for(x.dtype) if eps is None else eps, out_dtype)
    x = x + delta
    return x, tF.rms_norm(x, (x.size(-1),), eps=eps)


# ------------------------------------------------------------------------------------------------
# RoPE + QK norm
# ------------------------------------------------------------------------------------------------
def _rope_torch(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    d = x.shape[3] // 2
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * c + x2 * s, x2 * c - x1 * s], 3).type_as(x)


def _row_stride(t: Tensor) -> Optional[int]:
    """Row stride of a ``[B, T, H, D]`` tensor whose (H, D) block is dense and whose (B, T)
    dims collapse to one row index, or None."""
    B, T, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D:
        return None
    rs = t.stride(1)
    if B > 1 and t.stride(0) != T * rs:
        return None
    return rs


class _RopeQKNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, eps: float):
        B, T, H, D = q.shape
        rs_q, rs_k = _row_stride(q), _row_stride(k)
        if rs_q is None or rs_k != rs_q or rs_q % 8 or q.data_ptr() % 16 or k.data_ptr() % 16:
            q, k = q.contiguous(), k.contiguous()
            rs_q = H * D
        qo = torch.empty((B, T, H, D), dtype=q.dtype, device=q.device)
        ko = torch.empty_like(qo)
        rstd = torch.empty((2, B * T * H), dtype=torch.float32, device=q.device)
        _check(_lib().dion_rope_qknorm_fwd(_c(q), _c(k), ctypes.c_longlong(rs_q), _c(cos), _c(sin),
                                           _c(qo), _c(ko), _c(rstd), B, T, H, D,
                                           ctypes.c_float(eps), _stream(q.device)),
               "dion_rope_qknorm_fwd")
        ctx.save_for_backward(q, k, cos, sin, rstd)
        ctx.rs = rs_q
        return qo, ko

    @staticmethod
    def backward(ctx, dqo: Tensor, dko: Tensor):
        dqo, dko = unwrap(dqo), unwrap(dko)
        q, k, cos, sin, rstd = ctx.saved_tensors
        B, T, H, D = q.shape
        dqo, dko = dqo.contiguous(), dko.contiguous()
        dq = torch.empty((B, T, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty_like(dq)
        _check(_lib().dion_rope_qknorm_bwd(_c(q), _c(k), ctypes.c_longlong(ctx.rs), _c(cos),
                                           _c(sin), _c(dqo), _c(dko), _c(rstd), _c(dq), _c(dk),
                                           ctypes.c_longlong(H * D), _c(None),
                                           ctypes.c_longlong(0), _c(None),
                                           B, T, H, D, _stream(q.device)), "dion_rope_qknorm_bwd")
        return dq, dk, None, None, None


def rope_qknorm(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> Tuple[Tensor, Tensor]:
    """Rotary embedding (``cos/sin``: ``[T, D/2]``) then RMS-norm over the last dim, for ``q``
    and ``k`` of shape ``[B, T, H, D]``."""
    q, k = materialize(q), materialize(k)
    D = q.size(-1)
    if (is_plain_tensor(q) and is_plain_tensor(k) and q.is_cuda and q.dtype == torch.bfloat16
            and k.dtype == torch.bfloat16
            and D in (32, 64, 128, 256) and cos.dtype == torch.bfloat16 and q.shape == k.shape
            and cos.is_contiguous() and sin.is_contiguous()):
        return _RopeQKNorm.apply(q, k, cos, sin, _eps_for(torch.bfloat16))
    q, k = _rope_torch(q, cos, sin), _rope_torch(k, cos, sin)
    return tF.rms_norm(q, (D,)), tF.rms_norm(k, (D,))


class _QKVRope(torch.autograd.Function):
    """``q, k, v = h W_q^T, h W_k^T, h W_v^T`` as ONE GEMM against the stacked weight, followed by
    rotary embedding and RMS-norm of q and k.  The three weights stay separate parameters (the
    optimizers orthogonalize them as separate matrices, as the reference model's c_q / c_k / c_v
    are, models/gpt_model.py:60-63); only the arithmetic is fused: one forward GEMM, one
    input-gradient GEMM over K = 3C with no summation of three partial gradients, and one
    weight-gradient GEMM written directly in the parameters' dtype."""

    @staticmethod
    def forward(ctx, h: Tensor, wq: Tensor, wk: Tensor, wv: Tensor, cos: Tensor, sin: Tensor,
                n_head: int, eps: float):
        B, T, C = h.shape
        D = C // n_head
        h2 = h.reshape(B * T, C)
        W = torch.empty((3 * C, C), dtype=h.dtype, device=h.device)
        torch._foreach_copy_([W[:C], W[C:2 * C], W[2 * C:]], [wq, wk, wv])  # one launch, casts
        qkv = torch.mm(h2, W.t())                       # [B*T, 3C]
        q = qkv[:, :C]
        k = qkv[:, C:2 * C]
        qo = torch.empty((B, T, n_head, D), dtype=h.dtype, device=h.device)
        ko = torch.empty_like(qo)
        rstd = torch.empty((2, B * T * n_head), dtype=torch.float32, device=h.device)
        _check(_lib().dion_rope_qknorm_fwd(_c(q), _c(k), ctypes.c_longlong(3 * C), _c(cos),
                                           _c(sin), _c(qo), _c(ko), _c(rstd), B, T, n_head, D,
                                           ctypes.c_float(eps), _stream(h.device)),
               "dion_rope_qknorm_fwd")
        ctx.save_for_backward(h2, W, qkv, cos, sin, rstd)
        ctx.dims = (B, T, C, n_head, D)
        ctx.wdtype = wq.dtype
        v = qkv.view(B, T, 3, n_head, D)[:, :, 2]
        return qo, ko, v

    @staticmethod
    def backward(ctx, dqo: Tensor, dko: Tensor, dv: Tensor):
        dqo, dko, dv = unwrap(dqo), unwrap(dko), unwrap(dv)
        h2, W, qkv, cos, sin, rstd = ctx.saved_tensors
        B, T, C, H, D = ctx.dims
        dqkv = torch.empty_like(qkv)
        dqo, dko = dqo.contiguous(), dko.contiguous()
        # The attention backward lays dv out like v itself (rows 3C apart): the kernel reads it
        # through its row pitch instead of a compacting copy first.
        if (dv.dim() == 4 and dv.stride(3) == 1 and dv.stride(2) == D and dv.stride(1) % 8 == 0
                and dv.stride(1) >= C and dv.stride(0) == T * dv.stride(1)
                and dv.data_ptr() % 16 == 0):
            dv_pitch = dv.stride(1)
        else:
            dv, dv_pitch = dv.contiguous(), C
        # One kernel: RoPE/QK-norm backward into the q and k columns, dv copied into the v columns.
        _check(_lib().dion_rope_qknorm_bwd(_c(qkv[:, :C]), _c(qkv[:, C:2 * C]),
                                           ctypes.c_longlong(3 * C), _c(cos), _c(sin), _c(dqo),
                                           _c(dko), _c(rstd), _c(dqkv[:, :C]),
                                           _c(dqkv[:, C:2 * C]), ctypes.c_longlong(3 * C),
                                           _c(dv), ctypes.c_longlong(dv_pitch),
                                           _c(dqkv[:, 2 * C:]),
                                           B, T, H, D, _stream(h2.device)),
               "dion_rope_qknorm_bwd")
        dh = torch.mm(dqkv, W).view(B, T, C)
        if ctx.wdtype == torch.float32 and dqkv.dtype == torch.bfloat16:
            dW = torch.mm(dqkv.t(), h2, out_dtype=torch.float32)
        else:
            dW = torch.mm(dqkv.t(), h2).to(ctx.wdtype)
        return dh, dW[:C], dW[C:2 * C], dW[2 * C:], None, None, None, None


def qkv_rope(h: Tensor, wq: Tensor, wk: Tensor, wv: Tensor, cos: Tensor, sin: Tensor,
             n_head: int) -> Tuple[Tensor, Tensor, Tensor]:
    """``(q, k, v)`` of shape ``[B, T, H, D]`` from the normalized hidden state ``h [B, T, C]``:
    the three projections, rotary embedding and QK RMS-norm (q and k are contiguous, v is a
    strided view of the projection output)."""
    h = materialize(h)
    B, T, C = h.shape
    D = C // n_head
    if (is_plain_tensor(h) and is_plain_tensor(wq) and is_plain_tensor(wk) and is_plain_tensor(wv)
            and h.is_cuda and h.dtype == torch.bfloat16 and D in (32, 64, 128, 256) and C % 8 == 0
            and cos.dtype == torch.bfloat16 and cos.is_contiguous() and sin.is_contiguous()
            and wq.shape == wk.shape == wv.shape == (C, C)):
        return _QKVRope.apply(h, wq, wk, wv, cos, sin, n_head, _eps_for(torch.bfloat16))
    q = tF.linear(h, wq).view(B, T, n_head, D)
    k = tF.linear(h, wk).view(B, T, n_head, D)
    v = tF.linear(h, wv).view(B, T, n_head, D)
    q, k = rope_qknorm(q, k, cos, sin)
    return q, k, v


# ------------------------------------------------------------------------------------------------
# Embedding and linear layers with mixed-precision-aware backward passes
# ------------------------------------------------------------------------------------------------
_sort_bytes: dict = {}


def _embedding_sort_bytes(n: int, V: int) -> int:
    key = (n, V)
    b = _sort_bytes.get(key)
    if b is None:
        fn = _backend.lib("embedding_ops")._dll.dion_embedding_sort_bytes
        fn.restype = ctypes.c_longlong
        b = int(fn(ctypes.c_longlong(n), ctypes.c_longlong(V)))
        if b < 0:
            raise RuntimeError("dion_embedding_sort_bytes failed")
        _sort_bytes[key] = b
    return b


class _Embedding(torch.autograd.Function):
    """``weight[idx]`` whose backward sorts (id, position) pairs over the bits an id needs and
    writes every row of the weight gradient exactly once - the sum of the id's rows in position
    order, or zeros (deterministic; replaces the zero fill, the 64-bit sort and the atomics of the
    stock dense backward)."""

    @staticmethod
    def forward(ctx, idx: Tensor, weight: Tensor):
        ctx.save_for_backward(idx)
        ctx.wshape = weight.shape
        return tF.embedding(idx, weight)

    @staticmethod
    def backward(ctx, dy: Tensor):
        dy = unwrap(dy)
        (idx,) = ctx.saved_tensors
        V, C = ctx.wshape
        flat = idx.reshape(-1)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        n = flat.numel()
        dy2 = dy.reshape(-1, C)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dev = dy.device
        gw = torch.empty((V, C), dtype=torch.float32, device=dev)   # every row is written
        scratch = torch.empty(4 * n + V + 1, dtype=torch.int32, device=dev)
        nbytes = _embedding_sort_bytes(n, V)
        temp = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        keys, vals, starts = scratch[:2 * n], scratch[2 * n:4 * n], scratch[4 * n:]
        _check(_backend.lib("embedding_ops").dion_embedding_bwd(
            _c(flat), _c(dy2), _DT[dy2.dtype], _c(gw), ctypes.c_longlong(n), C,
            ctypes.c_longlong(V), _c(keys), _c(vals), _c(starts), _c(temp),
            ctypes.c_longlong(nbytes), _stream(dev)), "dion_embedding_bwd")
        return None, gw


def embedding(idx: Tensor, weight: Tensor) -> Tensor:
    idx = materialize(idx)
    if (is_plain_tensor(idx) and is_plain_tensor(weight) and weight.is_cuda
            and weight.dtype == torch.float32 and weight.size(1) % 8 == 0
            and weight.size(1) <= 7168 and idx.numel() < 2 ** 31 - 256
            and idx.dtype == torch.int64 and weight.requires_grad and torch.is_grad_enabled()):
        return _Embedding.apply(idx, weight)
    return tF.embedding(idx, weight)


class _LinearBF16(torch.autograd.Function):
    """``x @ W^T`` in bf16 for an fp32 master weight: the weight gradient is accumulated in fp32
    by the GEMM itself (no bf16 round trip and no cast kernel)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor):
        wb = weight.to(torch.bfloat16)
        x2 = x.reshape(-1, x.size(-1))
        ctx.save_for_backward(x2, wb)
        ctx.xshape = x.shape
        ctx.wdtype = weight.dtype
        return torch.mm(x2, wb.t()).view(*x.shape[:-1], weight.size(0))

    @staticmethod
    def backward(ctx, dy: Tensor):
        dy = unwrap(dy)
        x2, wb = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        dx = torch.mm(dy2, wb).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = torch.mm(dy2.t(), x2, out_dtype=torch.float32)
        return dx, dw if ctx.wdtype == torch.float32 else dw.to(ctx.wdtype)


def linear(x: Tensor, weight: Tensor) -> Tensor:
    """Bias-free linear layer.  Under bf16 autocast on a GPU (bf16 activations, fp32 weight) the
    mixed-precision form above is used; otherwise ``torch.nn.functional.linear``."""
    x = materialize(x)
    if (is_plain_tensor(x) and x.is_cuda and x.dtype == torch.bfloat16
            and weight.dtype == torch.float32 and is_plain_tensor(weight) and x.size(-1) % 8 == 0
            and weight.size(0) % 8 == 0):
        return _LinearBF16.apply(x, weight)
    return tF.linear(x, weight)


class _MLPRelu2(torch.autograd.Function):
    """``relu(h W_fc^T)^2 W_proj^T`` with the activation folded into the GEMM epilogues of the
    two-CTA tcgen05 kernel: the forward GEMM writes ``relu(.)^2`` directly (the pre-activation is
    never stored), and the backward GEMM ``dY W_proj`` multiplies by ``2*sqrt(act)`` - the
    derivative of ReLU^2 expressed through its output - as it drains the accumulator."""

    @staticmethod
    def forward(ctx, h: Tensor, wfc: Tensor, wproj: Tensor):
        from ..ops import gemm
        x2 = h.reshape(-1, h.size(-1))
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        wfb, wpb = wfc.to(torch.bfloat16), wproj.to(torch.bfloat16)
        act = gemm.ns_gemm(x2, wfb, epilogue="relu2")
        y = torch.mm(act, wpb.t())
        ctx.save_for_backward(x2, act, wfb, wpb)
        ctx.hshape = h.shape
        ctx.wdtypes = (wfc.dtype, wproj.dtype)
        return y.view(*h.shape[:-1], wproj.size(0))

    @staticmethod
    def backward(ctx, dy: Tensor):
        dy = unwrap(dy)
        from ..ops import gemm
        x2, act, wfb, wpb = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dz = gemm.ns_gemm(dy2, wpb, b_is_kn=True, D=act, epilogue="mul_2sqrt")
        dwp = torch.mm(dy2.t(), act, out_dtype=torch.float32)
        dh = torch.mm(dz, wfb).view(ctx.hshape)
        dwf = torch.mm(dz.t(), x2, out_dtype=torch.float32)
        return dh, dwf.to(ctx.wdtypes[0]), dwp.to(ctx.wdtypes[1])


def mlp_relu2(h: Tensor, wfc: Tensor, wproj: Tensor) -> Tensor:
    """The ReLU^2 MLP of the GPT block.  With ``DION_B200_FUSED_MLP=1``, bf16 activations with
    ordinary (non-DTensor) weights on a GPU take the fused form above; otherwise the plain
    composition (library GEMMs + element-wise kernels), which is the default: timed inside the
    GPT-160M training step the fused form is slower (39.2 against 35.8 ms per step) although
    it saves two element-wise passes, because at K = 768 the two-CTA kernel is bound by operand
    traffic from L2 (no multicast loads) and trails the library GEMM by about 10 %."""
    h = materialize(h)
    if (is_plain_tensor(h) and h.is_cuda and h.dtype == torch.bfloat16 and is_plain_tensor(wfc)
            and is_plain_tensor(wproj)
            and wfc.dtype in (torch.float32, torch.bfloat16) and wfc.dtype == wproj.dtype
            and h.size(-1) % 8 == 0 and wfc.size(0) % 8 == 0 and wfc.size(0) > 128
            and h.numel() // h.size(-1) > 128 and fused_mlp_enabled()):
        return _MLPRelu2.apply(h, wfc, wproj)
    return linear(relu2(linear(h, wfc)), wproj)


def fused_mlp_enabled() -> bool:
    import os
    return os.environ.get("DION_B200_FUSED_MLP", "0") == "1"


# ------------------------------------------------------------------------------------------------
# ReLU^2
# ------------------------------------------------------------------------------------------------
class _Relu2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor):
        x = x.contiguous()
        y = torch.empty_like(x)
        _check(_lib().dion_relu2_fwd(_c(x), _c(y), _DT[x.dtype], ctypes.c_longlong(x.numel()),
                                     _stream(x.device)), "dion_relu2_fwd")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        dy = unwrap(dy)
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        _check(_lib().dion_relu2_bwd(_c(x), _c(dy), _c(dx), _DT[x.dtype],
                                     ctypes.c_longlong(x.numel()), _stream(x.device)),
               "dion_relu2_bwd")
        return dx


def relu2(x: Tensor) -> Tensor:
    x = materialize(x)
    if is_plain_tensor(x) and x.is_cuda and x.dtype in _DT and x.numel() % 8 == 0:
        return _Relu2.apply(x)
    return tF.relu(x).square()


# ------------------------------------------------------------------------------------------------
# Cross entropy
# ------------------------------------------------------------------------------------------------
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: Tensor, targets: Tensor, ignore_index: int):
        N, V = logits.shape
        need_grad = bool(ctx.needs_input_grad[0])
        losses = torch.empty(N, dtype=torch.float32, device=logits.device)
        count = torch.zeros(1, dtype=torch.float32, device=logits.device)
        tgt = targets if targets.dtype == torch.int64 else targets.long()
        lib = _lib()
        _check(lib.dion_ce_count(_c(tgt), ctypes.c_longlong(N), ignore_index, _c(count),
                                 _stream(logits.device)), "dion_ce_count")
        # Loss per row and, when a backward pass will follow, d(mean loss)/d(logits) written
        # over the logits themselves (nothing else reads them afterwards).
        _check(lib.dion_ce_fwd_bwd(_c(logits), _DT[logits.dtype], _c(tgt), ctypes.c_longlong(N), V,
                                   ctypes.c_longlong(logits.stride(0)), ignore_index, _c(losses),
                                   _c(count), int(need_grad), _stream(logits.device)),
               "dion_ce_fwd_bwd")
        loss = losses.sum() / count.clamp(min=1.0)
        if need_grad:
            ctx.save_for_backward(logits)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, dloss: Tensor):
        dloss = unwrap(dloss)
        (grad,) = ctx.saved_tensors
        # The upstream gradient is 1 for a plain ``loss.backward()``: the kernel reads it on the
        # device and returns at once in that case, otherwise it rescales the stored gradient.
        scale = dloss.detach().reshape(1).to(torch.float32)
        _check(_lib().dion_scale_unless_one(_c(grad), _DT[grad.dtype],
                                            ctypes.c_longlong(grad.numel()), _c(scale),
                                            _stream(grad.device)), "dion_scale_unless_one")
        return grad, None, None


def cross_entropy(logits: Tensor, targets: Tensor, ignore_index: int = -1) -> Tensor:
    """Mean cross entropy over the rows whose target is not ``ignore_index``; softmax
    arithmetic in fp32 regardless of the logits' dtype."""
    logits, targets = materialize(logits), materialize(targets)
    if (is_plain_tensor(logits) and is_plain_tensor(targets) and logits.is_cuda
            and logits.dtype in _DT and logits.ndim == 2 and logits.stride(1) == 1
            and logits.size(1) % 8 == 0):
        return _CrossEntropy.apply(logits, targets, ignore_index)
    return tF.cross_entropy(logits.float(), targets, ignore_index=ignore_index)
