"""GPT decoder used by the trainer and the benchmarks: RoPE, QK-RMSNorm, ReLU^2 MLP, no biases,
no learnable norm weights, untied output head.  Module and parameter names match
models/gpt_model.py:64-193 of the reference (``transformer.wte``, ``transformer.h.{i}.attn.c_q``
... ``lm_head``), so checkpoints and param-group rules carry over.

The element-wise parts of the block (RMSNorm, RoPE + QK-norm, ReLU^2) and the loss go through
``dion_b200.models.functional``, which runs fused CUDA kernels with hand-written backward passes
on the GPU and plain PyTorch elsewhere - there is no tracing compiler on this path.  The GEMMs
are library calls and attention is PyTorch's fused SDPA.

``parallelize_gpt_model`` applies tensor parallelism (column/row-parallel linears), FSDP2
(``fully_shard`` per block, then the root) and HSDP on a ``DeviceMesh`` exactly as
models/gpt_model.py:236-398 does.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as tF
from torch.distributed.device_mesh import DeviceMesh

from . import functional as Fn


@dataclass
class GPTConfig:
    sequence_len: int = 1024
    vocab_size: int = 50304
    n_layer: int = 2
    n_head: int = 6
    n_embd: int = 768


class Rotary(nn.Module):
    """Cached cos/sin tables (bf16) for rotary position embedding over ``dim`` features."""

    def __init__(self, dim: int, base: float = 10000.0):
        super().__init__()
        self.dim, self.base = dim, base
        self.inv_freq: Optional[torch.Tensor] = None
        self.seq_len_cached: Optional[int] = None
        self.cos_cached = self.sin_cached = None

    def init_inv_freq(self) -> None:
        self.inv_freq = 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.dim))

    def forward(self, x: torch.Tensor):
        assert self.inv_freq is not None, "inv_freq not initialized"
        T = x.shape[1]
        if T != self.seq_len_cached or self.cos_cached.device != x.device:
            self.seq_len_cached = T
            inv = self.inv_freq.to(x.device)
            freqs = torch.outer(torch.arange(T, device=x.device, dtype=inv.dtype), inv)
            self.cos_cached = freqs.cos().bfloat16().contiguous()
            self.sin_cached = freqs.sin().bfloat16().contiguous()
        return self.cos_cached, self.sin_cached


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Reference formulation on ``[B, T, H, D]`` with ``cos/sin`` of shape ``[T, D/2]``."""
    assert x.ndim == 4
    d = x.shape[3] // 2
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * c + x2 * s, x2 * c - x1 * s], 3).type_as(x)


def _is_plain(module: nn.Module) -> bool:
    """True when ``module`` can be bypassed by a functional call on its weight: the weight is an
    ordinary tensor (not a DTensor shard) and nothing hooks the module's forward (tensor
    parallelism redistributes activations in such hooks)."""
    w = module.weight
    return (type(w) in (torch.Tensor, nn.Parameter) and not module._forward_hooks
            and not module._forward_pre_hooks)


def _linear(module: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    if module.bias is None and _is_plain(module):
        return Fn.linear(x, module.weight)
    return module(x)


class CausalSelfAttention(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.n_head, self.n_embd = config.n_head, config.n_embd
        self.head_dim = config.n_embd // config.n_head
        self.c_q = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_k = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_v = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_proj = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.rotary = Rotary(self.head_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, _ = x.size()
        cos, sin = self.rotary(x)
        if _is_plain(self.c_q) and _is_plain(self.c_k) and _is_plain(self.c_v):
            # q/k/v projections (one GEMM), rotary embedding, then RMS-norm over head_dim
            q, k, v = Fn.qkv_rope(x, self.c_q.weight, self.c_k.weight, self.c_v.weight, cos, sin,
                                  self.n_head)
        else:
            q = self.c_q(x).view(B, T, -1, self.head_dim)
            k = self.c_k(x).view(B, T, -1, self.head_dim)
            v = self.c_v(x).view(B, T, -1, self.head_dim)
            q, k = Fn.rope_qknorm(q, k, cos, sin)
        y = tF.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        y = y.transpose(1, 2).contiguous().view(B, T, -1)
        return _linear(self.c_proj, y)


class MLP(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, bias=False)
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (self.c_fc.bias is None and self.c_proj.bias is None and _is_plain(self.c_fc)
                and _is_plain(self.c_proj)):
            return Fn.mlp_relu2(x, self.c_fc.weight, self.c_proj.weight)
        return _linear(self.c_proj, Fn.relu2(_linear(self.c_fc, x)))


class Block(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.attn = CausalSelfAttention(config)
        self.mlp = MLP(config)

    def forward(self, x: torch.Tensor, h: Optional[torch.Tensor] = None):
        """``x`` is the residual stream; ``h = rms_norm(x)`` may be passed in by the caller that
        already computed it.  Returns the new residual stream and its normalisation, so that the
        next block (or the output head) does not have to read ``x`` again."""
        if h is None:
            h = Fn.rms_norm(x)
        x, h = Fn.add_rms_norm(x, self.attn(h))
        x, h = Fn.add_rms_norm(x, self.mlp(h))
        return x, h


class GPT(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.config = config
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            h=nn.ModuleList([Block(config) for _ in range(config.n_layer)]),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)

    def init_weights(self) -> None:
        self.apply(self._init_weights)

    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, nn.Linear):
            fan_out, fan_in = module.weight.size(0), module.weight.size(1)
            std = 1.0 / math.sqrt(fan_in) * min(1.0, math.sqrt(fan_out / fan_in))
            torch.nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                torch.nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=1.0)
        elif isinstance(module, Rotary):
            module.init_inv_freq()

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None,
                return_logits: bool = False):
        wte = self.transformer.wte
        x = Fn.embedding(idx, wte.weight) if _is_plain(wte) else wte(idx)
        h = None
        for block in self.transformer.h:
            x, h = block(x, h)
        x = h if h is not None else Fn.rms_norm(x)  # final norm rides on the last residual add
        if targets is not None:
            logits = _linear(self.lm_head, x)
            if return_logits:
                return logits.float()
            return Fn.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1),
                                    ignore_index=-1)
        logits = self.lm_head(x[:, [-1], :]).float()
        return logits if return_logits else None

    def compile(self) -> None:  # kept for call-site compatibility; there is nothing to trace
        return None

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None) -> torch.Tensor:
        """Sample ``max_new_tokens`` continuations, keeping the last ``sequence_len`` tokens as
        context."""
        idx = input_ids
        for _ in range(max_new_tokens):
            ctx = idx[:, -self.config.sequence_len:]
            logits = self(ctx, targets=None, return_logits=True)[:, -1, :] / temperature
            if top_k is not None:
                kth = torch.topk(logits, min(top_k, logits.size(-1))).values[:, [-1]]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            nxt = torch.multinomial(tF.softmax(logits, dim=-1), num_samples=1)
            idx = torch.cat([idx, nxt], dim=1)
        return idx


# ------------------------------------------------------------------------------------------------
# Parallelization
# ------------------------------------------------------------------------------------------------
def parallelize_gpt_model(
    model: GPT,
    device_mesh: DeviceMesh,
    dp_name: Optional[str] = "dp",
    fs_name: Optional[str] = "fs",
    tp_name: Optional[str] = "tp",
    fsdp_reshard_after_forward: bool = True,
) -> None:
    """Parallelize ``model`` in place over the named mesh dimensions: ``tp_name`` tensor
    parallel, ``fs_name`` fully sharded, ``dp_name`` replicated (HSDP, needs ``fs_name``)."""
    wanted = [n for n in (dp_name, fs_name, tp_name) if n]
    if not wanted:
        raise ValueError("At least one of dp_name, fs_name, or tp_name must be provided")
    if dp_name and not fs_name:
        raise ValueError("Data parallelism with fully_shard() requires 2D FSDP mesh")
    if device_mesh.ndim < len(wanted):
        raise ValueError(
            f"Expected {len(wanted)}-D device mesh {wanted}, but got mesh with "
            f"{device_mesh.ndim} dimensions")
    names = list(device_mesh.mesh_dim_names)
    if not all(n in names for n in wanted):
        raise ValueError(f"Expected device mesh to have names {wanted}, but got {names}")

    tp_enabled = False
    if tp_name and device_mesh[tp_name].size() > 1:
        _apply_tp(model, device_mesh[tp_name])
        tp_enabled = True
    if fs_name:
        fsdp_mesh = device_mesh[fs_name] if not dp_name else device_mesh[dp_name, fs_name]
        _apply_fsdp(model, fsdp_mesh, fsdp_reshard_after_forward, tp_enabled)


def _apply_tp(model: GPT, tp_mesh: DeviceMesh) -> None:
    from torch.distributed.tensor import Replicate
    from torch.distributed.tensor.parallel import (ColwiseParallel, RowwiseParallel,
                                                   parallelize_module)

    parallelize_module(model, tp_mesh, {
        "transformer.wte": RowwiseParallel(input_layouts=Replicate(), output_layouts=Replicate()),
        "lm_head": ColwiseParallel(input_layouts=Replicate(), output_layouts=Replicate()),
    })
    for block in model.transformer.h:
        parallelize_module(block, tp_mesh, {
            "attn.c_q": ColwiseParallel(), "attn.c_k": ColwiseParallel(),
            "attn.c_v": ColwiseParallel(), "attn.c_proj": RowwiseParallel(),
            "mlp.c_fc": ColwiseParallel(), "mlp.c_proj": RowwiseParallel(),
        })
        if block.attn.n_head % tp_mesh.size() != 0:
            raise AssertionError(
                f"attn.n_head {block.attn.n_head} must be divisible by TP size {tp_mesh.size()}")
        block.attn.n_head //= tp_mesh.size()


def _apply_fsdp(model: GPT, fsdp_mesh: DeviceMesh, reshard_after_forward: bool,
                tp_enabled: bool) -> None:
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from torch.distributed.tensor import Shard

    policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for block in model.transformer.h:
        placement_fn = None
        if tp_enabled:
            # FSDP shards the dimension that tensor parallelism left whole.
            dims = {block.attn.c_q.weight: 1, block.attn.c_k.weight: 1, block.attn.c_v.weight: 1,
                    block.attn.c_proj.weight: 0, block.mlp.c_fc.weight: 1,
                    block.mlp.c_proj.weight: 0}
            placement_fn = lambda p, dims=dims: Shard(dims[p]) if p in dims else None  # noqa: E731
        fully_shard(block, mesh=fsdp_mesh, shard_placement_fn=placement_fn, mp_policy=policy,
                    reshard_after_forward=reshard_after_forward)
    placement_fn = None
    if tp_enabled:
        dims = {model.transformer.wte.weight: 1, model.lm_head.weight: 1}
        placement_fn = lambda p, dims=dims: Shard(dims[p]) if p in dims else None  # noqa: E731
    fully_shard(model, mesh=fsdp_mesh, mp_policy=policy, shard_placement_fn=placement_fn,
                reshard_after_forward=False)
