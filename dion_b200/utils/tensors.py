"""Small tensor / DTensor helpers shared by the optimizers (the non-scheduling part of
dion/opt_utils.py:9-94 in the reference)."""
from __future__ import annotations

import math
from collections import defaultdict
from typing import Iterator, List, Sequence, Union

import torch
from torch import Tensor
from torch.distributed.tensor import DTensor

TensorOrList = Union[Tensor, List[Tensor]]


def lm_head_lr_scale(scalar_opt: str, model_dim: int) -> float:
    """Lion on the output head uses ``1/sqrt(d_in)`` of the base LR; AdamW uses it unchanged."""
    return 1.0 / math.sqrt(model_dim) if scalar_opt == "lion" else 1.0


def as_scalar_tensor(value) -> Tensor:
    """A hyper-parameter as a tensor.  An existing tensor is returned as is (never copied), so a
    persistent device scalar keeps its identity and a captured graph keeps reading it."""
    return value if isinstance(value, Tensor) else torch.tensor(value)


def unwrap(t):
    """Complete a pending functional collective and return the ordinary tensor behind an
    ``AsyncCollectiveTensor`` (what tensor-parallel layers and ``DTensor.to_local()`` hand out
    after an all-reduce / all-gather); anything else passes through.  The kernels of this package
    take raw device pointers, which bypasses the operator dispatch that would otherwise wait.
    Not differentiable: for use in optimizer code and inside autograd ``Function`` bodies."""
    if type(t) is Tensor or t is None:
        return t
    try:
        from torch.distributed._functional_collectives import AsyncCollectiveTensor
    except Exception:  # pragma: no cover - torch without functional collectives
        return t
    if isinstance(t, AsyncCollectiveTensor):
        return t.trigger_wait()
    return t


class _Wait(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t):
        return unwrap(t)

    @staticmethod
    def backward(ctx, grad):
        return grad


def materialize(t):
    """Differentiable form of :func:`unwrap` for activations."""
    if type(t) is Tensor or t is None:
        return t
    try:
        from torch.distributed._functional_collectives import AsyncCollectiveTensor
    except Exception:  # pragma: no cover
        return t
    if isinstance(t, AsyncCollectiveTensor):
        return _Wait.apply(t)
    return t


def is_plain_tensor(t) -> bool:
    """True for ordinary tensors / parameters (no DTensor, no wrapper subclass): only those may
    be handed to a kernel by address."""
    return type(t) is Tensor or type(t) is torch.nn.Parameter


def to_local(x: TensorOrList) -> TensorOrList:
    """Local shard(s) of DTensor(s), with pending collectives completed; plain tensors pass
    through."""
    if isinstance(x, Tensor):
        return unwrap(x.to_local() if isinstance(x, DTensor) else x)
    return [unwrap(t.to_local() if isinstance(t, DTensor) else t) for t in x]


def dtensor_from_local(x: TensorOrList, ref: Tensor) -> TensorOrList:
    """Wrap local tensor(s) with ``ref``'s mesh and placements (no-op when ``ref`` is plain)."""
    if not isinstance(ref, DTensor):
        return x
    mesh, placements = ref.device_mesh, ref.placements
    if isinstance(x, Tensor):
        return DTensor.from_local(x, device_mesh=mesh, placements=placements)
    return [DTensor.from_local(t, device_mesh=mesh, placements=placements) for t in x]


def bucket_key(p: Tensor):
    return (p.shape, p.placements if isinstance(p, DTensor) else None, p.dtype)


def group_by_shape(params: Sequence[Tensor]):
    """Parameters bucketed by (shape, placements, dtype), in first-seen order."""
    buckets = defaultdict(list)
    for p in params:
        buckets[bucket_key(p)].append(p)
    return buckets


def create_param_batches(params: Sequence[Tensor], batch_size: int) -> Iterator[List[Tensor]]:
    """Batches of at most ``batch_size`` parameters with identical shape, sharding and dtype."""
    for bucket in group_by_shape(params).values():
        for start in range(0, len(bucket), batch_size):
            yield bucket[start:start + batch_size]


def pad_batch(batch: List[Tensor], batch_size: int) -> List[Tensor]:
    """Append uninitialised stand-ins until the batch has ``batch_size`` entries."""
    assert 0 < len(batch) <= batch_size
    return batch + [torch.empty_like(batch[0]) for _ in range(batch_size - len(batch))]
