"""Per-optimizer scratch arena with stable addresses.

An optimizer step is a fixed sequence of kernels over fixed shapes.  Handing out its temporaries
from an arena that is rewound at the start of every step gives each temporary the same device
address in every step, so the multi-tensor kernels' pointer tables are built once, and a CUDA
graph captured after the warm-up steps keeps pointing at live memory.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
from torch import Tensor


class StepArena:
    def __init__(self) -> None:
        self._slots: List[Tensor] = []
        self._cursor = 0

    def reset(self) -> None:
        self._cursor = 0

    def alloc(self, shape: Sequence[int], dtype: torch.dtype, device: torch.device,
              zero: bool = False) -> Tensor:
        n = math.prod(shape)
        i = self._cursor
        self._cursor += 1
        slot: Optional[Tensor] = self._slots[i] if i < len(self._slots) else None
        if slot is None or slot.dtype != dtype or slot.device != device or slot.numel() < n:
            slot = torch.empty(max(n, 1), dtype=dtype, device=device)
            if i < len(self._slots):
                self._slots[i] = slot
            else:
                self._slots.append(slot)
        out = slot[:n].view(tuple(shape))
        if zero and n:
            out.zero_()
        return out

    def bytes(self) -> int:
        return sum(s.numel() * s.element_size() for s in self._slots)


def alloc(arena: Optional[StepArena], shape, dtype, device, zero: bool = False) -> Tensor:
    """Arena allocation when an arena is given, plain allocation otherwise."""
    if arena is not None:
        return arena.alloc(shape, dtype, device, zero)
    return (torch.zeros if zero else torch.empty)(tuple(shape), dtype=dtype, device=device)
