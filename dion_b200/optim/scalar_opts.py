"""AdamW and Lion for the non-matrix parameter groups, under the function names the reference
exposes (dion/scalar_opts.py:7-342).  The work is done by ``ops.foreach``: one multi-tensor CUDA
kernel per call on the GPU, plain PyTorch elsewhere."""
from __future__ import annotations

from typing import Generator, List, Optional

from torch import Tensor

from ..ops import foreach as F


def adamw_update(X: Tensor, G: Tensor, M: Tensor, V: Tensor, lr, beta1, beta2, weight_decay,
                 step: int, epsilon: float, cautious_wd: bool = False) -> None:
    """Single-tensor AdamW with a host-side step count."""
    F.adamw([X], [G], [M], [V], lr, float(beta1), float(beta2), weight_decay, float(epsilon),
            step=int(step), cautious_wd=cautious_wd)


def lion_update(X: Tensor, G: Tensor, M: Tensor, lr, beta1, beta2, weight_decay,
                cautious_wd: bool = False) -> None:
    """Single-tensor Lion."""
    F.lion([X], [G], [M], lr, float(beta1), float(beta2), weight_decay, cautious_wd=cautious_wd)


def adamw_update_foreach(
    X: List[Tensor], G: List[Tensor], M: List[Tensor], V: List[Tensor], lr, beta1, beta2,
    weight_decay, step: Optional[int] = None, epsilon: float = 1e-8, cautious_wd: bool = False,
    state_steps: Optional[List[Tensor]] = None,
) -> None:
    """AdamW over lists.  ``step`` (host int, baked into the launch) or ``state_steps``
    (per-tensor fp32 device counters advanced on the device, CUDA-graph capturable; requires a
    tensor ``lr``) - exactly one of the two.  A device-tensor ``weight_decay`` is read live."""
    F.adamw(X, G, M, V, lr, float(beta1), float(beta2), weight_decay, float(epsilon),
            step=step, state_steps=state_steps, cautious_wd=cautious_wd)


def lion_update_foreach(X: List[Tensor], G: List[Tensor], M: List[Tensor], lr, beta1, beta2,
                        weight_decay, cautious_wd: bool = False) -> None:
    F.lion(X, G, M, lr, float(beta1), float(beta2), weight_decay, cautious_wd=cautious_wd)


def adamw_update_foreach_async(*args, **kwargs) -> Generator[None, None, None]:
    adamw_update_foreach(*args, **kwargs)
    yield


def lion_update_foreach_async(*args, **kwargs) -> Generator[None, None, None]:
    lion_update_foreach(*args, **kwargs)
    yield
