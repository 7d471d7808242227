"""Single-device Dion in its shortest form: fixed rank, Householder QR, one parameter at a time
(reference: dion/dion_simple.py:18-226).  Intended for reading and for small experiments."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.distributed.tensor import DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from ..ops import foreach as F


@dataclass
class DionMixedPrecisionConfig:
    momentum_dtype: Optional[torch.dtype] = None
    Q_dtype: Optional[torch.dtype] = None


def dion_update(X: Tensor, G: Tensor, M: Tensor, Q: Tensor, lr, mu, weight_decay,
                epsilon=1e-8) -> None:
    """One Dion step on a single matrix, all state updated in place."""
    lr, mu, wd, eps = float(lr), float(mu), float(weight_decay), float(epsilon)
    M.add_(G.to(M.dtype))
    P = torch.linalg.qr((M @ Q.to(M.dtype)).to(torch.float32))[0].to(M.dtype)
    R = M.T @ P
    M.addmm_(P, R.T, alpha=-(1 - mu))                      # error feedback
    R32 = R.to(torch.float32)
    Q.copy_((R32 / (R32.norm(dim=0, keepdim=True) + eps)).to(Q.dtype))
    X.mul_(1 - wd * lr)
    X.addmm_(P.to(X.dtype), Q.T.to(X.dtype), alpha=-lr * (X.size(0) / X.size(1)) ** 0.5)


class Dion(Optimizer):
    """``rank`` is an absolute number of columns (clamped to the matrix size); ``Q`` is
    ``[cols, rank]`` and no transposition heuristics are applied."""

    def __init__(self, params: ParamsT, lr: float, mu: float = 0.95,
                 betas: Tuple[float, float] = (0.9, 0.95), weight_decay: float = 0.01,
                 rank: int = 768, epsilon: float = 1e-8,
                 mixed_precision_config: Optional[DionMixedPrecisionConfig] = None):
        checks = (("learning rate", lr, lr >= 0.0), ("momentum factor (mu)", mu, mu >= 0.0),
                  ("betas", betas, len(betas) == 2 and min(betas) >= 0.0),
                  ("weight_decay value", weight_decay, weight_decay >= 0.0),
                  ("rank value", rank, rank >= 1))
        for what, value, ok in checks:
            if not ok:
                raise ValueError(f"Invalid {what}: {value}")
        defaults = dict(lr=lr, mu=mu, beta1=betas[0], beta2=betas[1], weight_decay=weight_decay,
                        algorithm="dion", step=0)
        super().__init__(params, defaults)
        self.rank = rank
        self.epsilon = torch.tensor(epsilon)
        self._mixed_precision_config = mixed_precision_config or DionMixedPrecisionConfig()
        matrices = [p for g in self.param_groups if g["algorithm"] == "dion" for p in g["params"]]
        for p in matrices:
            if p.dim() != 2:
                raise ValueError(f"Expected Dion parameters to be 2D tensor, but got {p.dim()}D.")
            if isinstance(p, DTensor):
                raise NotImplementedError(
                    "This version of Dion optimizer does not support distributed tensors.")

    def _new_state(self, p: Tensor, algo: str) -> dict:
        mp = self._mixed_precision_config
        if algo == "dion":
            r = min(self.rank, min(p.shape))
            return {"momentum": torch.zeros_like(p, dtype=mp.momentum_dtype or p.dtype),
                    "Q": torch.randn((p.size(1), r), device=p.device, dtype=mp.Q_dtype or p.dtype)}
        state = {"momentum": torch.zeros_like(p)}
        if algo == "adamw":
            state["variance"] = torch.zeros_like(p)
        return state

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            algo = group["algorithm"]
            if algo not in ("dion", "adamw", "lion"):
                raise ValueError(f"Unknown algorithm: {algo}")
            group["step"] += 1
            for p in (q for q in group["params"] if q.grad is not None):
                st = self.state[p]
                if len(st) == 0:
                    st.update(self._new_state(p, algo))
                if algo == "dion":
                    dion_update(p, p.grad, st["momentum"], st["Q"], group["lr"], group["mu"],
                                group["weight_decay"], self.epsilon)
                elif algo == "adamw":
                    F.adamw([p], [p.grad], [st["momentum"]], [st["variance"]], group["lr"],
                            group["beta1"], group["beta2"], group["weight_decay"],
                            float(self.epsilon), step=group["step"])
                else:
                    F.lion([p], [p.grad], [st["momentum"]], group["lr"], group["beta1"],
                           group["beta2"], group["weight_decay"])
        return loss
