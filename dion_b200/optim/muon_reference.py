"""Per-parameter Muon variants without megabatching (reference: dion/muon_reference.py:32-337).

``Muon`` orthogonalizes one parameter at a time with the classic fixed-coefficient quintic
Newton-Schulz iteration; a DTensor parameter is gathered in full, orthogonalized on every rank
and re-sharded.  ``MuonKellerJordan`` round-robins whole parameters over the ranks and sums the
updates with one all-reduce.  Both are baselines for the megabatch optimizer, not fast paths;
the Newton-Schulz iteration still runs on the tcgen05 kernels when the tensors are on a GPU.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed.tensor import DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from ..ops.newton_schulz import newton_schulz_classic


def zeropower_via_newtonschulz5(G: Tensor, steps: int = 5, eps: float = 1e-7) -> Tensor:
    """Quintic Newton-Schulz with the fixed coefficients (3.4445, -4.7750, 2.0315)."""
    assert G.ndim == 2
    return newton_schulz_classic(G, epsilon=eps, steps=steps)


class Muon(Optimizer):
    """Muon with per-parameter orthogonalization.  Param groups choose ``algorithm`` in
    ``{"muon", "adamw", "lion"}``; the choice is stored per parameter in ``state[p]``."""

    def __init__(self, params: ParamsT, lr: float = 1e-3, mu: float = 0.95,
                 betas: Tuple[float, float] = (0.95, 0.95), weight_decay: float = 0.1,
                 epsilon: float = 1e-8, nesterov: bool = True,
                 adjust_lr: Optional[str] = "spectral_norm", ns_steps: int = 5):
        if adjust_lr not in ("spectral_norm", "rms_norm", None):
            raise ValueError(
                f"Invalid adjust_lr value: {adjust_lr}. Must be 'spectral_norm', 'rms_norm', or None.")
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=mu, nesterov=nesterov,
                        ns_steps=ns_steps, adjust_lr=adjust_lr, betas=betas, epsilon=epsilon)
        params = list(params) if not isinstance(params, dict) else [params]
        super().__init__(params, defaults)
        for entry in params:
            if isinstance(entry, dict):
                algo = entry.get("algorithm", "muon")
                if algo not in ("muon", "adamw", "lion"):
                    raise ValueError(f"Unknown algorithm: {algo}")
                members = entry["params"]
                members = [members] if isinstance(members, Tensor) else list(members)
            elif isinstance(entry, Tensor):
                algo, members = "muon", [entry]
            elif isinstance(entry, tuple) and len(entry) == 2:
                algo, members = "muon", [entry[1]]
            else:
                raise ValueError(f"Invalid parameter type: {type(entry)}")
            for p in members:
                self.state[p]["algorithm"] = algo
                if algo == "muon" and p.ndim != 2:
                    raise ValueError(f"Muon requires 2D parameters, but got {p.ndim}D")

    @staticmethod
    def _adjusted_lr(rule, lr, shape):
        if rule is None:
            return lr
        a, b = shape[:2]
        if rule == "spectral_norm":
            return lr * math.sqrt(a / b)
        if rule == "rms_norm":
            return lr * 0.2 * math.sqrt(max(a, b))
        raise ValueError(f"Unknown adjust_lr value: {rule}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd, eps = group["lr"], group["weight_decay"], group["epsilon"]
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self.state[p]
                algo = st["algorithm"]
                if algo == "muon":
                    if g.ndim > 2:
                        g = g.view(g.size(0), -1)
                    buf = st.get("momentum_buffer")
                    if buf is None:
                        buf = st["momentum_buffer"] = torch.zeros_like(g)
                    buf.mul_(group["momentum"]).add_(g)
                    g = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    if isinstance(g, DTensor):
                        full = zeropower_via_newtonschulz5(g.full_tensor(), group["ns_steps"], eps)
                        u = DTensor.from_local(full, device_mesh=g.device_mesh, placements=None,
                                               run_check=False).redistribute(placements=g.placements)
                    else:
                        u = zeropower_via_newtonschulz5(g, group["ns_steps"], eps)
                    p.mul_(1 - lr * wd)
                    p.add_(u.to(p.dtype), alpha=-self._adjusted_lr(group["adjust_lr"], lr, p.shape))
                elif algo == "adamw":
                    if "step" not in st:
                        st["step"] = 0
                        st["moment1"] = torch.zeros_like(g)
                        st["moment2"] = torch.zeros_like(g)
                    st["step"] += 1
                    t = st["step"]
                    st["moment1"].lerp_(g, 1 - beta1)
                    st["moment2"].lerp_(g.square(), 1 - beta2)
                    upd = st["moment1"] / (eps + st["moment2"].sqrt())
                    scale = (1 - beta1 ** t) / (1 - beta2 ** t) ** 0.5
                    p.mul_(1 - lr * wd)
                    p.add_(upd, alpha=-lr / scale)
                else:  # lion
                    buf = st.get("momentum_buffer")
                    if buf is None:
                        buf = st["momentum_buffer"] = torch.zeros_like(p)
                    upd = buf.lerp(g, 1 - beta1).sign_()
                    buf.lerp_(g, 1 - beta2)
                    p.mul_(1 - lr * wd)
                    p.add_(upd, alpha=-lr)
        return loss


class MuonKellerJordan(Optimizer):
    """Whole parameters are dealt round-robin to the ranks (``RANK`` / ``WORLD_SIZE`` from the
    environment); each rank orthogonalizes its share and one all-reduce of a flat bf16 buffer
    distributes the updates."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps))
        for group in self.param_groups:
            if any(isinstance(p, DTensor) for p in group["params"]):
                raise NotImplementedError("DTensor parameters not supported.")

    @torch.no_grad()
    def step(self):
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        for group in self.param_groups:
            params = group["params"]
            if not params:
                continue
            flat = torch.zeros(sum(p.numel() for p in params), device=params[0].device,
                               dtype=torch.bfloat16)
            off = 0
            for i, p in enumerate(params):
                if i % world == rank:
                    g = p.grad
                    assert g is not None, "Gradient is None"
                    st = self.state[p]
                    buf = st.get("momentum_buffer")
                    if buf is None:
                        buf = st["momentum_buffer"] = torch.zeros_like(g)
                    buf.mul_(group["momentum"]).add_(g)
                    g = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    u = zeropower_via_newtonschulz5(g, steps=group["ns_steps"])
                    flat[off:off + p.numel()] = (u * (g.size(0) / g.size(1)) ** 0.5).flatten()
                off += p.numel()
            if world > 1 and dist.is_initialized():
                dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            off = 0
            for p in params:
                p.add_(flat[off:off + p.numel()].view_as(p).type_as(p), alpha=-group["lr"])
                off += p.numel()
