#!/usr/bin/env python
"""Roofline microbenchmarks of the memory-bound kernels and the batched factorizations.

    python benchmark/bench_kernels.py                 # every kernel, one JSON line each
    python benchmark/bench_kernels.py --only ce       # one kernel (used for ncu captures)

For each kernel: algorithmic bytes (what must be read and written once), CUDA-event time after
warm-up with an L2 flush before every timed launch, achieved GB/s and the fraction of the
measured copy bandwidth (``hbm_gbs`` of MEASURED_PEAKS.json; 6650 GB/s if the file is absent).
Shapes are those of the GPT-160M step (32768 tokens, d = 768, vocab 50304) and of a GPT-1B
optimizer bucket.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from dion_b200.models import functional as Fn  # noqa: E402
from dion_b200.ops import foreach as F  # noqa: E402
from dion_b200.ops import lowrank as LR  # noqa: E402
from dion_b200.ops import select as SEL  # noqa: E402


def hbm_peak() -> float:
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


_flush = None


def timed(fn, iters=10, warmup=3, inner=4):
    """Mean time of one call; ``inner`` calls are queued back to back per measurement so that
    short kernels are not timed by the host's launch latency (their working sets are several
    times the L2, so the calls do not feed each other from cache)."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(inner):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1) / inner
    return total / iters


def cases():
    dev = "cuda"
    T, C, V = 32768, 768, 50304
    bf, f32 = torch.bfloat16, torch.float32
    out = {}

    x = torch.randn(T, C, device=dev)
    delta = torch.randn(T, C, device=dev).to(bf)

    def rms_fwd():
        with torch.autocast("cuda", dtype=bf):
            Fn.add_rms_norm(x, delta)
    out["add_rms_norm_fwd"] = (rms_fwd, T * C * (4 + 2 + 4 + 2))

    xr = x.clone().requires_grad_()
    dr = delta.clone().requires_grad_()
    with torch.autocast("cuda", dtype=bf):
        xn, h = Fn.add_rms_norm(xr, dr)
    gx, gh = torch.randn_like(xn), torch.randn_like(h)

    def rms_bwd():
        torch.autograd.grad((xn, h), (xr, dr), (gx, gh), retain_graph=True)
    out["add_rms_norm_bwd"] = (rms_bwd, T * C * (4 + 2 + 4 + 4 + 2))

    act = torch.randn(T, 4 * C, device=dev).to(bf).requires_grad_()
    out["relu2_fwd"] = (lambda: Fn.relu2(act.detach()), T * 4 * C * 4)
    y = Fn.relu2(act)
    gy = torch.randn_like(y)
    out["relu2_bwd"] = (lambda: torch.autograd.grad(y, act, gy, retain_graph=True), T * 4 * C * 6)

    logits = torch.randn(T // 4, V, device=dev).to(bf)
    tgt = torch.randint(0, V, (T // 4,), device=dev)

    def ce():
        lg = logits.detach().requires_grad_()
        Fn.cross_entropy(lg, tgt)
    out["ce"] = (ce, (T // 4) * V * 4)

    W = torch.randn(V, C, device=dev, requires_grad=True)
    idx = torch.randint(0, V, (32, 1024), device=dev)
    emb = Fn.embedding(idx, W)
    ge = torch.randn_like(emb)
    out["embedding_bwd"] = (lambda: torch.autograd.grad(emb, W, ge, retain_graph=True),
                            T * C * 4 + V * C * 4)

    # Optimizer kernels on a GPT-1B-sized bucket: 24 matrices of 2048 x 2048 (bf16 weights).
    n, d = 24, 2048
    G = [torch.randn(d, d, device=dev).to(bf) for _ in range(n)]
    M = [torch.zeros(d, d, device=dev, dtype=bf) for _ in range(n)]
    X = [torch.randn(d, d, device=dev).to(bf) for _ in range(n)]
    U = [torch.empty(d, d, device=dev, dtype=bf) for _ in range(n)]
    lr = F.device_scalar(0.02, torch.device(dev))
    out["muon_pre"] = (lambda: F.muon_pre(G, M, 0.95, True, out=U), n * d * d * (2 + 2 + 2 + 2))
    out["muon_post"] = (lambda: F.muon_post(X, U, lr, 0.01, 1.0), n * d * d * (2 + 2 + 2))
    Xf = [torch.randn(d, d, device=dev) for _ in range(8)]
    Gf = [torch.randn(d, d, device=dev) for _ in range(8)]
    Mf = [torch.zeros(d, d, device=dev) for _ in range(8)]
    Vf = [torch.zeros(d, d, device=dev) for _ in range(8)]
    steps = [torch.zeros((), device=dev) for _ in range(8)]
    out["adamw_fp32"] = (lambda: F.adamw(Xf, Gf, Mf, Vf, lr, 0.9, 0.95, 0.01, 1e-8,
                                         state_steps=steps), 8 * d * d * 4 * 7)
    out["dion2_select_rows"] = (lambda: SEL.dion2_select(G, M, d // 4, -2, 0.95, True),
                                n * d * d * (2 + 2 + 2) + n * (d // 4) * d * (2 + 2 + 2))

    A = torch.randn(48, 256, 192, device=dev)
    out["qr_r_factor_48x256x192"] = (lambda: LR.qr_r_factor(A), A.numel() * 4)
    A2 = torch.randn(96, 640, 512, device=dev)
    out["qr_r_factor_96x640x512"] = (lambda: LR.qr_r_factor(A2), A2.numel() * 4)
    Gm = A2.mT @ A2
    out["cholesky_96x512"] = (lambda: LR.cholesky_upper(Gm), Gm.numel() * 8)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    peak = hbm_peak()
    for name, (fn, nbytes) in cases().items():
        if args.only and args.only != name:
            continue
        ms = timed(fn, iters=args.iters)
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "algorithmic_MB": round(nbytes / 1e6, 1),
                          "GBs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peak, 3)}),
              flush=True)


if __name__ == "__main__":
    main()
