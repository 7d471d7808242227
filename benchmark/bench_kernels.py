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


T, C, V = 32768, 768, 50304
DEV = "cuda"
BF, F32 = torch.bfloat16, torch.float32
CASES = {}


def case(name):
    """Register ``builder() -> (callable, algorithmic bytes)`` under ``name``; inputs are built
    only for the cases that run, so a capture of one kernel holds little else on the device."""
    def deco(builder):
        CASES[name] = builder
        return builder
    return deco


@case("add_rms_norm_fwd")
def _():
    x = torch.randn(T, C, device=DEV)
    delta = torch.randn(T, C, device=DEV).to(BF)

    def run():
        with torch.autocast("cuda", dtype=BF):
            Fn.add_rms_norm(x, delta)
    return run, T * C * (4 + 2 + 4 + 2)


@case("add_rms_norm_bwd")
def _():
    xr = torch.randn(T, C, device=DEV).requires_grad_()
    dr = torch.randn(T, C, device=DEV).to(BF).requires_grad_()
    with torch.autocast("cuda", dtype=BF):
        xn, h = Fn.add_rms_norm(xr, dr)
    gx, gh = torch.randn_like(xn), torch.randn_like(h)
    return (lambda: torch.autograd.grad((xn, h), (xr, dr), (gx, gh), retain_graph=True),
            T * C * (4 + 2 + 4 + 4 + 2))


def _act():
    return torch.randn(T, 4 * C, device=DEV).to(BF).requires_grad_()


@case("relu2_fwd")
def _():
    act = _act()
    return (lambda: Fn.relu2(act.detach())), T * 4 * C * 4


@case("relu2_bwd")
def _():
    act = _act()
    y = Fn.relu2(act)
    gy = torch.randn_like(y)
    return (lambda: torch.autograd.grad(y, act, gy, retain_graph=True)), T * 4 * C * 6


@case("ce")
def _():
    logits = torch.randn(T // 4, V, device=DEV).to(BF)
    tgt = torch.randint(0, V, (T // 4,), device=DEV)

    def run():
        lg = logits.detach().requires_grad_()
        Fn.cross_entropy(lg, tgt)
    return run, (T // 4) * V * 4


@case("embedding_bwd")
def _():
    W = torch.randn(V, C, device=DEV, requires_grad=True)
    idx = torch.randint(0, V, (32, 1024), device=DEV)
    emb = Fn.embedding(idx, W)
    ge = torch.randn_like(emb)
    return (lambda: torch.autograd.grad(emb, W, ge, retain_graph=True)), T * C * 4 + V * C * 4


# Optimizer kernels on a GPT-1B-sized bucket: 24 matrices of 2048 x 2048 (bf16 weights).
N_MAT, D_MAT = 24, 2048


def _bucket(kind, n=N_MAT, dtype=BF):
    make = {"randn": lambda: torch.randn(D_MAT, D_MAT, device=DEV).to(dtype),
            "zeros": lambda: torch.zeros(D_MAT, D_MAT, device=DEV, dtype=dtype),
            "empty": lambda: torch.empty(D_MAT, D_MAT, device=DEV, dtype=dtype)}[kind]
    return [make() for _ in range(n)]


@case("muon_pre")
def _():
    G, M, U = _bucket("randn"), _bucket("zeros"), _bucket("empty")
    return (lambda: F.muon_pre(G, M, 0.95, True, out=U)), N_MAT * D_MAT * D_MAT * (2 + 2 + 2 + 2)


@case("muon_post")
def _():
    X, U = _bucket("randn"), _bucket("randn")
    lr = F.device_scalar(0.02, torch.device(DEV))
    return (lambda: F.muon_post(X, U, lr, 0.01, 1.0)), N_MAT * D_MAT * D_MAT * (2 + 2 + 2)


@case("adamw_fp32")
def _():
    Xf, Gf = _bucket("randn", 8, F32), _bucket("randn", 8, F32)
    Mf, Vf = _bucket("zeros", 8, F32), _bucket("zeros", 8, F32)
    steps = [torch.zeros((), device=DEV) for _ in range(8)]
    lr = F.device_scalar(0.02, torch.device(DEV))
    return (lambda: F.adamw(Xf, Gf, Mf, Vf, lr, 0.9, 0.95, 0.01, 1e-8, state_steps=steps),
            8 * D_MAT * D_MAT * 4 * 7)


@case("lion_fp32")
def _():
    Xf, Gf, Mf = _bucket("randn", 8, F32), _bucket("randn", 8, F32), _bucket("zeros", 8, F32)
    lr = F.device_scalar(0.02, torch.device(DEV))
    return (lambda: F.lion(Xf, Gf, Mf, lr, 0.9, 0.99, 0.01)), 8 * D_MAT * D_MAT * 4 * 5


@case("normuon_rowstats")
def _():
    U = torch.randn(N_MAT, D_MAT, D_MAT, device=DEV).to(BF)
    Vs = [torch.zeros(D_MAT, 1, device=DEV) for _ in range(N_MAT)]
    return (lambda: F.normuon_rowstats(U, Vs, 0.95)), N_MAT * D_MAT * D_MAT * 2


@case("dion2_select_rows")
def _():
    G, M = _bucket("randn"), _bucket("zeros")
    d = D_MAT
    return (lambda: SEL.dion2_select(G, M, d // 4, -2, 0.95, True),
            N_MAT * d * d * (2 + 2 + 2) + N_MAT * (d // 4) * d * (2 + 2 + 2))


@case("qr_r_factor_48x256x192")
def _():
    A = torch.randn(48, 256, 192, device=DEV)
    return (lambda: LR.qr_r_factor(A)), A.numel() * 4


@case("qr_r_factor_96x640x512")
def _():
    A = torch.randn(96, 640, 512, device=DEV)
    return (lambda: LR.qr_r_factor(A)), A.numel() * 4


@case("cholesky_96x512")
def _():
    A = torch.randn(96, 640, 512, device=DEV)
    Gm = A.mT @ A
    return (lambda: LR.cholesky_upper(Gm)), Gm.numel() * 8


# ---- low-rank (Dion) kernels: 24 matrices of 2048 x 2048 in fp32, rank 512 -----------------------
LR_B, LR_D, LR_R = 24, 2048, 512
FLOPS = {}   # kernel name -> floating-point operations per call (reported as TFLOP/s)


def _lr_inputs():
    g = torch.Generator(device=DEV).manual_seed(0)
    M = torch.randn(LR_B, LR_D, LR_D, device=DEV, generator=g)
    Q = torch.randn(LR_B, LR_D, LR_R, device=DEV, generator=g) / LR_D ** 0.5
    return M, Q


@case("lowrank_p_gemm_tf32")
def _():
    """P = M Q: M read once in fp32 (K-major), Q as a [K, N] operand."""
    M, Q = _lr_inputs()
    FLOPS["lowrank_p_gemm_tf32"] = 2.0 * LR_B * LR_D * LR_D * LR_R
    return (lambda: LR.power_iteration_p(M, Q, False)), \
        LR_B * (LR_D * LR_D + 2 * LR_D * LR_R) * 4


@case("lowrank_r_gemm_tf32")
def _():
    """R = M^T P: M read in place as an MN-major tf32 operand."""
    M, Q = _lr_inputs()
    FLOPS["lowrank_r_gemm_tf32"] = 2.0 * LR_B * LR_D * LR_D * LR_R
    return (lambda: LR.power_iteration_r(M, Q, False)), \
        LR_B * (LR_D * LR_D + 2 * LR_D * LR_R) * 4


@case("lowrank_p_gemm_reduce")
def _():
    """P = M Q with the epilogue adding every tile into per-matrix accumulators (the local form
    of the reduce-scatter over peer memory: the same red.add instructions, targets in this
    GPU's memory)."""
    M, Q = _lr_inputs()
    acc = torch.zeros(LR_B, LR_D, LR_R, device=DEV)
    where = torch.tensor([acc[b].data_ptr() for b in range(LR_B)], dtype=torch.int64).to(DEV)
    FLOPS["lowrank_p_gemm_reduce"] = 2.0 * LR_B * LR_D * LR_D * LR_R
    return (lambda: LR.power_iteration_p(M, Q, False, reduce_into=where, alpha=0.5)), \
        LR_B * (LR_D * LR_D + 3 * LR_D * LR_R) * 4


@case("lowrank_rank_update_inplace")
def _():
    """M -= c P R^T in place: the fp32 matrix is read and written once by the GEMM epilogue."""
    M, Q = _lr_inputs()
    P = torch.randn(LR_B, LR_D, LR_R, device=DEV) / LR_R ** 0.5
    FLOPS["lowrank_rank_update_inplace"] = 2.0 * LR_B * LR_D * LR_D * LR_R
    return (lambda: LR.rank_update_stack_(M, P, Q, -0.05, 1.0)), \
        LR_B * (2 * LR_D * LR_D + 2 * LR_D * LR_R) * 4


@case("lowrank_triu_inverse_96x512")
def _():
    A = torch.randn(96, 640, 512, device=DEV)
    U = torch.linalg.qr(A, mode="r")[1].contiguous()
    FLOPS["lowrank_triu_inverse_96x512"] = 96 * 512 ** 3 / 3.0
    return (lambda: LR.triu_inverse(U)), U.numel() * 8


@case("lowrank_orthogonalize_96x2048x512")
def _():
    """The whole randomized Cholesky-QR of 96 factors [2048, 512] (sketch, QR, two inversions,
    Gram, Cholesky, split-precision products)."""
    P = torch.randn(96, 2048, 512, device=DEV)
    return (lambda: LR.orthogonalize(P, 1.25)), P.numel() * 8


@case("philox_sketch_96x640x2048")
def _():
    dev = torch.device(DEV)
    gen = torch.Generator(device=dev).manual_seed(1)
    return (lambda: LR.random_sketch(96, 640, 2048, F32, dev, gen)), 96 * 640 * 2048 * 4


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="one kernel name, or several separated by commas")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    peak = hbm_peak()
    only = [s for s in args.only.split(",") if s] if args.only else []
    for name in only:
        if name not in CASES:
            raise SystemExit(f"unknown kernel {name!r}; one of: {', '.join(CASES)}")
    for name, builder in CASES.items():
        if only and name not in only:
            continue
        fn, nbytes = builder()
        ms = timed(fn, iters=args.iters)
        gbs = nbytes / ms / 1e6
        line = {"kernel": name, "ms": round(ms, 4), "algorithmic_MB": round(nbytes / 1e6, 1),
                "GBs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peak, 3)}
        if name in FLOPS:
            line["TFLOPs"] = round(FLOPS[name] / ms / 1e9, 1)
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
