#!/usr/bin/env python
"""Newton-Schulz sweep: time and TFLOP/s of the orthogonalization drivers on batched bf16
matrices, against PyTorch (cuBLAS) and, when ``baseline/_ref`` is installed, the reference's
Triton kernels.

    python benchmark/bench_newton_schulz.py --grid            # shapes x batch sizes
    python benchmark/bench_newton_schulz.py --single 4096 4096 --batch 8
    python benchmark/bench_newton_schulz.py --gemms 2048 2048 --batch 24   # per-GEMM breakdown
    python benchmark/bench_newton_schulz.py --sweep --expansion 4          # d x 4d, speed-ups
    python benchmark/bench_newton_schulz.py --curve --batch 4 --out-dir plots  # TFLOP/s vs size

FLOP model (the reference's, benchmark/benchmark_newton_shultz.py:40-48): ``4 m^2 n + 2 m^3``
per iteration with ``m <= n``, i.e. without crediting the symmetric half-work, so the numbers
are directly comparable; the fraction of the measured cuBLAS bf16 peak is reported alongside.
Entries are N(0,1), timed with CUDA events after warm-up; between timed runs a buffer larger
than L2 is overwritten.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from dion_b200.ops import gemm  # noqa: E402
from dion_b200.ops import newton_schulz as NS  # noqa: E402

GRID_SHAPES = [(768, 768), (768, 3072), (2048, 8192), (4096, 4096), (8192, 8192)]
GRID_BATCH = [1, 4, 16, 64]


def peak_tflops() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops"])
    except Exception:
        return 1590.0  # fallback when no measured-peaks file is present: cuBLAS bf16 burst on a B200


def ns_flops(b: int, m: int, n: int, iters: int = 5) -> float:
    m, n = min(m, n), max(m, n)
    return b * iters * (4.0 * m * m * n + 2.0 * m ** 3)


_flush = None


def flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def bench(fn, iters: int = 10, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def graphed(fn, G):
    """``fn(G)`` captured once in a CUDA graph; returns a callable that replays it (device time
    without the per-launch host cost, which is what a captured optimizer or training step pays)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn(G)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn(G)
    return graph.replay


def reference_drivers():
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "dion")):
        return {}
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"], os.environ["CC"] = "/usr/bin/g++", "/usr/bin/gcc"
    sys.path.insert(1, ref_root)
    try:
        from dion.newton_schulz_triton import newton_schulz_triton
        from dion.polar_express import polar_express_triton
        return {"ref_triton_quintic": newton_schulz_triton, "ref_triton_pe": polar_express_triton}
    except Exception as exc:  # noqa: BLE001
        print(f"# reference kernels unavailable: {exc}", file=sys.stderr)
        return {}


def run_case(b: int, m: int, n: int, drivers, peak: float, max_bytes: float = 6e9,
             graph_too: bool = False):
    if b * m * n * 2 * 4 > max_bytes:
        return None
    G = torch.randn(b, m, n, device="cuda", dtype=torch.bfloat16)
    G = G / G.float().norm(dim=(-2, -1), keepdim=True).to(G.dtype)
    row = {"batch": b, "m": m, "n": n}
    fl = ns_flops(b, m, n)
    for name, fn in drivers.items():
        try:
            ms = bench(lambda: fn(G))
        except Exception as exc:  # noqa: BLE001
            row[name] = {"error": str(exc)[:120]}
            continue
        tf = fl / (ms * 1e-3) / 1e12
        row[name] = {"ms": round(ms, 4), "tflops": round(tf, 1),
                     "frac_of_measured_cublas_peak": round(tf / peak, 3)}
        if graph_too and name.startswith("ours_quintic"):
            try:
                replay = graphed(fn, G)
                gms = bench(replay)
                row[name + "_graphed"] = {"ms": round(gms, 4),
                                          "tflops": round(fl / (gms * 1e-3) / 1e12, 1)}
            except Exception as exc:  # noqa: BLE001
                row[name + "_graphed"] = {"error": str(exc)[:120]}
    gemm.check_status()
    return row


def gemm_breakdown(b: int, m: int, n: int):
    X = torch.randn(b, m, n, device="cuda").bfloat16()
    A = torch.empty(b, m, m, device="cuda", dtype=torch.bfloat16)
    Bm = torch.empty_like(A)
    C = torch.empty_like(X)
    out = {}
    cases = {}
    for tag, pair in (("1cta", False), ("2cta", True)):
        cases[f"gram  A=XX^T (sym) {tag}"] = (
            lambda pair=pair: gemm.ns_gemm(X, X, out=A, sym=True, pair=pair), 2.0 * b * m * m * n)
        cases[f"poly  B=bA+cA^2 (sym) {tag}"] = (
            lambda pair=pair: gemm.ns_gemm(A, A, out=Bm, sym=True, D=A, alpha=1.0, beta=1.0,
                                           pair=pair), 2.0 * b * m ** 3)
        cases[f"upd   X'=aX+BX {tag}"] = (
            lambda pair=pair: gemm.ns_gemm(Bm, X, out=C, b_is_kn=True, D=X, alpha=1.0, beta=1.0,
                                           pair=pair), 2.0 * b * m * m * n)
    cases["gram  cuBLAS bmm"] = (lambda: torch.bmm(X, X.mT, out=A), 2.0 * b * m * m * n)
    cases["upd   cuBLAS baddbmm"] = (lambda: torch.baddbmm(X, Bm, X, out=C), 2.0 * b * m * m * n)
    for name, (fn, fl) in cases.items():
        ms = bench(fn)
        out[name] = {"ms": round(ms, 4), "nominal_tflops": round(fl / (ms * 1e-3) / 1e12, 1)}
    gemm.check_status()
    return out


def speedup_sweep(dims, expansion: int, batch: int, drivers, peak: float):
    """Square / rectangular sweep ``d x (d * expansion)`` with the speed-up of the symmetric
    kernels over the plain-PyTorch iteration and its upper bound ``(4e + 2) / (3e + 1)`` from
    skipping the mirrored half of the two symmetric products (the reference prints the same
    summary, benchmark/benchmark_newton_shultz.py:90-108)."""
    rows, ups = [], []
    for d in dims:
        row = run_case(batch, d, d * expansion, drivers, peak, max_bytes=24e9)
        if row is None:
            continue
        rows.append(row)
        print(json.dumps(row), flush=True)
        if "ms" in row.get("ours_quintic", {}) and "ms" in row.get("torch_quintic", {}):
            ups.append(row["torch_quintic"]["ms"] / row["ours_quintic"]["ms"])
    print("speed-up over torch:", ", ".join(f"{u:4.2f}x" for u in ups))
    print(f"bound from symmetry alone: {(4 * expansion + 2) / (3 * expansion + 1):4.2f}x")
    return rows


def write_curve(rows, names, out_dir: str, title: str) -> str:
    """TFLOP/s against matrix size as a CSV file and a text chart (and a PNG when matplotlib is
    importable; the reference draws this with Triton's perf_report,
    benchmark/benchmark_newton_shultz.py:111-137).  Returns the CSV path."""
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, title + ".csv")
    with open(path, "w") as f:
        f.write("dim," + ",".join(names) + "\n")
        for row in rows:
            f.write(str(row["m"]) + "," + ",".join(
                str(row.get(n, {}).get("tflops", "")) for n in names) + "\n")
    top = max([row.get(n, {}).get("tflops", 0.0) for row in rows for n in names] + [1e-9])
    for row in rows:
        for n in names:
            tf = row.get(n, {}).get("tflops")
            if tf is not None:
                print(f"{row['m']:6d} {n:22s} {tf:8.1f} " + "#" * int(round(50 * tf / top)))
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        for n in names:
            plt.plot([r["m"] for r in rows], [r.get(n, {}).get("tflops", float("nan")) for r in rows],
                     marker="o", label=n)
        plt.xlabel("dim"); plt.ylabel("TFLOPS"); plt.legend(); plt.title(title)
        plt.savefig(os.path.join(out_dir, title + ".png"), dpi=120)
    except ImportError:
        pass
    return path


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--grid", action="store_true")
    ap.add_argument("--single", nargs=2, type=int, metavar=("M", "N"))
    ap.add_argument("--gemms", nargs=2, type=int, metavar=("M", "N"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-reference", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="also time our quintic driver replayed from a CUDA graph")
    ap.add_argument("--out", type=str, default=None)
    ap.add_argument("--sweep", action="store_true",
                    help="d x (d*expansion) for d in 512..8192 with speed-ups over torch")
    ap.add_argument("--expansion", type=int, default=1)
    ap.add_argument("--curve", action="store_true",
                    help="TFLOP/s for dim = 128..896 (CSV, text chart, PNG with matplotlib)")
    ap.add_argument("--out-dir", type=str, default="plots")
    args = ap.parse_args()
    peak = peak_tflops()
    drivers = {
        "ours_quintic": NS.newton_schulz_quintic,
        "ours_polar_express": NS.polar_express,
        "ours_gram_ns": NS.gram_newton_schulz,
        "ours_aol4": NS.newton_schulz_aol,
        "torch_quintic": NS.torch_reference("quintic"),
    }
    if not args.no_reference:
        drivers.update(reference_drivers())
    results = []
    if args.gemms:
        r = gemm_breakdown(args.batch, *args.gemms)
        print(json.dumps({"gemm_breakdown": r, "batch": args.batch, "shape": args.gemms}, indent=1))
        return
    if args.sweep:
        results = speedup_sweep([512, 1024, 2048, 4096, 8192], args.expansion, args.batch,
                                drivers, peak)
        if args.out:
            json.dump({"measured_cublas_bf16_peak_tflops": peak, "rows": results},
                      open(args.out, "w"), indent=1)
        return
    if args.curve:
        rows = [r for r in (run_case(args.batch, 128 * i, 128 * i, drivers, peak)
                            for i in range(1, 8)) if r is not None]
        print("wrote", write_curve(rows, list(drivers), args.out_dir,
                                   f"newton_schulz_batch{args.batch}"))
        return
    cases = ([(b, m, n) for (m, n) in GRID_SHAPES for b in GRID_BATCH] if args.grid
             else [(args.batch, *(args.single or (4096, 4096)))])
    for b, m, n in cases:
        row = run_case(b, m, n, drivers, peak, graph_too=args.graph)
        if row is None:
            continue
        results.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        json.dump({"measured_cublas_bf16_peak_tflops": peak, "rows": results},
                  open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
