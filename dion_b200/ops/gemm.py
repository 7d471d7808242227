"""Python front end of the tcgen05 batched GEMM (``csrc/ns_gemm_sm100.cu``).

``ns_gemm`` computes ``C = alpha * s^pa * A @ op(B) + beta * s^pb * D`` on bf16 batches, where
``op(B)`` is ``B^T`` for ``B`` given as ``[N, K]`` and ``B`` itself for ``B`` given as ``[K, N]``.
With ``sym=True`` only the upper-triangle tiles are computed and mirrored.  It stands in for the
reference's three Triton kernels and its cuBLAS ``baddbmm`` call
(dion/newton_schulz_triton.py:160-198, 290-333, 450-491, 557-563).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from . import _backend

_BM = 128
_tile_cache: Dict[Tuple, Tensor] = {}
_tile_hosts: Dict[Tuple, Tensor] = {}
_status: Dict[int, Tensor] = {}
_sm_count: Dict[int, int] = {}

STATUS_MESSAGES = {
    1: "MMA warp timed out waiting for a TMA stage",
    2: "TMA producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for an accumulator",
    4: "MMA warp timed out waiting for a drained accumulator",
    5: "wait on a peer GPU's flag timed out",
    6: "bad arguments",
    7: "grid-wide barrier of a persistent kernel timed out",
}


def status_tensor(device: torch.device) -> Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def _raise_for(idx: int, record) -> None:
    code, who, want, found = (int(v) for v in record)
    if code == 0:
        return
    detail = ""
    if code == 5 and (who or want or found):
        detail = (f" (flag of source rank {who}: waited for sequence {want}, found {found})")
    raise RuntimeError(
        f"dion_b200 kernel error on cuda:{idx}: {STATUS_MESSAGES.get(code, code)}{detail}; "
        f"updates that depended on the missing data were skipped")


def check_status(device: Optional[torch.device] = None) -> None:
    """Read the device status word (synchronizes) and raise if a kernel reported a timeout."""
    devs = list(_status) if device is None else [device.index or 0]
    for idx in devs:
        t = _status.get(idx)
        if t is None:
            continue
        record = t.tolist()
        if record[0] != 0:
            t.zero_()
            _snapshots.pop(idx, None)
            _raise_for(idx, record)


# Non-blocking watch: a copy of the status record in pinned host memory, refreshed by an
# asynchronous copy at the end of each step, read once that copy has completed.
_snapshots: Dict[int, Tuple[Tensor, "torch.cuda.Event"]] = {}


def snapshot_status(device: torch.device) -> None:
    """Queue a copy of the device status record to the host on the current stream (nothing is
    queued while the stream is being captured)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None or torch.cuda.is_current_stream_capturing():
        return
    snap = _snapshots.get(idx)
    if snap is None:
        host = torch.zeros(4, dtype=torch.int32).pin_memory()
        snap = _snapshots[idx] = (host, torch.cuda.Event())
    host, event = snap
    host.copy_(t, non_blocking=True)
    event.record(torch.cuda.current_stream(t.device))


def poll_status(device: torch.device) -> None:
    """Raise if the last completed snapshot shows an error; never waits for the GPU."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    snap = _snapshots.get(idx)
    if snap is None or torch.cuda.is_current_stream_capturing():
        return
    host, event = snap
    if not event.query():
        return
    record = host.tolist()
    if record[0] != 0:
        host.zero_()
        _status[idx].zero_()
        _raise_for(idx, record)


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_count[idx] = n
    return n


def tile_table(M: int, N: int, bn: int, sym: bool, device: torch.device,
               bm: int = _BM) -> Tensor:
    """Device array of (tile_m, tile_n) pairs.  For ``sym`` only tiles that intersect the
    upper triangle (column range reaching the tile's first row) are listed."""
    key = (M, N, bn, sym, device.index, bm)
    t = _tile_cache.get(key)
    if t is not None:
        return t
    tm_n = (M + bm - 1) // bm
    tn_n = (N + bn - 1) // bn
    pairs = []
    for tm in range(tm_n):
        for tn in range(tn_n):
            if sym and (tn + 1) * bn - 1 < tm * bm:
                continue
            pairs.append((tm, tn))
    host = torch.tensor(pairs, dtype=torch.int32)
    if device.type == "cuda" and torch.cuda.is_current_stream_capturing():
        # First use of this shape inside a graph capture: the copy is recorded, so it has to
        # read pinned memory that stays alive as long as the table does.
        host = host.pin_memory()
        _tile_hosts[key] = host
        t = host.to(device, non_blocking=True)
    else:
        t = host.to(device)
    _tile_cache[key] = t
    return t


def _p(t: Optional[Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _as3d(t: Tensor) -> Tensor:
    return t.unsqueeze(0) if t.ndim == 2 else t


def _ld_stride(t: Tensor) -> Tuple[int, int]:
    assert t.stride(-1) == 1, "innermost dimension must be contiguous"
    ld = t.stride(-2) if t.size(-2) > 1 else max(t.stride(-2), t.size(-1))
    bs = t.stride(0) if t.size(0) > 1 else t.size(-2) * ld
    return ld, bs


def supported(A: Tensor, B: Tensor) -> bool:
    """True when the TMA constraints hold (16-byte aligned bases, strides multiples of 8)."""
    for t in (A, B):
        if t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(-1) != 1:
            return False
        if t.data_ptr() % 16 or t.stride(-2) % 8:
            return False
        if t.ndim == 3 and t.size(0) > 1 and t.stride(0) % 8:
            return False
    return True


class GemmExtra(ctypes.Structure):
    """Cross-GPU coupling of one launch (mirrors ``DionGemmExtra`` in csrc/ns_gemm_sm100.cu)."""

    _fields_ = [
        ("wait_flags", ctypes.c_void_p), ("seq_ptr", ctypes.c_void_p),
        ("n_src", ctypes.c_int), ("rows_per_src", ctypes.c_int),
        ("wait_a", ctypes.c_int), ("wait_b", ctypes.c_int), ("wait_k", ctypes.c_int),
        ("scale_partials", ctypes.c_void_p),
        ("scale_mult", ctypes.c_float), ("scale_eps", ctypes.c_float),
        ("remote_c", ctypes.c_longlong * 8),
        ("rows_per_dst", ctypes.c_int), ("remote_slot", ctypes.c_int),
        ("cols_per_dst", ctypes.c_int),
    ]


_EPILOGUES = {"axpby": 0, "relu2": 1, "mul_2sqrt": 2}


def pair_default() -> bool:
    """Whether eligible GEMMs go to the two-CTA kernel (``DION_B200_PAIR_GEMM``, default on)."""
    return os.environ.get("DION_B200_PAIR_GEMM", "1") != "0"


def pair_exchange() -> bool:
    """Whether launches coupled to other GPUs (flag-gated loads, rows stored to their owners) may
    use the two-CTA kernel (``DION_B200_PAIR_EXCHANGE``, default on)."""
    return os.environ.get("DION_B200_PAIR_EXCHANGE", "1") != "0"


def _num_tiles(M: int, N: int, bm: int, bn: int, sym: bool) -> int:
    tm_n, tn_n = -(-M // bm), -(-N // bn)
    if not sym:
        return tm_n * tn_n
    return sum(1 for tm in range(tm_n) for tn in range(tn_n) if (tn + 1) * bn - 1 >= tm * bm)


_config_cache: Dict[Tuple, Tuple[bool, int]] = {}


def _choose_config(M: int, N: int, K: int, batch: int, sym: bool, pair_ok: bool,
                   device: torch.device) -> Tuple[bool, int]:
    """-> (use the two-CTA kernel, BN of the single-CTA kernel).  Picks the tiling with the
    smallest estimated time ``waves x tile size x (K / efficiency + fixed cost)``: large batches
    go to 256 x 256 pair tiles, while a lone matrix whose tiles would leave most SMs idle goes to
    smaller tiles (e.g. the 2048 x 2048 Gram matrix of one 2048 x 8192 input: 36 pair tiles for
    74 pairs, but 136 single-CTA 128 x 128 tiles for 148 SMs).  Efficiencies and the fixed cost
    per tile (pipeline fill + epilogue, expressed in K elements) are fitted to the timings of
    ``benchmark/bench_newton_schulz.py --gemms``."""
    key = (M, N, K, batch, sym, pair_ok, device.index)
    hit = _config_cache.get(key)
    if hit is not None:
        return hit
    sms = sm_count(device)
    cands = []
    # (pair?, bn, execution units, tile size per unit, efficiency, fixed cost in K elements)
    if pair_ok and M > 128 and N > 128:
        cands.append((True, 256, sms // 2, 1.0, 1.0, 768.0))
    if N > 128:
        cands.append((False, 256, sms, 1.0, 0.7 if sym else 0.9, 2048.0 if sym else 1024.0))
    cands.append((False, 128, sms, 0.5, 0.6 if sym else 0.8, 2048.0 if sym else 1024.0))
    best, best_t = None, None
    for is_pair, bn, units, size, eff, fixed in cands:
        tiles = _num_tiles(M, N, 256 if is_pair else _BM, bn, sym) * batch
        t = -(-tiles // units) * size * (K / eff + fixed)
        if best_t is None or t < best_t - 1e-9:
            best, best_t = (is_pair, bn), t
    _config_cache[key] = best
    return best


def ns_gemm(
    A: Tensor,
    B: Tensor,
    out: Optional[Tensor] = None,
    *,
    a_is_km: bool = False,
    b_is_kn: bool = False,
    extra: Optional[GemmExtra] = None,
    out_shape: Optional[Tuple[int, int, int]] = None,
    D: Optional[Tensor] = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    scale: Optional[Tensor] = None,
    alpha_pow: int = 0,
    beta_pow: int = 0,
    sym: bool = False,
    out_t: Optional[Tensor] = None,
    out_f32: Optional[Tensor] = None,
    bn: Optional[int] = None,
    pair: Optional[bool] = None,
    epilogue: str = "axpby",
) -> Tensor:
    """``epilogue``: ``"axpby"`` (``alpha*acc + beta*D``), ``"relu2"`` (``relu(alpha*acc)**2``) or
    ``"mul_2sqrt"`` (``alpha*acc * 2*sqrt(D)``, the backward of ReLU^2 expressed through its
    output); the last two exist in the two-CTA kernel only."""
    A3, B3 = _as3d(A), _as3d(B)
    batch = A3.size(0)
    M, K = (A3.size(-1), A3.size(-2)) if a_is_km else (A3.size(-2), A3.size(-1))
    N = B3.size(-1) if b_is_kn else B3.size(-2)
    assert (B3.size(-2) if b_is_kn else B3.size(-1)) == K and B3.size(0) == batch
    if not supported(A3, B3):
        raise ValueError("ns_gemm operands violate the TMA alignment rules; see supported()")
    dev = A.device
    remote = extra is not None and extra.remote_c[0] != 0
    if out is None and out_f32 is None and not remote:
        out = torch.empty((batch, M, N), dtype=torch.bfloat16, device=dev)
        if A.ndim == 2:
            out = out[0]
    C3 = _as3d(out) if out is not None else None
    Cf3 = _as3d(out_f32) if out_f32 is not None else None
    tgt = Cf3 if Cf3 is not None else C3
    ldc, sc = _ld_stride(tgt) if tgt is not None else (N, M * N)
    D3 = _as3d(D) if D is not None else None
    ldd, sd = _ld_stride(D3) if D3 is not None else (0, 0)
    CT3 = _as3d(out_t) if out_t is not None else None
    ldct, sct = _ld_stride(CT3) if CT3 is not None else (0, 0)
    lda, sa = _ld_stride(A3)
    ldb, sb = _ld_stride(B3)
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.numel() >= batch
    st = status_tensor(dev)
    epi = _EPILOGUES[epilogue]
    if epi != 0:
        pair = True
    if pair is None:
        pair_ok = pair_default() and bn is None and out_t is None and out_f32 is None \
            and (extra is None or pair_exchange())
        if remote and (sym or N % 8 or D3 is None):
            pair_ok = False
        # The two-CTA kernel moves C and D by TMA: 16-byte aligned bases, strides multiples of 8.
        for t3, ld_, bs_ in ((C3, ldc, sc), (D3, ldd, sd)):
            if t3 is not None and (t3.data_ptr() % 16 or ld_ % 8 or bs_ % 8):
                pair_ok = False
        if bn is None:
            pair, bn_pick = _choose_config(M, N, K, batch, sym, pair_ok, dev)
            if not pair:
                bn = bn_pick
        else:
            pair = False
    if pair:
        if out_t is not None or out_f32 is not None:
            raise ValueError("the two-CTA kernel has no transposed/fp32 outputs")
        tiles = tile_table(M, N, 256, sym, dev, bm=256)
        rc = _backend.lib("ns_gemm2_sm100").dion_ns_gemm2_ex(
            _p(A3), ctypes.c_longlong(lda), ctypes.c_longlong(sa),
            ctypes.c_int(1 if a_is_km else 0),
            _p(B3), ctypes.c_longlong(ldb), ctypes.c_longlong(sb),
            ctypes.c_int(1 if b_is_kn else 0),
            _p(C3), ctypes.c_longlong(ldc), ctypes.c_longlong(sc),
            _p(D3), ctypes.c_longlong(ldd), ctypes.c_longlong(sd),
            ctypes.c_int(batch), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_float(alpha), ctypes.c_float(beta), _p(scale),
            ctypes.c_int(alpha_pow), ctypes.c_int(beta_pow), ctypes.c_int(1 if sym else 0),
            _p(tiles), ctypes.c_int(tiles.size(0)), ctypes.c_int(epi), _p(st),
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream),
            ctypes.byref(extra) if extra is not None else None,
        )
        if rc != 0:
            raise RuntimeError(f"dion_ns_gemm2 launch failed with code {rc}")
        return out
    if bn is None:
        bn = 256 if N > 128 else 128
    tiles = tile_table(M, N, bn, sym, dev)
    rc = _backend.lib("ns_gemm_sm100").dion_ns_gemm_ex(
        _p(A3), ctypes.c_longlong(lda), ctypes.c_longlong(sa), ctypes.c_int(1 if a_is_km else 0),
        _p(B3), ctypes.c_longlong(ldb), ctypes.c_longlong(sb), ctypes.c_int(1 if b_is_kn else 0),
        _p(C3), ctypes.c_longlong(ldc), ctypes.c_longlong(sc),
        _p(D3), ctypes.c_longlong(ldd), ctypes.c_longlong(sd),
        _p(CT3), ctypes.c_longlong(ldct), ctypes.c_longlong(sct),
        _p(Cf3),
        ctypes.c_int(batch), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_float(alpha), ctypes.c_float(beta), _p(scale),
        ctypes.c_int(alpha_pow), ctypes.c_int(beta_pow), ctypes.c_int(1 if sym else 0),
        _p(tiles), ctypes.c_int(tiles.size(0)), ctypes.c_int(bn),
        ctypes.c_int(sm_count(dev)), _p(st),
        ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream),
        ctypes.byref(extra) if extra is not None else None,
    )
    if rc != 0:
        raise RuntimeError(f"dion_ns_gemm launch failed with code {rc}")
    return out if out is not None else out_f32


def iterate_in_one_call(X: Tensor, batch: int, m: int, n: int) -> bool:
    """True when all three GEMMs of a Newton-Schulz iteration on ``[batch, m, n]`` would go to the
    two-CTA kernel, so that the whole iteration can be issued by one host call."""
    if not pair_default() or not X.is_contiguous() or X.data_ptr() % 16 or m % 8 or n % 8:
        return False
    dev = X.device
    tall = m > n
    g = n if tall else m
    k_gram = m if tall else n
    return (_choose_config(g, g, k_gram, batch, True, True, dev)[0]
            and _choose_config(g, g, g, batch, True, True, dev)[0]
            and _choose_config(m, n, g, batch, False, True, dev)[0])


def ns_iterate(X: Tensor, Xalt: Tensor, A: Tensor, Bm: Tensor, coeffs, scale: Optional[Tensor]
               ) -> Tensor:
    """All iterations ``(a, b, c) in coeffs`` of ``X <- aX + (bA + cA^2)X`` with ``A = X X^T``
    (right-multiplied forms for tall ``X``) issued by one call into the library; ``scale`` (one
    fp32 per matrix) normalizes the input inside the first iteration.  ``X`` is overwritten;
    returns whichever of ``X`` / ``Xalt`` holds the result."""
    batch, m, n = X.shape
    dev = X.device
    g = min(m, n)
    tiles_gg = tile_table(g, g, 256, True, dev, bm=256)
    tiles_mn = tile_table(m, n, 256, False, dev, bm=256)
    flat = (ctypes.c_float * (3 * len(coeffs)))(*[float(v) for abc in coeffs for v in abc])
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.numel() >= batch
    st = status_tensor(dev)
    rc = _backend.lib("ns_gemm2_sm100").dion_ns_iterate2(
        _p(X), _p(Xalt), _p(A), _p(Bm), ctypes.c_int(batch), ctypes.c_int(m), ctypes.c_int(n),
        flat, ctypes.c_int(len(coeffs)), _p(scale), _p(tiles_gg), ctypes.c_int(tiles_gg.size(0)),
        _p(tiles_mn), ctypes.c_int(tiles_mn.size(0)), _p(st),
        ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"dion_ns_iterate2 failed with code {rc}")
    _backend.add_launches(3 * len(coeffs))
    return Xalt if len(coeffs) % 2 else X


_persist_tiles: Dict[Tuple, Tensor] = {}
_persist_counter: Dict[int, Tensor] = {}


def persistent_enabled() -> bool:
    """``DION_B200_PERSISTENT_NS`` (default on): small batches run the whole Newton-Schulz loop
    in one cooperative launch instead of three launches per iteration."""
    return os.environ.get("DION_B200_PERSISTENT_NS", "1") != "0"


def persistent_waves() -> float:
    """Largest GEMM of the loop, in waves of 128 x 128 tiles over the SMs, up to which the
    one-launch form is used (``DION_B200_PERSISTENT_WAVES``, default 1: beyond that the
    256 x 256 two-CTA kernel's better efficiency outweighs the saved launches)."""
    try:
        return float(os.environ.get("DION_B200_PERSISTENT_WAVES", "1"))
    except ValueError:
        return 1.0


def persistent_in_graphs() -> bool:
    """Whether the cooperative one-launch loop may be recorded into a CUDA graph
    (``DION_B200_PERSISTENT_NS=graph``)."""
    return os.environ.get("DION_B200_PERSISTENT_NS", "1") == "graph"


def persistent_fits(X: Tensor, batch: int, m: int, n: int, iters: int) -> bool:
    """The one-launch form pays when no GEMM of the loop has more 128 x 128 tiles than the GPU
    has SMs (every phase is then a single wave and launch / fill / drain dominate)."""
    if not persistent_enabled() or not X.is_contiguous() or X.data_ptr() % 16 or m % 8 or n % 8:
        return False
    if iters > 8:
        return False
    if torch.cuda.is_current_stream_capturing() and not persistent_in_graphs():
        return False
    g = min(m, n)
    tiles = max(_num_tiles(g, g, _BM, 128, True), _num_tiles(m, n, _BM, 128, False)) * batch
    return tiles <= persistent_waves() * sm_count(X.device)


def ns_persistent(X: Tensor, Xalt: Tensor, A: Tensor, Bm: Tensor, coeffs,
                  scale: Optional[Tensor]) -> Optional[Tensor]:
    """All iterations in one cooperative launch (csrc/ns_persistent_sm100.cu).  Returns the
    buffer that holds the result, or None when the launch could not be made co-resident (the
    caller falls back to per-GEMM launches; nothing has been written then)."""
    batch, m, n = X.shape
    dev = X.device
    g = min(m, n)
    key = (m, n, dev.index)
    tab = _persist_tiles.get(key)
    if tab is None:
        gg = tile_table(g, g, 128, True, dev)
        mn = tile_table(m, n, 128, False, dev)
        tab = _persist_tiles[key] = (torch.cat([gg, mn]).contiguous(), gg.size(0), mn.size(0))
    tiles, n_gg, n_mn = tab
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    counter = _persist_counter.get(idx)
    if counter is None:
        counter = _persist_counter[idx] = torch.zeros(2, dtype=torch.int32, device=dev)
    flat = (ctypes.c_float * (3 * len(coeffs)))(*[float(v) for abc in coeffs for v in abc])
    st = status_tensor(dev)
    rc = _backend.lib("ns_persistent_sm100").dion_ns_persistent(
        _p(X), _p(Xalt), _p(A), _p(Bm), ctypes.c_int(batch), ctypes.c_int(m), ctypes.c_int(n),
        flat, ctypes.c_int(len(coeffs)), _p(scale), _p(tiles), ctypes.c_int(n_gg),
        ctypes.c_int(n_mn), _p(counter), ctypes.c_int(sm_count(dev)), _p(st),
        ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc == -20:
        return None
    if rc != 0:
        raise RuntimeError(f"dion_ns_persistent failed with code {rc}")
    return Xalt if len(coeffs) % 2 else X
