"""Host-side tiling logic of the GEMM front end (no GPU needed)."""
import torch

from dion_b200.ops import gemm


def test_tile_count_matches_tile_table():
    dev = torch.device("cpu")
    for M, N, bm, bn, sym in [(768, 768, 128, 256, True), (768, 768, 128, 128, True),
                              (2048, 2048, 256, 256, True), (328, 456, 256, 256, False),
                              (192, 192, 256, 256, True), (1000, 1000, 128, 128, True)]:
        table = gemm.tile_table(M, N, bn, sym, dev, bm=bm)
        assert table.size(0) == gemm._num_tiles(M, N, bm, bn, sym)
        if sym:
            # every upper-triangle element is covered by a listed tile
            covered = torch.zeros(M, N, dtype=torch.bool)
            for tm, tn in table.tolist():
                covered[tm * bm:(tm + 1) * bm, tn * bn:(tn + 1) * bn] = True
            assert bool(covered[torch.triu(torch.ones(M, N, dtype=torch.bool))].all())


def test_config_choice_fills_the_machine(monkeypatch):
    monkeypatch.setattr(gemm, "sm_count", lambda device: 148)
    gemm._config_cache.clear()
    dev = torch.device("cuda", 0)
    # many matrices: 256 x 256 pair tiles
    assert gemm._choose_config(2048, 2048, 2048, 24, True, True, dev) == (True, 256)
    assert gemm._choose_config(2048, 2048, 2048, 24, False, True, dev) == (True, 256)
    # one 2048 x 2048 Gram matrix: 36 pair tiles would idle half the pairs
    assert gemm._choose_config(2048, 2048, 8192, 1, True, True, dev) == (False, 128)
    # pair kernel not allowed (e.g. fp32 output requested): single-CTA tiles only
    assert gemm._choose_config(2048, 2048, 2048, 24, True, False, dev)[0] is False
    # thin outputs never go to the pair kernel
    assert gemm._choose_config(128, 4096, 512, 8, False, True, dev)[0] is False
    gemm._config_cache.clear()


def test_pointer_tables_layout_and_cache():
    """Host-side construction of the multi-tensor tables: ``[n, chunk prefix, numels, pointers]``,
    cached by the addresses they hold."""
    import torch
    from dion_b200.ops import tables
    tables.clear_cache()
    a, b = torch.zeros(5000), torch.zeros(10)
    g, h = torch.zeros(5000), torch.zeros(10)
    tb = tables.build_table([[a, b], [g, h], [None, tables.RawPointer(4096)]], tag="t")
    flat = tb.device_tensor.tolist()
    assert tb.n == 2 and tb.n_chunks == 3            # ceil(5000 / 4096) + ceil(10 / 4096)
    assert flat[0] == 2 and flat[1:4] == [0, 2, 3] and flat[4:6] == [5000, 10]
    assert flat[6:8] == [a.data_ptr(), b.data_ptr()] and flat[8:10] == [g.data_ptr(), h.data_ptr()]
    assert flat[10:12] == [0, 4096]
    assert tables.build_table([[a, b], [g, h], [None, tables.RawPointer(4096)]], tag="t") is tb
    g2 = torch.zeros(5000)                            # a gradient buffer that moved
    tb2 = tables.build_table([[a, b], [g2, h], [None, tables.RawPointer(4096)]], tag="t")
    assert tb2 is not tb and tb2.device_tensor.tolist()[8] == g2.data_ptr()
    arr = tables.build_ptr_array([[a, b], [g, h]], tag="p")
    assert arr.tolist() == [[a.data_ptr(), b.data_ptr()], [g.data_ptr(), h.data_ptr()]]
    assert tables.build_ptr_array([[a, b], [g, h]], tag="p") is arr


def test_tensor_map_cache_hits_only_on_identical_keys(tmp_path):
    """The host-side cache of encoded tensor maps (csrc/tmap_cache.h, opt-in) checked with a
    counting stand-in for the driver's encoder: off by default, and when on, a map is reused only
    for the same address, extents, strides and box."""
    import os
    import shutil
    import subprocess
    import pytest
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda.h")):
        pytest.skip("needs g++ and the CUDA headers")
    exe = str(tmp_path / "tmap_cache_check")
    subprocess.run([gxx, "-std=c++17", "-O1", "-I" + cuda_inc,
                    "-I" + os.path.join(root, "dion_b200", "csrc"),
                    os.path.join(root, "tests", "native", "tmap_cache_check.cpp"), "-o", exe,
                    "-lpthread"], check=True, timeout=300)
    env = {k: v for k, v in os.environ.items() if k != "DION_B200_TMAP_CACHE"}
    off = subprocess.run([exe], env=env, capture_output=True, text=True, check=True).stdout.split()
    on = subprocess.run([exe], env=dict(env, DION_B200_TMAP_CACHE="1"), capture_output=True,
                        text=True, check=True).stdout.split()
    assert off == ["3", "6", "0", "1", "1"]      # every call encodes
    assert on == ["1", "3", "1", "1", "1"]       # repeats hit, other box / address miss
