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
