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
