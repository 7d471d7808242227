"""Dion2's selection step on the host: accumulate, pick the largest slices by L1 norm, gather them
as the bf16 Newton-Schulz input, decay them in the accumulator (error feedback), scatter back."""
import torch

from dion_b200.ops import select as SEL


def _setup(seed=0, n=3, rows=6, cols=5):
    torch.manual_seed(seed)
    return ([torch.randn(rows, cols) for _ in range(n)], [torch.randn(rows, cols) for _ in range(n)])


def test_rows_with_largest_l1_norm_are_taken_and_decayed():
    G, M = _setup()
    acc = [m + g for m, g in zip(M, G)]                       # what the accumulator must become
    U, idx, maps = SEL.dion2_select(G, M, 2, -2, 0.9)
    assert U.shape == (3, 2, 5) and U.dtype == torch.bfloat16 and idx.shape == (3, 2)
    assert maps is None                                       # only the CUDA path returns maps
    for i in range(3):
        want = set(acc[i].abs().sum(-1).topk(2).indices.tolist())
        got = idx[i].tolist()
        assert set(got) == want
        for j, r in enumerate(got):
            assert torch.equal(U[i, j], acc[i][r].bfloat16())
            assert torch.allclose(M[i][r], acc[i][r] * 0.9)   # selected rows decay ...
        rest = [r for r in range(6) if r not in want]
        assert torch.equal(M[i][rest], acc[i][rest])          # ... the others keep their sum


def test_columns_no_gradient_and_no_decay():
    _, M = _setup(1)
    before = [m.clone() for m in M]
    U, idx, _ = SEL.dion2_select(None, M, 3, -1, 0.5, apply_ef=False)
    assert U.shape == (3, 6, 3)
    for i in range(3):
        assert torch.equal(M[i], before[i])                   # nothing added, nothing decayed
        want = set(before[i].abs().sum(-2).topk(3).indices.tolist())
        assert set(idx[i].tolist()) == want
        for j, c in enumerate(idx[i].tolist()):
            assert torch.equal(U[i, :, j], before[i][:, c].bfloat16())


def test_batched_parameters_and_empty_selection():
    torch.manual_seed(2)
    M = [torch.randn(2, 4, 8), torch.randn(2, 4, 8)]          # two parameters of two matrices each
    U, idx, _ = SEL.dion2_select(None, M, 1, -2, 0.9)
    assert U.shape == (4, 1, 8) and idx.shape == (4, 1)       # N counts 2-D matrices
    U0, idx0, _ = SEL.dion2_select(None, M, 0, -2, 0.9)
    assert U0.shape == (4, 0, 8) and idx0.shape == (4, 0)


def test_scatter_puts_slices_back_at_their_indices():
    torch.manual_seed(3)
    src = torch.randn(2, 3, 5).bfloat16()
    idx = torch.tensor([[4, 0, 2], [1, 5, 3]])
    rows = SEL.scatter_selected(src, idx, 6, -2)
    assert rows.shape == (2, 6, 5)
    for n in range(2):
        for j, r in enumerate(idx[n].tolist()):
            assert torch.equal(rows[n, r], src[n, j])
        untouched = [r for r in range(6) if r not in idx[n].tolist()]
        assert float(rows[n, untouched].abs().sum()) == 0.0
    src_c = torch.randn(2, 5, 3)
    cols = SEL.scatter_selected(src_c, idx, 6, -1)
    assert cols.shape == (2, 5, 6) and torch.equal(cols[0][:, 4], src_c[0][:, 0])
    assert float(cols[1][:, [0, 2, 4]].abs().sum()) == 0.0
