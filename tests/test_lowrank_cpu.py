"""Low-rank building blocks of Dion on the host (the PyTorch paths that double as the oracle of
the CUDA kernels): rcQR orthonormalization, its factors, guards and update helpers."""
import torch

from dion_b200.ops import lowrank as LR


def test_sketch_size_and_reproducible_sketch():
    assert LR.sketch_rows(192, 1.25) == 256 and LR.sketch_rows(128, 1.0) == 128
    assert LR.sketch_rows(1, 1.25) == 128
    g1, g2 = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
    a = LR.random_sketch(2, 128, 40, torch.float32, torch.device("cpu"), g1)
    b = LR.random_sketch(2, 128, 40, torch.float32, torch.device("cpu"), g2)
    assert torch.equal(a, b) and a.shape == (2, 128, 40)
    assert abs(float(a.var()) - 1.0 / 128) < 0.3 / 128        # entries ~ N(0, 1/k)


def test_r_factor_and_cholesky_reproduce_the_gram_matrix():
    torch.manual_seed(0)
    A = torch.randn(3, 40, 12)
    R = LR.qr_r_factor(A)
    assert R.shape == (3, 12, 12) and torch.equal(R, R.triu())
    assert torch.allclose(R.mT @ R, A.mT @ A, rtol=1e-4, atol=1e-4)
    G = A.mT @ A
    U = LR.cholesky_upper(G)
    assert torch.equal(U, U.triu()) and torch.allclose(U.mT @ U, G, rtol=1e-4, atol=1e-4)
    bad = -torch.eye(4).expand(2, 4, 4).contiguous()          # not positive definite
    out = LR.cholesky_upper(bad)                              # no exception: NaNs or garbage
    assert out.shape == bad.shape
    X = torch.randn(3, 7, 12)
    assert torch.allclose(LR.right_solve_upper(R, X) @ R, X, rtol=1e-3, atol=1e-3)


def test_orthogonalize_gives_an_orthonormal_basis_of_the_same_column_space():
    torch.manual_seed(1)
    for shape in ((2, 64, 8), (1, 300, 32), (3, 16, 16)):    # tall and square (r never exceeds m)
        P = torch.randn(*shape, dtype=torch.float64).float()
        Q = LR.orthogonalize(P, 1.25, generator=torch.Generator().manual_seed(0))
        assert Q.shape == P.shape and Q.dtype == P.dtype
        k = min(shape[-2], shape[-1])
        gram = (Q.mT @ Q)[..., :k, :k] if shape[-2] >= shape[-1] else (Q @ Q.mT)
        eye = torch.eye(gram.size(-1)).expand_as(gram)
        assert (gram - eye).abs().max().item() < 5e-3, shape
        if shape[-2] >= shape[-1]:      # projector onto span(Q) leaves P unchanged
            assert (Q @ (Q.mT @ P) - P).abs().max().item() < 5e-3 * P.abs().max().item() * 10
    bf = torch.randn(2, 64, 8).bfloat16()
    assert LR.orthogonalize(bf).dtype == torch.bfloat16


def test_guard_replaces_dead_matrices_and_nans():
    torch.manual_seed(2)
    B = torch.randn(3, 6, 5)
    B[1].zero_()                                              # momentum entirely zero
    P, R, Q0 = torch.randn(3, 6, 2), torch.randn(3, 5, 2), torch.randn(3, 5, 2)
    P[2, 0, 0] = float("nan")
    R[0, 1, 1] = float("nan")
    P2, R2 = LR.fix_all_zero_or_nan(P.clone(), R.clone(), Q0, B)
    assert torch.equal(P2[1], torch.zeros(6, 2)) and torch.equal(R2[1], Q0[1])
    assert torch.isfinite(P2).all() and torch.isfinite(R2).all()
    assert P2[2, 0, 0] == 0 and R2[0, 1, 1] == 0
    assert torch.equal(P2[0], P[0]) and torch.equal(R2[2], R[2])          # the rest untouched


def test_column_normalize_and_rank_r_updates():
    torch.manual_seed(3)
    X = torch.randn(2, 10, 4)
    Q = LR.column_normalize(X, epsilon=1e-8)
    assert torch.allclose(Q.float().square().sum(-2), torch.ones(2, 4), atol=1e-5)
    # a row-sharded matrix passes the all-reduced sums of squares of the whole columns
    top, bottom = X[:, :6], X[:, 6:]
    ss = LR.local_column_sum_sq(top) + LR.local_column_sum_sq(bottom)
    assert ss.shape == (2, 1, 4)
    assert torch.allclose(LR.column_normalize(top, full_column_sum_sq=ss), Q[:, :6], atol=1e-6)
    zero = LR.column_normalize(torch.zeros(1, 5, 3))
    assert torch.isfinite(zero).all() and float(zero.abs().sum()) == 0.0

    Ms = [torch.randn(6, 5) for _ in range(2)]
    want = [0.9 * m - 0.3 * (a @ b.T) for m, a, b in zip(Ms, torch.randn(2, 6, 2), torch.randn(2, 5, 2))]
    torch.manual_seed(3)
    X = torch.randn(2, 10, 4)                                 # replay the generator to the same point
    Ms2 = [torch.randn(6, 5) for _ in range(2)]
    A, B = torch.randn(2, 6, 2), torch.randn(2, 5, 2)
    LR.foreach_baddbmm_(Ms2, A, B, alpha=-0.3, beta=0.9)
    for got, ref in zip(Ms2, want):
        assert torch.allclose(got, ref, atol=1e-6)
    Mt = [torch.randn(5, 6) for _ in range(2)]
    ref_t = [m - 0.5 * (b @ a.T) for m, a, b in zip(Mt, A, B)]
    LR.foreach_baddbmm_(Mt, A, B, alpha=-0.5, transpose=True)
    for got, ref in zip(Mt, ref_t):
        assert torch.allclose(got, ref, atol=1e-6)


def test_power_iteration_products_and_stacking():
    torch.manual_seed(4)
    M = [torch.randn(6, 9) for _ in range(3)]
    Qs = [torch.randn(9, 2) for _ in range(3)]
    Mb, Qb = LR.stack_for_power_iteration(M, Qs, transposed=False)
    P = LR.power_iteration_p(Mb, Qb)
    R = LR.power_iteration_r(Mb, P)
    for i in range(3):
        assert torch.allclose(P[i], M[i] @ Qs[i], atol=1e-5)
        assert torch.allclose(R[i], M[i].T @ P[i], atol=1e-5)
    Mt, Qt = LR.stack_for_power_iteration(M, [torch.randn(6, 2) for _ in range(3)], transposed=True)
    assert Mt.shape == (3, 9, 6) and Mt.is_contiguous() and torch.equal(Mt[1], M[1].T)
    mixed, q = LR.stack_for_power_iteration([m.bfloat16() for m in M], Qs, transposed=False)
    assert q.dtype == torch.bfloat16                         # Q follows the momentum dtype
