"""Batched Householder QR (R factor) and Cholesky kernels against torch.linalg in fp64."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(3, 128, 96), (5, 256, 192), (2, 640, 512), (2, 1024, 768),
                                   (4, 40, 40), (3, 72, 17)])
def test_qr_r_factor(shape):
    from dion_b200.ops import lowrank as LR
    B, k, r = shape
    torch.manual_seed(0)
    A = torch.randn(B, k, r, device="cuda")
    A[:, :, 1] *= 1e-3          # badly scaled column
    R = LR.qr_r_factor(A)
    torch.cuda.synchronize()
    assert R.shape == (B, r, r)
    assert torch.equal(R, R.triu())
    A64 = A.double()
    gram = A64.mT @ A64
    got = R.double().mT @ R.double()
    assert (got - gram).abs().max().item() < 1e-4 * gram.abs().max().item()
    # Same factor as LAPACK up to the sign of each row.
    ref = torch.linalg.qr(A64, mode="r")[1]
    assert (R.double().abs() - ref.abs()).abs().max().item() < 1e-3 * ref.abs().max().item()
    # P R^-1 has orthonormal columns.
    Q = torch.linalg.solve_triangular(R.double(), A64, upper=True, left=False)
    eye = torch.eye(r, device="cuda", dtype=torch.float64)
    assert (Q.mT @ Q - eye).abs().max().item() < 1e-3


def test_qr_r_factor_zero_column_is_finite():
    from dion_b200.ops import lowrank as LR
    A = torch.randn(2, 128, 64, device="cuda")
    A[0, :, 5] = 0
    A[1] = 0
    R = LR.qr_r_factor(A)
    assert torch.isfinite(R).all()
    assert R[1].abs().max().item() == 0.0


@pytest.mark.parametrize("shape", [(3, 96), (5, 192), (2, 512), (2, 768), (4, 17)])
def test_cholesky_upper(shape):
    from dion_b200.ops import lowrank as LR
    B, r = shape
    torch.manual_seed(1)
    X = torch.randn(B, 2 * r, r, device="cuda")
    G = X.mT @ X
    U = LR.cholesky_upper(G)
    torch.cuda.synchronize()
    assert torch.equal(U, U.triu())
    ref = torch.linalg.cholesky(G.double(), upper=True)
    assert (U.double() - ref).abs().max().item() < 1e-4 * ref.abs().max().item()


def test_cholesky_of_indefinite_matrix_gives_nan_not_hang():
    from dion_b200.ops import lowrank as LR
    G = -torch.eye(64, device="cuda").unsqueeze(0).repeat(2, 1, 1)
    G[1] = torch.eye(64, device="cuda")
    U = LR.cholesky_upper(G)
    assert torch.isnan(U[0]).any()
    assert torch.allclose(U[1], torch.eye(64, device="cuda"))


def test_orthogonalize_batched_matches_fp64():
    from dion_b200.ops import lowrank as LR
    torch.manual_seed(2)
    P = torch.randn(6, 768, 192, device="cuda") @ torch.diag(torch.logspace(0, -3, 192).cuda())
    Q = LR.orthogonalize(P, 1.25)
    eye = torch.eye(192, device="cuda")
    assert (Q.mT @ Q - eye).abs().max().item() < 1e-3
    # Same column space: projecting P onto Q loses nothing.
    assert ((Q @ (Q.mT @ P)) - P).abs().max().item() < 1e-3 * P.abs().max().item()


@pytest.mark.parametrize("shape", [(6, 768, 768, 192), (3, 3072, 768, 192), (2, 2048, 8192, 512)])
def test_power_iteration_gemms_on_tcgen05(shape):
    """P = M Q and R = M^T P for bf16 batches run on the package's GEMM kernels."""
    from dion_b200.ops import _backend, lowrank as LR
    from dion_b200.ops.gemm import check_status
    B, m, n, r = shape
    torch.manual_seed(3)
    M = torch.randn(B, m, n, device="cuda").bfloat16()
    Q = (torch.randn(B, n, r, device="cuda") / n ** 0.5).bfloat16()
    before = _backend.launch_count()
    P = LR.power_iteration_p(M, Q)
    R = LR.power_iteration_r(M, P)
    torch.cuda.synchronize()
    check_status()
    assert _backend.launch_count() == before + 2          # own kernels, not torch.bmm
    Pref = M.float() @ Q.float()
    assert (P.float() - Pref).abs().max().item() < 1e-2 * Pref.abs().max().item()
    Rref = M.float().mT @ P.float()
    assert (R.float() - Rref).abs().max().item() < 1e-2 * Rref.abs().max().item()
    # fp32 batches keep the library path
    assert torch.allclose(LR.power_iteration_p(M.float(), Q.float()), Pref, rtol=1e-3, atol=1e-3)
