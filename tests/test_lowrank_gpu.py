"""Batched Householder QR (R factor) and Cholesky kernels against torch.linalg in fp64."""
import os

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


@pytest.mark.parametrize("shape", [(3, 640, 512), (2, 256, 192), (2, 128, 64), (1, 1280, 1024),
                                   (2, 1408, 96)])
@pytest.mark.parametrize("conditioning", ["random", "graded"])
def test_blocked_qr_r_factor_matches_fp64(shape, conditioning, monkeypatch):
    """Blocked Householder (panel kernel + tensor-core trailing updates): R is upper triangular,
    R^T R reproduces A^T A, and |R| agrees with LAPACK's factor in fp64 - also for columns scaled
    over six orders of magnitude, where a factor of sloppy products would be useless as the
    preconditioner it is computed for."""
    from dion_b200.ops import lowrank as LR
    monkeypatch.setattr(LR, "_QR_BLOCKED_MIN_COLS", 64)    # narrow cases too
    B, k, r = shape
    torch.manual_seed(11)
    A = torch.randn(B, k, r, device="cuda")
    if conditioning == "graded":
        A = A @ torch.diag(torch.logspace(0, -6, r, device="cuda"))
    keep = A.clone()
    R = LR.qr_r_factor(A)
    torch.cuda.synchronize()
    assert torch.equal(A, keep)                    # the caller's matrix is left alone
    assert torch.equal(R, R.triu())
    ref = torch.linalg.qr(A.double(), mode="r")[1]
    scale = ref.abs().amax(dim=(1, 2), keepdim=True)
    # row signs are a convention; compare magnitudes column-scaled so small columns count too
    colmax = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-300)
    err = ((R.double().abs() - ref.abs()) / colmax).abs().max().item()
    assert err < 1e-3, err
    G = A.double().mT @ A.double()
    assert ((R.double().mT @ R.double()) - G).abs().max().item() < 1e-4 * G.abs().max().item()
    # as a preconditioner: A R^-1 has orthonormal columns
    Q = torch.linalg.solve_triangular(R.double(), A.double(), upper=True, left=False)
    eye = torch.eye(r, device="cuda", dtype=torch.float64)
    assert (Q.mT @ Q - eye).abs().max().item() < (5e-3 if conditioning == "graded" else 1e-3)


def test_blocked_qr_equals_column_kernel_up_to_signs():
    from dion_b200.ops import lowrank as LR
    torch.manual_seed(12)
    A = torch.randn(3, 384, 256, device="cuda")
    Rb = LR.qr_r_factor(A)
    os.environ["DION_B200_BLOCKED_QR"] = "0"
    try:
        Rc = LR.qr_r_factor(A)
    finally:
        del os.environ["DION_B200_BLOCKED_QR"]
    assert (Rb.abs() - Rc.abs()).abs().max().item() < 1e-3 * Rc.abs().max().item()


@pytest.mark.parametrize("shape", [(3, 96), (5, 192), (2, 512), (2, 768), (4, 17), (2, 64), (1, 1024)])
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
    # fp32 batches run on the same kernel family as tf32 products
    before = _backend.launch_count()
    P32 = LR.power_iteration_p(M.float(), Q.float())
    assert _backend.launch_count() == before + 1
    assert (P32 - Pref).abs().max().item() < 4e-3 * Pref.abs().max().item()


def _rel(got, ref):
    return ((got.double() - ref).abs().max() / ref.abs().max()).item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("dims", [(3, 256, 256, 128), (2, 200, 136, 104), (1, 128, 520, 64),
                                  (2, 1000, 48, 520)])
def test_lr_gemm_layouts_against_fp64(dtype, a_mn, b_mn, dims):
    """C = alpha A op(B) + beta D for every operand layout, ragged sizes included, fp32 output
    written over D in place, and a bf16 output."""
    from dion_b200.ops import lowrank as LR
    from dion_b200.ops.gemm import check_status
    B, M, N, K = dims
    torch.manual_seed(0)
    A = torch.randn((B, K, M) if a_mn else (B, M, K), device="cuda").to(dtype)
    Bm = torch.randn((B, K, N) if b_mn else (B, N, K), device="cuda").to(dtype)
    D = torch.randn(B, M, N, device="cuda")
    A64 = (A.mT if a_mn else A).double()
    B64 = (Bm if b_mn else Bm.mT).double()
    ref = 0.5 * (A64 @ B64) - 1.5 * D.double()
    out = D.clone()
    LR.lr_gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out=out, D=out, alpha=0.5, beta=-1.5)
    lo = LR.lr_gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    check_status()
    # tf32 keeps 10 mantissa bits of each operand, bf16 operands are exact here
    assert _rel(out, ref) < (4e-3 if dtype == torch.float32 else 1e-5)
    assert lo.dtype == torch.bfloat16 and _rel(lo, A64 @ B64) < 1.5e-2


def test_lr_gemm_split_operands_reach_fp32_accuracy():
    from dion_b200.ops import lowrank as LR
    torch.manual_seed(1)
    A = torch.randn(4, 384, 512, device="cuda")
    Bm = torch.randn(4, 512, 256, device="cuda")
    ref = A.double() @ Bm.double()
    one = LR.lr_gemm(A, Bm, b_mn=True)
    three = LR.lr_gemm(A, Bm, b_mn=True, precise=True)
    torch.cuda.synchronize()
    e1, e3 = _rel(one, ref), _rel(three, ref)
    assert e3 < 2e-5 and e3 < e1 / 20, (e1, e3)
    G = LR.gram(A)          # A^T A, both operands MN-major, split
    assert _rel(G, A.double().mT @ A.double()) < 2e-5


def test_lr_gemm_pointer_tables_column_sums_and_reduction():
    from dion_b200.ops import lowrank as LR
    from dion_b200.ops.gemm import check_status
    torch.manual_seed(2)
    P = torch.randn(5, 320, 64, device="cuda")
    Q = torch.randn(5, 192, 64, device="cuda")
    X = [torch.randn(320, 192, device="cuda") for _ in range(5)]       # separate allocations
    want = [0.9 * x.double() - 0.1 * (p.double() @ q.double().mT) for x, p, q in zip(X, P, Q)]
    LR.foreach_baddbmm_(X, P, Q, alpha=-0.1, beta=0.9)
    torch.cuda.synchronize()
    for x, w in zip(X, want):
        assert _rel(x, w) < 1e-3
    # transpose form: X[i] = X[i] + B A^T
    Xt = [torch.zeros(192, 320, device="cuda") for _ in range(5)]
    LR.foreach_baddbmm_(Xt, P, Q, alpha=1.0, beta=1.0, transpose=True)
    assert _rel(Xt[2], Q[2].double() @ P[2].double().mT) < 4e-3
    # column sums of squares of R = M^T P
    Mx = torch.randn(5, 320, 192, device="cuda")
    colsq = torch.zeros(5, 64, device="cuda")
    R = LR.power_iteration_r(Mx, P, False, colsq=colsq)
    torch.cuda.synchronize()
    assert _rel(R, Mx.double().mT @ P.double()) < 4e-3
    assert _rel(colsq, R.double().square().sum(dim=1)) < 1e-4
    # reduce mode: the result is added at one address per matrix
    acc = torch.ones(5, 320, 192, device="cuda")
    where = torch.tensor([acc[b].data_ptr() for b in (4, 3, 2, 1, 0)], dtype=torch.int64).cuda()
    for _ in range(2):
        LR.lr_gemm(P, Q.contiguous(), reduce_into=where, reduce_ld=192)
    # broadcast mode: matrix b is stored into slot 1 + b of every target
    t0 = torch.zeros(7, 320, 192, device="cuda")
    t1 = torch.zeros(7, 320, 192, device="cuda")
    LR.lr_gemm(P, Q.contiguous(), broadcast_to=[t0.data_ptr(), t1.data_ptr()], slot0=1)
    torch.cuda.synchronize()
    check_status()
    prod = P.double() @ Q.double().mT
    assert _rel(acc, 2 * prod.flip(0) + 1) < 4e-3
    for t in (t0, t1):
        assert _rel(t[1:6], prod) < 4e-3 and float(t[0].abs().max()) == 0 and \
            float(t[6].abs().max()) == 0


@pytest.mark.parametrize("shape", [(3, 17), (4, 96), (2, 200), (6, 512), (2, 768), (1, 1024)])
def test_triu_inverse(shape):
    from dion_b200.ops import lowrank as LR
    B, r = shape
    torch.manual_seed(3)
    A = torch.randn(B, 2 * r, r, device="cuda", dtype=torch.float64)
    U = torch.linalg.qr(A, mode="r")[1]
    X = LR.triu_inverse(U.float())
    torch.cuda.synchronize()
    assert torch.equal(X, X.triu())
    eye = torch.eye(r, device="cuda", dtype=torch.float64)
    assert ((X.double() @ U) - eye).abs().max().item() < 2e-4
    ref = torch.linalg.inv(U)
    assert _rel(X, ref) < 1e-4


def test_orthogonalize_at_model_sizes_issues_no_library_solver():
    """rank 512 factors of 2048-row matrices: orthonormal to fp32-level accuracy, same column
    space, and every product / solve of the tall matrix is one of this package's kernels."""
    from dion_b200.ops import _backend, lowrank as LR
    from dion_b200.ops.gemm import check_status
    torch.manual_seed(4)
    P = torch.randn(4, 2048, 512, device="cuda") @ torch.diag(torch.logspace(0, -3, 512).cuda())
    before = _backend.launch_count()
    Q = LR.orthogonalize(P, 1.25)
    torch.cuda.synchronize()
    check_status()
    # sketch product, QR, 2 x (inverse + 2 splits + product), Gram (+1 split), Cholesky
    assert _backend.launch_count() - before >= 12
    eye = torch.eye(512, device="cuda", dtype=torch.float64)
    assert (Q.double().mT @ Q.double() - eye).abs().max().item() < 1e-3
    assert ((Q @ (Q.mT @ P)) - P).abs().max().item() < 1e-3 * P.abs().max().item()


def test_sketch_is_a_function_of_the_seed_and_gaussian():
    from dion_b200.ops import lowrank as LR
    dev = torch.device("cuda")
    g1 = torch.Generator(device=dev).manual_seed(42)
    g2 = torch.Generator(device=dev).manual_seed(42)
    g3 = torch.Generator(device=dev).manual_seed(43)
    a = LR.random_sketch(3, 256, 1000, torch.float32, dev, g1)
    b = LR.random_sketch(3, 256, 1000, torch.float32, dev, g2)
    c = LR.random_sketch(3, 256, 1000, torch.float32, dev, g3)
    assert torch.equal(a, b) and not torch.equal(a, c)
    x = a.flatten().double() * 16.0            # std 1/sqrt(256)
    assert abs(x.mean().item()) < 5e-3 and abs(x.std().item() - 1) < 5e-3
    assert abs((x ** 3).mean().item()) < 2e-2 and abs((x ** 4).mean().item() - 3) < 5e-2
    assert torch.isfinite(a).all()
    h = LR.random_sketch(2, 128, 77, torch.bfloat16, dev, g1)
    assert h.dtype == torch.bfloat16 and abs(h.float().std().item() * 128 ** 0.5 - 1) < 2e-2
