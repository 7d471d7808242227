"""tcgen05 GEMM kernel against an fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(got, ref):
    return (got.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(1, 128, 128, 64), (3, 192, 328, 200), (6, 768, 768, 768),
                                   (2, 72, 40, 24)])
def test_nt(bn, shape):
    from dion_b200.ops import gemm
    b, M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(b, M, K, device="cuda").bfloat16()
    B = torch.randn(b, N, K, device="cuda").bfloat16()
    C = gemm.ns_gemm(A, B, bn=bn)
    torch.cuda.synchronize()
    gemm.check_status()
    assert _rel_err(C, A.float() @ B.float().mT) < 1e-2


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(1, 128, 256, 64), (2, 768, 3072, 768), (3, 192, 328, 200)])
def test_nn_with_epilogue(bn, shape):
    from dion_b200.ops import gemm
    b, M, N, K = shape
    torch.manual_seed(1)
    A = torch.randn(b, M, K, device="cuda").bfloat16()
    B = torch.randn(b, K, N, device="cuda").bfloat16()
    D = torch.randn(b, M, N, device="cuda").bfloat16()
    sc = torch.rand(b, device="cuda") + 0.5
    C = gemm.ns_gemm(A, B, b_is_kn=True, D=D, alpha=0.5, beta=2.0, scale=sc, alpha_pow=1,
                     beta_pow=1, bn=bn)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = (0.5 * (A.float() @ B.float()) + 2.0 * D.float()) * sc[:, None, None]
    assert _rel_err(C, ref) < 1e-2


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(2, 768, 3072), (3, 200, 136), (1, 1024, 512)])
def test_symmetric(bn, shape):
    from dion_b200.ops import gemm
    b, M, K = shape
    torch.manual_seed(2)
    X = torch.randn(b, M, K, device="cuda").bfloat16()
    C = torch.full((b, M, M), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.ns_gemm(X, X, out=C, sym=True, bn=bn)
    torch.cuda.synchronize()
    gemm.check_status()
    assert _rel_err(C, X.float() @ X.float().mT) < 1e-2
    assert (C - C.mT).abs().max().item() == 0.0  # mirrored stores make it exactly symmetric


def test_fp32_and_transposed_outputs():
    from dion_b200.ops import gemm
    torch.manual_seed(3)
    A = torch.randn(2, 256, 128, device="cuda").bfloat16()
    B = torch.randn(2, 192, 128, device="cuda").bfloat16()
    Cf = torch.empty(2, 256, 192, device="cuda", dtype=torch.float32)
    gemm.ns_gemm(A, B, out_f32=Cf)
    CT = torch.empty(2, 192, 256, device="cuda", dtype=torch.bfloat16)
    C = gemm.ns_gemm(A, B, out_t=CT)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = A.float() @ B.float().mT
    assert _rel_err(Cf, ref) < 1e-4
    assert torch.equal(CT, C.mT.contiguous())


def test_rejects_unaligned():
    from dion_b200.ops import gemm
    A = torch.randn(1, 64, 20, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        gemm.ns_gemm(A, A)


# ---- two-CTA (cta_group::2) kernel -----------------------------------------------------------

@pytest.mark.parametrize("shape", [(1, 256, 256, 64), (3, 328, 456, 200), (4, 768, 768, 768),
                                   (2, 512, 1024, 2048), (5, 192, 192, 768), (2, 136, 200, 72)])
def test_pair_nt(shape):
    from dion_b200.ops import gemm
    b, M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(b, M, K, device="cuda").bfloat16()
    B = torch.randn(b, N, K, device="cuda").bfloat16()
    C = gemm.ns_gemm(A, B, pair=True)
    torch.cuda.synchronize()
    gemm.check_status()
    assert _rel_err(C, A.float() @ B.float().mT) < 1e-2


@pytest.mark.parametrize("shape", [(1, 256, 256, 64), (2, 768, 3072, 768), (3, 328, 456, 200),
                                   (3, 192, 768, 192)])
def test_pair_nn_with_epilogue(shape):
    from dion_b200.ops import gemm
    b, M, N, K = shape
    torch.manual_seed(1)
    A = torch.randn(b, M, K, device="cuda").bfloat16()
    B = torch.randn(b, K, N, device="cuda").bfloat16()
    D = torch.randn(b, M, N, device="cuda").bfloat16()
    sc = torch.rand(b, device="cuda") + 0.5
    C = gemm.ns_gemm(A, B, b_is_kn=True, D=D, alpha=0.5, beta=2.0, scale=sc, alpha_pow=1,
                     beta_pow=1, pair=True)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = (0.5 * (A.float() @ B.float()) + 2.0 * D.float()) * sc[:, None, None]
    assert _rel_err(C, ref) < 1e-2


@pytest.mark.parametrize("shape", [(2, 768, 3072), (3, 328, 136), (1, 1024, 512), (4, 192, 768)])
def test_pair_symmetric(shape):
    from dion_b200.ops import gemm
    b, M, K = shape
    torch.manual_seed(2)
    X = torch.randn(b, M, K, device="cuda").bfloat16()
    C = torch.full((b, M, M), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm.ns_gemm(X, X, out=C, sym=True, pair=True)
    torch.cuda.synchronize()
    gemm.check_status()
    assert _rel_err(C, X.float() @ X.float().mT) < 1e-2
    assert (C - C.mT).abs().max().item() == 0.0


def test_pair_km_a_operand():
    """A given as [K, M] (tall Gram matrix X^T X without a transposed copy)."""
    from dion_b200.ops import gemm
    torch.manual_seed(4)
    X = torch.randn(2, 1024, 384, device="cuda").bfloat16()
    C = gemm.ns_gemm(X, X, a_is_km=True, b_is_kn=True, sym=True, pair=True)
    torch.cuda.synchronize()
    gemm.check_status()
    assert _rel_err(C, X.float().mT @ X.float()) < 1e-2


def test_pair_relu2_epilogues():
    """relu(A B^T)^2 and its backward form (dY W) * 2 sqrt(act) fused into the GEMM epilogue."""
    from dion_b200.ops import gemm
    torch.manual_seed(5)
    T, C, F = 1000, 256, 1024
    h = (torch.randn(T, C, device="cuda") * 0.3).bfloat16()
    Wfc = (torch.randn(F, C, device="cuda") * 0.1).bfloat16()
    act = gemm.ns_gemm(h, Wfc, epilogue="relu2")
    ref = torch.relu(h.float() @ Wfc.float().T).square()
    assert _rel_err(act, ref) < 1e-2
    dy = torch.randn(T, C, device="cuda").bfloat16()
    Wpr = (torch.randn(C, F, device="cuda") * 0.1).bfloat16()
    dz = gemm.ns_gemm(dy, Wpr, b_is_kn=True, D=act, epilogue="mul_2sqrt")
    torch.cuda.synchronize()
    gemm.check_status()
    ref_dz = (dy.float() @ Wpr.float()) * 2.0 * act.float().sqrt()
    assert _rel_err(dz, ref_dz) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("sym", [False, True])
def test_output_canaries_and_run_to_run_determinism(pair, sym):
    """The kernels write exactly the M x N window of a padded output (rows and columns beyond
    it keep their sentinel) and give bit-identical results on repeated runs."""
    from dion_b200.ops import gemm
    torch.manual_seed(6)
    b, M, K = 3, 328, 200
    N = M if sym else 456
    A = torch.randn(b, M, K, device="cuda").bfloat16()
    B = A if sym else torch.randn(b, N, K, device="cuda").bfloat16()
    big = torch.full((b, M + 8, N + 8), 12345.0, device="cuda", dtype=torch.bfloat16)
    out = big[:, :M, :N]
    gemm.ns_gemm(A, B, out=out, sym=sym, pair=pair)
    first = out.clone()
    gemm.ns_gemm(A, B, out=out, sym=sym, pair=pair)
    torch.cuda.synchronize()
    gemm.check_status()
    assert torch.equal(first, out)
    assert torch.all(big[:, M:, :] == 12345.0) and torch.all(big[:, :, N:] == 12345.0)
    assert _rel_err(out, A.float() @ B.float().mT) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
def test_batch_offsets_beyond_32_bits(pair):
    """Operands and output of more than 2^31 elements: the last matrix of the batch starts past
    the range of 32-bit element offsets (the reference guards the same case with int64 batch
    offsets, dion/newton_schulz_triton.py:48-50)."""
    from dion_b200.ops import gemm
    b, m, n = 260, 1024, 8192
    assert (b - 1) * m * n > 2 ** 31
    torch.manual_seed(11)
    X = torch.randn(b, m, n, device="cuda", dtype=torch.bfloat16)
    Bm = (torch.randn(b, m, m, device="cuda", dtype=torch.bfloat16) / m ** 0.5)
    out = torch.empty_like(X)
    gemm.ns_gemm(Bm, X, out=out, b_is_kn=True, D=X, alpha=1.0, beta=0.5, pair=pair)
    A = gemm.ns_gemm(X, X, sym=True, pair=pair)
    torch.cuda.synchronize()
    gemm.check_status()
    for i in (0, b - 1):
        ref = Bm[i].float() @ X[i].float() + 0.5 * X[i].float()
        assert _rel_err(out[i], ref) < 1e-2
        assert _rel_err(A[i], X[i].float() @ X[i].float().T) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("tall", [False, True])
def test_exchange_coupling_on_one_gpu(pair, tall):
    """The cross-GPU coupling of the GEMM kernels with this GPU standing in for every peer: the
    first Gram waits on (already raised) arrival flags and builds its scale from per-source
    partial sums; the update GEMM stores each output row into the buffer of its owner."""
    from dion_b200.ops import gemm
    torch.manual_seed(0)
    dev = torch.device("cuda")
    W, batch = 4, 3
    m, n = (1024, 512) if tall else (512, 1024)
    X = torch.randn(batch, m, n, device=dev).bfloat16()
    flags = torch.full((W,), 7, dtype=torch.int32, device=dev)
    seq = torch.full((), 7, dtype=torch.int32, device=dev)
    # per-source partial sums of squares (row blocks of m / W rows each)
    parts = X.float().reshape(batch, W, m // W, n).square().sum(dim=(2, 3)).contiguous()
    g = n if tall else m
    ex = gemm.GemmExtra()
    ex.wait_flags, ex.seq_ptr = flags.data_ptr(), seq.data_ptr()
    ex.n_src, ex.rows_per_src = W, m // W
    ex.wait_a = ex.wait_b = 0 if tall else 1
    ex.wait_k = 1 if tall else 0
    ex.scale_partials = parts.data_ptr()
    ex.scale_mult, ex.scale_eps = 1.0, 1e-7
    A = torch.empty(batch, g, g, device=dev, dtype=torch.bfloat16)
    gemm.ns_gemm(X, X, out=A, sym=True, a_is_km=tall, b_is_kn=tall, alpha_pow=2, extra=ex,
                 pair=pair)
    scale = 1.0 / (X.float().flatten(1).norm(dim=1) + 1e-7)
    Xs = X.float() * scale.view(-1, 1, 1)
    ref = (Xs.mT @ Xs) if tall else (Xs @ Xs.mT)
    torch.cuda.synchronize()
    gemm.check_status()
    assert (A.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    # update GEMM with rows scattered to W owners: owner d gets rows [d*m/W, (d+1)*m/W)
    Bm = torch.randn(batch, g, g, device=dev).bfloat16()
    slots = 5
    bufs = [torch.zeros(slots, m // W, n, device=dev, dtype=torch.bfloat16) for _ in range(W)]
    ex2 = gemm.GemmExtra()
    for d in range(W):
        ex2.remote_c[d] = bufs[d].data_ptr()
    ex2.rows_per_dst, ex2.remote_slot = m // W, 1
    if tall:
        gemm.ns_gemm(X, Bm, out=None, D=X, alpha=1.0, beta=0.5, extra=ex2, pair=pair)
        want = 0.5 * X.float() + X.float() @ Bm.float().mT
    else:
        gemm.ns_gemm(Bm, X, out=None, b_is_kn=True, D=X, alpha=1.0, beta=0.5, extra=ex2, pair=pair)
        want = 0.5 * X.float() + Bm.float() @ X.float()
    torch.cuda.synchronize()
    gemm.check_status()
    got = torch.cat([b_[1:1 + batch] for b_ in bufs], dim=1)        # [batch, m, n]
    assert (got.float() - want).abs().max().item() < 2e-2 * want.abs().max().item()
    for b_ in bufs:
        assert float(b_[0].abs().max()) == 0 and float(b_[4].abs().max()) == 0


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("tall", [False, True])
def test_exchange_coupling_by_columns_on_one_gpu(pair, tall):
    """Column-split form of the coupling: with the sharded dimension being the columns, the first
    Gram gates on K-slabs where the row form gates on tile rows (and the other way round), and the
    update GEMM sends each 16-byte piece of an output row to the owner of its columns, who holds
    ``[slots, m, n / W]``."""
    from dion_b200.ops import gemm
    torch.manual_seed(1)
    dev = torch.device("cuda")
    W, batch = 4, 3
    m, n = (1024, 512) if tall else (512, 1024)
    pc = n // W
    X = torch.randn(batch, m, n, device=dev).bfloat16()
    flags = torch.full((W,), 3, dtype=torch.int32, device=dev)
    seq = torch.full((), 3, dtype=torch.int32, device=dev)
    parts = X.float().reshape(batch, m, W, pc).square().sum(dim=(1, 3)).contiguous()
    g = n if tall else m
    ex = gemm.GemmExtra()
    ex.wait_flags, ex.seq_ptr = flags.data_ptr(), seq.data_ptr()
    ex.n_src, ex.rows_per_src = W, pc
    contracted = not tall          # wide: X X^T contracts over the (sharded) columns
    ex.wait_a = ex.wait_b = 0 if contracted else 1
    ex.wait_k = 1 if contracted else 0
    ex.scale_partials = parts.data_ptr()
    ex.scale_mult, ex.scale_eps = 1.0, 1e-7
    A = torch.empty(batch, g, g, device=dev, dtype=torch.bfloat16)
    gemm.ns_gemm(X, X, out=A, sym=True, a_is_km=tall, b_is_kn=tall, alpha_pow=2, extra=ex,
                 pair=pair)
    scale = 1.0 / (X.float().flatten(1).norm(dim=1) + 1e-7)
    Xs = X.float() * scale.view(-1, 1, 1)
    ref = (Xs.mT @ Xs) if tall else (Xs @ Xs.mT)
    torch.cuda.synchronize()
    gemm.check_status()
    assert (A.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    Bm = torch.randn(batch, g, g, device=dev).bfloat16()
    slots = 5
    bufs = [torch.zeros(slots, m, pc, device=dev, dtype=torch.bfloat16) for _ in range(W)]
    ex2 = gemm.GemmExtra()
    for d in range(W):
        ex2.remote_c[d] = bufs[d].data_ptr()
    ex2.rows_per_dst, ex2.cols_per_dst, ex2.remote_slot = m, pc, 1
    if tall:
        gemm.ns_gemm(X, Bm, out=None, D=X, alpha=1.0, beta=0.5, extra=ex2, pair=pair)
        want = 0.5 * X.float() + X.float() @ Bm.float().mT
    else:
        gemm.ns_gemm(Bm, X, out=None, b_is_kn=True, D=X, alpha=1.0, beta=0.5, extra=ex2, pair=pair)
        want = 0.5 * X.float() + Bm.float() @ X.float()
    torch.cuda.synchronize()
    gemm.check_status()
    got = torch.cat([b_[1:1 + batch] for b_ in bufs], dim=2)        # [batch, m, n]
    assert (got.float() - want).abs().max().item() < 2e-2 * want.abs().max().item()
    for b_ in bufs:
        assert float(b_[0].abs().max()) == 0 and float(b_[4].abs().max()) == 0
