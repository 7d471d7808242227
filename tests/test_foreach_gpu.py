"""Multi-tensor kernels against the PyTorch implementations of the same functions."""
import pytest
import torch

from dion_b200.ops import foreach as F

pytestmark = pytest.mark.gpu

SHAPES = [(64, 128), (33, 7), (768, 768), (5,), (1,), (4097,)]


def _mk(dtype, seed, shapes=SHAPES):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*s, generator=g).to(dtype) for s in shapes]


def _pair(ts):
    return [t.clone() for t in ts], [t.clone().cuda() for t in ts]


def _close(cpu, gpu, tol):
    """``tol`` acts absolutely for small values and relatively (bf16 ulps) for large ones."""
    for a, b in zip(cpu, gpu):
        a, b = a.float(), b.float().cpu()
        assert ((a - b).abs() <= tol * (1 + a.abs())).all().item(), (a.shape,)


@pytest.mark.parametrize("m_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nesterov", [False, True])
def test_muon_pre(m_dtype, nesterov):
    Gc, Gg = _pair(_mk(torch.float32, 0))
    Mc, Mg = _pair(_mk(m_dtype, 1))
    ss = torch.zeros(len(Gg), device="cuda")
    Uc = F.muon_pre(Gc, Mc, 0.95, nesterov)
    Ug = F.muon_pre(Gg, Mg, 0.95, nesterov, sumsq=ss)
    tol = 1e-6 if m_dtype == torch.float32 else 4e-2
    _close(Mc, Mg, tol)
    _close(Uc, Ug, 4e-2)
    ref = torch.stack([u.float().square().sum() for u in Ug]).cpu()
    assert torch.allclose(ss.cpu(), ref, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_muon_pre_stores_into_a_column_block(dtype):
    """``out_block``: the bf16 output of each ``[rows, cols]`` tensor lands in columns
    ``[off, off + cols)`` of a wider matrix, the rest of which stays untouched; the dense output
    of a second call gives the expected values."""
    from dion_b200.ops.tables import RawPointer
    torch.manual_seed(4)
    rows, cols, pitch, off = 40, 64, 256, 128
    G = [torch.randn(rows, cols, device="cuda").to(dtype) for _ in range(3)]
    M1 = [torch.randn(rows, cols, device="cuda").to(dtype) for _ in range(3)]
    M2 = [m.clone() for m in M1]
    wide = torch.full((3, rows, pitch), 7.0, device="cuda", dtype=torch.bfloat16)
    outs = [RawPointer(wide[i].data_ptr() + off * 2) for i in range(3)]
    F.muon_pre(G, M1, 0.9, True, out=outs, out_block=(cols, pitch))
    dense = F.muon_pre(G, M2, 0.9, True)
    torch.cuda.synchronize()
    for i in range(3):
        assert torch.equal(wide[i, :, off:off + cols], dense[i])
        assert torch.equal(M1[i], M2[i])
    rest = torch.cat([wide[:, :, :off], wide[:, :, off + cols:]], dim=2)
    assert (rest == 7.0).all().item()


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cautious", [False, True])
def test_muon_post(x_dtype, cautious):
    Xc, Xg = _pair(_mk(x_dtype, 0))
    Uc, Ug = _pair(_mk(torch.bfloat16, 1))
    lr = torch.tensor(0.02)
    F.muon_post(Xc, Uc, lr, 0.01, 1.5, cautious)
    F.muon_post(Xg, Ug, lr.cuda(), 0.01, 1.5, cautious)
    _close(Xc, Xg, 1e-6 if x_dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("cautious", [False, True])
@pytest.mark.parametrize("tensor_wd", [False, True])
def test_adamw_matches_torch_fused(cautious, tensor_wd):
    X = _mk(torch.float32, 0)
    Xg = [x.clone().cuda() for x in X]
    Xr = [x.clone().cuda() for x in X]
    Mg = [torch.zeros_like(x) for x in Xg]
    Vg = [torch.zeros_like(x) for x in Xg]
    Mr = [torch.zeros_like(x) for x in Xg]
    Vr = [torch.zeros_like(x) for x in Xg]
    steps_g = [torch.zeros((), device="cuda") for _ in Xg]
    steps_r = [torch.zeros((), device="cuda") for _ in Xg]
    lr = torch.tensor(3e-3, device="cuda")
    wd = torch.tensor(0.1, device="cuda") if tensor_wd else 0.1
    for it in range(4):
        G = [g.cuda() for g in _mk(torch.float32, 10 + it)]
        F.adamw(Xg, G, Mg, Vg, lr, 0.9, 0.95, wd, 1e-8, state_steps=steps_g, cautious_wd=cautious)
        if not cautious:
            torch._foreach_add_(steps_r, 1)
            torch._fused_adamw_(Xr, G, Mr, Vr, [], steps_r, amsgrad=False, beta1=0.9, beta2=0.95,
                                lr=lr, weight_decay=0.1, eps=1e-8, maximize=False,
                                grad_scale=None, found_inf=None)
    assert all(float(s) == 4.0 for s in steps_g)
    if not cautious:
        for a, b in zip(Xg, Xr):
            assert (a - b).abs().max().item() < 2e-6
    else:
        Xc = [x.clone() for x in X]
        Mc = [torch.zeros_like(x) for x in Xc]
        Vc = [torch.zeros_like(x) for x in Xc]
        sc = [torch.zeros(()) for _ in Xc]
        for it in range(4):
            F.adamw(Xc, _mk(torch.float32, 10 + it), Mc, Vc, torch.tensor(3e-3), 0.9, 0.95, 0.1,
                    1e-8, state_steps=sc, cautious_wd=True)
        _close(Xc, Xg, 2e-6)


def test_adamw_host_step_and_shared_counter():
    Xc, Xg = _pair(_mk(torch.float32, 0))
    Gc, Gg = _pair(_mk(torch.float32, 1))
    Mc, Mg = _pair([torch.zeros_like(x) for x in Xc])
    Vc, Vg = _pair([torch.zeros_like(x) for x in Xc])
    F.adamw(Xc, Gc, Mc, Vc, 1e-2, 0.9, 0.95, 0.0, 1e-8, step=3)
    F.adamw(Xg, Gg, Mg, Vg, 1e-2, 0.9, 0.95, 0.0, 1e-8, step=3)
    _close(Xc, Xg, 2e-6)
    shared = torch.zeros((), device="cuda")
    F.adamw(Xg, Gg, Mg, Vg, torch.tensor(1e-2, device="cuda"), 0.9, 0.95, 0.0, 1e-8,
            state_steps=[shared] * len(Xg))
    assert float(shared) == 1.0


@pytest.mark.parametrize("cautious", [False, True])
def test_lion(cautious):
    Xc, Xg = _pair(_mk(torch.float32, 0))
    Gc, Gg = _pair(_mk(torch.float32, 1))
    Mc, Mg = _pair(_mk(torch.float32, 2))
    F.lion(Xc, Gc, Mc, torch.tensor(1e-3), 0.9, 0.99, 0.1, cautious)
    F.lion(Xg, Gg, Mg, torch.tensor(1e-3).cuda(), 0.9, 0.99, 0.1, cautious)
    _close(Xc, Xg, 1e-6)
    _close(Mc, Mg, 1e-6)


@pytest.mark.parametrize("select_dim", [-2, -1])
def test_dion2_post(select_dim):
    torch.manual_seed(0)
    X = [torch.randn(64, 96) for _ in range(3)]
    Xc, Xg = _pair(X)
    k = 16
    num = 64 if select_dim == -2 else 96
    idx = [torch.randperm(num)[:k] for _ in X]
    ushape = (k, 96) if select_dim == -2 else (64, k)
    U = [torch.randn(*ushape).bfloat16() for _ in X]
    maps = []
    for i in idx:
        m = torch.full((num,), -1, dtype=torch.int32)
        m[i] = torch.arange(k, dtype=torch.int32)
        maps.append(m.cuda())
    F.dion2_post(Xc, U, idx, None, torch.tensor(0.02), 0.01, 1.3, select_dim)
    F.dion2_post(Xg, [u.cuda() for u in U], [i.cuda() for i in idx], maps,
                 torch.tensor(0.02).cuda(), 0.01, 1.3, select_dim)
    _close(Xc, Xg, 1e-6)


@pytest.mark.parametrize("shape", [(3, 40, 72), (5, 37, 2056), (4, 13, 75), (2, 9, 1024)])
def test_normuon_rowstats_and_apply(shape):
    torch.manual_seed(0)
    N, rows, cols = shape   # rows not a multiple of 8: blocks span two matrices
    U = torch.randn(N, rows, cols).bfloat16()
    Vc = [torch.rand(rows, 1) for _ in range(N)]
    Vg = [v.clone().cuda() for v in Vc]
    rc, uc, nc = F.normuon_rowstats(U, Vc, 0.95)
    rg, ug, ng = F.normuon_rowstats(U.cuda(), Vg, 0.95)
    assert torch.allclose(rc, rg.cpu(), rtol=1e-4)
    assert torch.allclose(uc, ug.cpu(), rtol=1e-3) and torch.allclose(nc, ng.cpu(), rtol=1e-3)
    _close(Vc, Vg, 1e-6)
    Xc, Xg = _pair([torch.randn(rows, cols) for _ in range(N)])
    F.muon_post(Xc, list(U.unbind(0)), torch.tensor(0.02), 0.01, 1.2, False,
                rowscale=list(rc.unbind(0)), normU2=uc, normNew2=nc)
    F.muon_post(Xg, list(U.cuda().unbind(0)), torch.tensor(0.02).cuda(), 0.01, 1.2, False,
                rowscale=list(rg.unbind(0)), normU2=ug, normNew2=ng)
    _close(Xc, Xg, 1e-5)


@pytest.mark.parametrize("select_dim", [-2, -1])
@pytest.mark.parametrize("m_dtype", [torch.float32, torch.bfloat16])
def test_dion2_post_masked_matches_torch(select_dim, m_dtype):
    """Global-scope post step: the kernels and the PyTorch form agree; slices of the momentum
    that were not selected are bit-identical."""
    from dion_b200.ops import foreach as F
    torch.manual_seed(0)
    n, rows, cols = 3, 72, 200
    X = [torch.randn(rows, cols) for _ in range(n)]
    M = [torch.randn(rows, cols).to(m_dtype) for _ in range(n)]
    U = []
    for _ in range(n):
        u = torch.zeros(rows, cols)
        num = rows if select_dim == -2 else cols
        pick = torch.randperm(num)[: num // 4]
        if select_dim == -2:
            u[pick] = torch.randn(len(pick), cols)
        else:
            u[:, pick] = torch.randn(rows, len(pick))
        U.append(u.bfloat16())
    Xc, Mc = [x.clone() for x in X], [m.clone() for m in M]
    F.dion2_post_masked(Xc, Mc, U, 0.02, 0.01, 1.7, 0.9, select_dim)          # PyTorch form
    Xg, Mg, Ug = [x.cuda() for x in X], [m.cuda() for m in M], [u.cuda() for u in U]
    lr = torch.tensor(0.02, device="cuda")
    F.dion2_post_masked(Xg, Mg, Ug, lr, 0.01, 1.7, 0.9, select_dim)           # kernels
    torch.cuda.synchronize()
    for t in range(n):
        # the PyTorch form rounds lr*ratio*u to bf16 before the subtraction (as the reference's
        # function does); the kernel keeps the product in fp32
        assert (Xc[t] - Xg[t].cpu()).abs().max().item() < 5e-4
        assert (Mc[t].float() - Mg[t].cpu().float()).abs().max().item() <= (
            1e-6 if m_dtype == torch.float32 else 2e-2)   # one bf16 step at |m| ~ 4
        untouched = (U[t].float().abs().sum(dim=-1 if select_dim == -2 else -2) == 0)
        a, b = M[t], Mg[t].cpu()
        if select_dim == -2:
            assert torch.equal(a[untouched], b[untouched])
        else:
            assert torch.equal(a[:, untouched], b[:, untouched])


def test_aol_rescale_matches_torch():
    torch.manual_seed(6)
    X = torch.randn(3, 136, 264, device="cuda").bfloat16()
    A = (X.float() @ X.float().mT).bfloat16()
    s = torch.rsqrt(A.abs().sum(dim=-1, dtype=torch.float32).clamp_min(1e-7))
    Xr = (X.float() * s.unsqueeze(-1)).bfloat16()
    Ar = (A.float() * s.unsqueeze(-1) * s.unsqueeze(-2)).bfloat16()
    F.aol_rescale_(X, A, 1e-7)
    torch.cuda.synchronize()
    assert (X.float() - Xr.float()).abs().max().item() <= 1e-2 * Xr.float().abs().max().item()
    assert (A.float() - Ar.float()).abs().max().item() <= 1e-2 * Ar.float().abs().max().item()
