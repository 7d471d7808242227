"""Fused model kernels (forward and backward) against PyTorch autograd in fp32."""
import pytest
import torch
import torch.nn.functional as tF

from dion_b200.models import functional as Fn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm(dtype):
    torch.manual_seed(0)
    x = torch.randn(4, 37, 768, device="cuda").to(dtype).requires_grad_()
    xr = x.detach().float().requires_grad_()
    y = Fn.rms_norm(x)
    yr = tF.rms_norm(xr, (768,), eps=torch.finfo(dtype).eps)
    g = torch.randn_like(yr)
    y.backward(g.to(y.dtype))
    yr.backward(g)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (y.float() - yr).abs().max().item() < tol
    assert (x.grad.float() - xr.grad).abs().max().item() < tol


def test_rms_norm_autocast_emits_bf16():
    x = torch.randn(8, 768, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = Fn.rms_norm(x)
    assert y.dtype == torch.bfloat16
    y.float().sum().backward()
    assert x.grad.dtype == torch.float32


@pytest.mark.parametrize("D", [64, 128])
def test_rope_qknorm(D):
    torch.manual_seed(0)
    B, T, H = 2, 50, 6
    q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(T, device="cuda").float(), inv)
    cos, sin = fr.cos().bfloat16(), fr.sin().bfloat16()
    qo, ko = Fn.rope_qknorm(q, k, cos, sin)
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()

    def ref(x):
        d = D // 2
        c, s = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
        y = torch.cat([x[..., :d] * c + x[..., d:] * s, x[..., d:] * c - x[..., :d] * s], 3)
        return tF.rms_norm(y, (D,), eps=torch.finfo(torch.bfloat16).eps)

    qro, kro = ref(qr), ref(kr)
    gq, gk = torch.randn_like(qro), torch.randn_like(kro)
    (qo.float() * gq + ko.float() * gk).sum().backward()
    (qro * gq + kro * gk).sum().backward()
    assert (qo.float() - qro).abs().max().item() < 3e-2
    assert (ko.float() - kro).abs().max().item() < 3e-2
    assert (q.grad.float() - qr.grad).abs().max().item() < 5e-2
    assert (k.grad.float() - kr.grad).abs().max().item() < 5e-2


def test_qkv_rope_matches_unfused():
    """Fused projection + RoPE + QK-norm against the three separate linears in fp32."""
    torch.manual_seed(0)
    B, T, H, D = 2, 48, 4, 64
    C = H * D
    h = (torch.randn(B, T, C, device="cuda") * 0.5).bfloat16().requires_grad_()
    ws = [(torch.randn(C, C, device="cuda") * C ** -0.5).requires_grad_() for _ in range(3)]
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(T, device="cuda").float(), inv)
    cos, sin = fr.cos().bfloat16(), fr.sin().bfloat16()
    q, k, v = Fn.qkv_rope(h, ws[0], ws[1], ws[2], cos, sin, H)
    assert q.shape == k.shape == v.shape == (B, T, H, D)
    gq, gk, gv = (torch.randn(B, T, H, D, device="cuda") for _ in range(3))
    (q.float() * gq + k.float() * gk + v.float() * gv).sum().backward()

    hr = h.detach().float().requires_grad_()
    wr = [w.detach().bfloat16().float().requires_grad_() for w in ws]

    def rope_norm(x):
        d = D // 2
        c, s = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
        y = torch.cat([x[..., :d] * c + x[..., d:] * s, x[..., d:] * c - x[..., :d] * s], 3)
        return tF.rms_norm(y, (D,), eps=torch.finfo(torch.bfloat16).eps)

    qr = rope_norm((hr @ wr[0].T).view(B, T, H, D))
    kr = rope_norm((hr @ wr[1].T).view(B, T, H, D))
    vr = (hr @ wr[2].T).view(B, T, H, D)
    (qr * gq + kr * gk + vr * gv).sum().backward()
    for got, ref in ((q, qr), (k, kr), (v, vr)):
        assert (got.float() - ref).abs().max().item() < 5e-2
    assert (h.grad.float() - hr.grad).abs().max().item() < 0.05 * hr.grad.abs().max().item() + 5e-2
    for w, r in zip(ws, wr):
        assert w.grad.dtype == torch.float32
        assert (w.grad - r.grad).abs().max().item() < 0.03 * r.grad.abs().max().item() + 5e-2


def test_embedding_backward_matches_torch():
    torch.manual_seed(0)
    V, C = 1000, 64
    w = torch.randn(V, C, device="cuda", requires_grad=True)
    wr = w.detach().clone().requires_grad_()
    idx = torch.randint(0, 50, (4, 200), device="cuda")  # many repeated ids
    idx[0, 0] = V - 1
    g = torch.randn(4, 200, C, device="cuda")
    Fn.embedding(idx, w).backward(g)
    tF.embedding(idx, wr).backward(g)
    assert torch.allclose(w.grad, wr.grad, atol=1e-4, rtol=1e-5)
    assert w.grad[60:V - 1].abs().max().item() == 0.0


def test_embedding_backward_long_runs_and_absent_rows():
    """Ids that occur hundreds of times (split over the block's warps), ids that occur once,
    rows that never occur (written as zeros, not left as allocated), a row count that is no
    multiple of the warps per block, and bit-identical results from call to call."""
    torch.manual_seed(3)
    V, C, T = 1003, 768, 4096
    w = torch.randn(V, C, device="cuda", requires_grad=True)
    idx = torch.randint(0, V, (T,), device="cuda")
    idx[:900] = 7            # one long run
    idx[900:1500] = V - 1    # another, in the last (partial) group of rows
    idx[1500:1565] = 500     # just above the threshold
    idx[1565:1629] = 501     # exactly at it
    idx = idx[torch.randperm(T, device="cuda")].reshape(4, T // 4)
    g = torch.randn(4, T // 4, C, device="cuda")
    junk = torch.full((V, C), float("nan"), device="cuda")   # what an uninitialised buffer may hold
    del junk
    (g1,) = torch.autograd.grad(Fn.embedding(idx, w), w, g)
    (g2,) = torch.autograd.grad(Fn.embedding(idx, w), w, g)
    assert torch.equal(g1, g2)
    ref = torch.zeros(V, C, device="cuda", dtype=torch.float64)
    ref.index_add_(0, idx.reshape(-1), g.reshape(-1, C).double())
    assert torch.isfinite(g1).all()
    assert (g1.double() - ref).abs().max().item() < 1e-3
    absent = torch.ones(V, dtype=torch.bool, device="cuda")
    absent[idx.reshape(-1)] = False
    assert absent.any() and g1[absent].abs().max().item() == 0.0


def test_linear_bf16_fp32_weight_grad():
    torch.manual_seed(0)
    x = torch.randn(3, 40, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(128, 256, device="cuda") * 0.05).requires_grad_()
    y = Fn.linear(x, w)
    assert y.dtype == torch.bfloat16 and y.shape == (3, 40, 128)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    yr = xr @ wr.T
    yr.backward(g.float())
    assert w.grad.dtype == torch.float32
    assert (y.float() - yr).abs().max().item() < 5e-2
    assert (w.grad - wr.grad).abs().max().item() < 1e-2 * wr.grad.abs().max().item() + 1e-3
    assert (x.grad.float() - xr.grad).abs().max().item() < 5e-2


def test_mlp_relu2_fused_matches_composition(monkeypatch):
    monkeypatch.setenv("DION_B200_FUSED_MLP", "1")
    torch.manual_seed(0)
    B, T, C = 2, 300, 256
    h = (torch.randn(B, T, C, device="cuda") * 0.5).bfloat16().requires_grad_()
    wfc = (torch.randn(4 * C, C, device="cuda") * C ** -0.5).requires_grad_()
    wpr = (torch.randn(C, 4 * C, device="cuda") * (4 * C) ** -0.5).requires_grad_()
    y = Fn.mlp_relu2(h, wfc, wpr)
    g = torch.randn_like(y)
    y.backward(g)
    hr = h.detach().float().requires_grad_()
    wf = wfc.detach().bfloat16().float().requires_grad_()
    wp = wpr.detach().bfloat16().float().requires_grad_()
    yr = torch.relu(hr @ wf.T).square() @ wp.T
    yr.backward(g.float())

    def close(a, b, tol=3e-2):
        return (a.float() - b).abs().max().item() < tol * b.abs().max().item() + 1e-3

    assert close(y, yr)
    assert close(h.grad, hr.grad)
    assert wfc.grad.dtype == torch.float32 and close(wfc.grad, wf.grad)
    assert close(wpr.grad, wp.grad)


def test_relu2():
    x = torch.randn(16, 3072, device="cuda").bfloat16().requires_grad_()
    xr = x.detach().float().requires_grad_()
    y = Fn.relu2(x)
    yr = tF.relu(xr).square()
    g = torch.randn_like(yr)
    y.backward(g.bfloat16())
    yr.backward(g)
    assert (y.float() - yr).abs().max().item() < 0.1
    assert (x.grad.float() - xr.grad).abs().max().item() < 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V", [64, 50304])
def test_cross_entropy(dtype, V):
    torch.manual_seed(0)
    N = 300
    logits = (torch.randn(N, V, device="cuda") * 2).to(dtype)
    tgt = torch.randint(0, V, (N,), device="cuda")
    tgt[::7] = -1
    lr = logits.detach().float().requires_grad_()
    ref = tF.cross_entropy(lr, tgt, ignore_index=-1)
    ref.backward()
    lg = logits.clone().requires_grad_()
    loss = Fn.cross_entropy(lg, tgt, ignore_index=-1)
    (loss * 0.5).backward()
    assert abs(float(loss) - float(ref)) < (1e-4 if dtype == torch.float32 else 2e-2)
    tol = 1e-6 if dtype == torch.float32 else 2e-4
    assert (lg.grad.float() - 0.5 * lr.grad).abs().max().item() < tol


def test_gpt_forward_backward_matches_torch_path():
    from dion_b200.models.gpt import GPT, GPTConfig
    torch.manual_seed(0)
    cfg = GPTConfig(sequence_len=64, vocab_size=512, n_layer=2, n_head=2, n_embd=128)
    m = GPT(cfg).cuda()
    m.init_weights()
    x = torch.randint(0, 512, (3, 64), device="cuda")
    y = torch.randint(0, 512, (3, 64), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = m(x, y)
    loss.backward()
    g_fused = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    mc = GPT(cfg)
    mc.load_state_dict({k: v.cpu() for k, v in m.state_dict().items()})
    for mod in mc.modules():
        if hasattr(mod, "init_inv_freq"):
            mod.init_inv_freq()
    lc = mc(x.cpu(), y.cpu())
    lc.backward()
    assert abs(float(loss) - float(lc)) < 5e-2
    for g, p in zip(g_fused, mc.parameters()):
        denom = p.grad.abs().max().item() + 1e-6
        assert (g.cpu() - p.grad).abs().max().item() / denom < 0.1


@pytest.mark.parametrize("D", [768, 2048, 3072])
def test_add_rms_norm(D):
    torch.manual_seed(0)
    x = torch.randn(3, 21, D, device="cuda", requires_grad=True)
    d = torch.randn(3, 21, D, device="cuda").bfloat16().requires_grad_()
    xr = x.detach().clone().requires_grad_()
    dr = d.detach().float().requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        xn, h = Fn.add_rms_norm(x, d)
    assert xn.dtype == torch.float32 and h.dtype == torch.bfloat16
    xnr = xr + dr
    hr = tF.rms_norm(xnr, (D,), eps=torch.finfo(torch.float32).eps)
    g1, g2 = torch.randn_like(xnr), torch.randn_like(hr)
    (xn * g1).sum().backward(retain_graph=True)
    (h.float() * g2).sum().backward()
    ((xnr * g1).sum() + (hr * g2).sum()).backward()
    assert (xn - xnr).abs().max().item() < 1e-5
    assert (h.float() - hr).abs().max().item() < 3e-2
    assert (x.grad - xr.grad).abs().max().item() < 2e-2  # g2 passed through bf16 h
    assert (d.grad.float() - dr.grad).abs().max().item() < 5e-2
