"""Dion2 selection kernels against the PyTorch path."""
import pytest
import torch

from dion_b200.ops.select import dion2_select, scatter_selected

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("select_dim", [-2, -1])
@pytest.mark.parametrize("shape,k", [((64, 96), 16), ((300, 70), 33), ((768, 3072), 192),
                                     ((3072, 768), 192)])
@pytest.mark.parametrize("m_dtype", [torch.float32, torch.bfloat16])
def test_select_matches_torch(select_dim, shape, k, m_dtype):
    torch.manual_seed(0)
    n = 3
    M = [torch.randn(*shape).to(m_dtype) for _ in range(n)]
    G = [torch.randn(*shape) for _ in range(n)]
    Mc, Gc = [m.clone() for m in M], [g.clone() for g in G]
    Mg, Gg = [m.clone().cuda() for m in M], [g.clone().cuda() for g in G]
    Uc, ic, _ = dion2_select(Gc, Mc, k, select_dim, 0.9)
    Ug, ig, maps = dion2_select(Gg, Mg, k, select_dim, 0.9)
    torch.cuda.synchronize()
    # same set of slices (order may differ), same gathered values, same momentum write-back
    for t in range(n):
        assert sorted(ic[t].tolist()) == sorted(ig[t].cpu().tolist())
        order_c = torch.argsort(ic[t])
        order_g = torch.argsort(ig[t].cpu())
        a = Uc[t].index_select(select_dim, order_c).float()
        b = Ug[t].cpu().index_select(select_dim, order_g).float()
        assert (a - b).abs().max().item() <= 4e-2
        tol = 1e-6 if m_dtype == torch.float32 else 4e-2
        assert (Mc[t].float() - Mg[t].cpu().float()).abs().max().item() <= tol
        m = maps[t].cpu()
        assert (m >= 0).sum().item() == k
        assert torch.equal(m[ig[t].cpu()].long(), torch.arange(k))


def test_ties_are_deterministic_and_lowest_index_first():
    M = [torch.zeros(32, 16, device="cuda") for _ in range(2)]
    U, idx, maps = dion2_select(None, M, 5, -2, 1.0, apply_ef=False)
    assert idx.cpu().tolist() == [[0, 1, 2, 3, 4]] * 2


def test_scatter_selected_rows():
    torch.manual_seed(0)
    src = torch.randn(2, 4, 8, device="cuda").bfloat16()
    idx = torch.tensor([[5, 1, 7, 2], [0, 9, 3, 4]], device="cuda")
    out = scatter_selected(src, idx, 10, -2)
    ref = torch.zeros(2, 10, 8, device="cuda", dtype=torch.bfloat16)
    ref.scatter_(-2, idx.unsqueeze(-1).expand_as(src), src)
    assert torch.equal(out, ref)
