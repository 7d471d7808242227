"""Newton-Schulz drivers: CPU math, and the CUDA kernels against the CPU/PyTorch oracle."""
import pytest
import torch

from dion_b200.ops import newton_schulz as NS


def _orth_err(X):
    X = X.float()
    if X.size(-2) > X.size(-1):
        X = X.mT
    eye = torch.eye(X.size(-2), device=X.device)
    return ((X @ X.mT) - eye).abs().max().item()


@pytest.mark.parametrize("name,fn", [("quintic", NS.newton_schulz_quintic),
                                     ("polar_express", NS.polar_express),
                                     ("aol", NS.newton_schulz_aol),
                                     ("gram", NS.gram_newton_schulz)])
@pytest.mark.parametrize("shape", [(48, 48), (32, 96), (96, 32), (3, 40, 64)])
def test_cpu_orthogonality(name, fn, shape):
    torch.manual_seed(0)
    G = torch.randn(*shape)
    X = fn(G)
    assert X.shape == G.shape and X.dtype == torch.bfloat16
    assert _orth_err(X) < 0.35  # five bf16 iterations leave singular values in [0.7, 1.2]


def test_classic_matches_reference_coeffs(ref_dion):
    from dion.muon_reference import zeropower_via_newtonschulz5 as ref_ns
    torch.manual_seed(0)
    G = torch.randn(64, 96)
    got = NS.newton_schulz_classic(G, epsilon=1e-7, steps=5)
    assert (got.float() - ref_ns(G, 5, 1e-7).float()).abs().max().item() < 2e-2


def test_cpu_matches_reference(ref_dion):
    from dion.muon import zeropower_via_newtonschulz5
    from dion.polar_express import polar_express
    torch.manual_seed(0)
    G = torch.randn(4, 64, 96)
    assert torch.equal(NS.newton_schulz_quintic(G, 1e-7), zeropower_via_newtonschulz5(G, 1e-7))
    assert (NS.polar_express(G, 1e-6).float() - polar_express(G, 1e-6).float()).abs().max() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["quintic", "classic", "polar_express", "aol", "gram"])
@pytest.mark.parametrize("shape", [(6, 768, 768), (2, 768, 3072), (2, 3072, 768), (3, 192, 768),
                                   (1, 100, 52), (256, 256)])
def test_cuda_vs_torch(variant, shape):
    from dion_b200.ops.gemm import check_status
    fn = {"quintic": NS.newton_schulz_quintic, "classic": NS.newton_schulz_classic,
          "polar_express": NS.polar_express, "aol": NS.newton_schulz_aol,
          "gram": NS.gram_newton_schulz}[variant]
    torch.manual_seed(0)
    G = torch.randn(*shape, device="cuda")
    got = fn(G)
    torch.cuda.synchronize()
    check_status()
    ref = NS.torch_reference(variant)(G)
    assert got.shape == G.shape and got.dtype == torch.bfloat16
    # Entries of an orthogonalized matrix are O(1/sqrt(n)), so a bound on the largest absolute
    # difference says little: compare every matrix by its relative Frobenius error.  Two bf16
    # evaluations of the same five iterations differ by a few percent (different accumulation
    # order and rounding points); a wrong coefficient or operand gives errors of order one.
    # Gram-NS keeps less precision in the small matrix it iterates on.
    g3 = got.float().reshape(-1, *got.shape[-2:])
    r3 = ref.float().reshape(-1, *ref.shape[-2:])
    rel = (g3 - r3).flatten(1).norm(dim=1) / r3.flatten(1).norm(dim=1)
    assert rel.max().item() < (0.2 if variant == "gram" else 0.1), rel.tolist()
    assert _orth_err(got) < 0.4


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 768, 768), (4, 768, 768), (1, 768, 3072), (1, 3072, 768),
                                   (3, 200, 136), (1, 1024, 1024)])
def test_one_launch_loop_matches_per_gemm_launches(shape, monkeypatch):
    """Small batches run all fifteen GEMMs of the loop in one cooperative launch with grid-wide
    barriers between them; the result is that of the three-launches-per-iteration path."""
    from dion_b200.ops import _backend, gemm
    from dion_b200.ops.gemm import check_status
    torch.manual_seed(1)
    G = torch.randn(*shape, device="cuda")
    monkeypatch.setenv("DION_B200_PERSISTENT_NS", "0")
    ref = NS.newton_schulz_quintic(G)
    monkeypatch.setenv("DION_B200_PERSISTENT_NS", "1")
    assert gemm.persistent_fits(G.bfloat16().contiguous(), *shape, 5)
    before = _backend.launch_count()
    got = NS.newton_schulz_quintic(G)
    launches = _backend.launch_count() - before
    torch.cuda.synchronize()
    check_status()
    assert launches <= 3                          # norm (2 kernels) + the loop
    g3, r3 = got.float().reshape(-1, *shape[-2:]), ref.float().reshape(-1, *shape[-2:])
    rel = (g3 - r3).flatten(1).norm(dim=1) / r3.flatten(1).norm(dim=1)
    assert rel.max().item() < 2e-2, rel.tolist()
    assert _orth_err(got) < 0.4
    # Bitwise repeatable for a given input scale (the scale itself comes from floating-point
    # atomics, so whole calls are only repeatable to the last bit of the scale); also shows that
    # the barrier counter is left at zero.
    B_, m, n = shape
    g = min(m, n)
    X0 = G.bfloat16().contiguous()
    scale = (1.0 / (X0.float().flatten(1).norm(dim=1) + 1e-7)).contiguous()
    outs = []
    for _ in range(3):
        X = X0.clone()
        bufs = [torch.empty_like(X), torch.empty(B_, g, g, device="cuda", dtype=torch.bfloat16),
                torch.empty(B_, g, g, device="cuda", dtype=torch.bfloat16)]
        outs.append(gemm.ns_persistent(X, bufs[0], bufs[1], bufs[2], NS.QUINTIC_COEFFS,
                                       scale).clone())
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
