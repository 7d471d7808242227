"""GPT model on CPU: shapes, generation, equivalence of the fused functional paths' fall-backs
with the module-by-module composition, and parameter naming (checkpoint compatibility with the
reference model: models/gpt_model.py:127-193)."""
import torch

from dion_b200.models import functional as Fn
from dion_b200.models.gpt import GPT, GPTConfig

CFG = dict(n_layer=2, n_embd=64, n_head=2, vocab_size=128, sequence_len=32)


def _model(seed=0):
    torch.manual_seed(seed)
    m = GPT(GPTConfig(**CFG))
    m.init_weights()
    return m


def test_forward_loss_logits_and_generate():
    m = _model()
    x = torch.randint(0, 128, (3, 16))
    y = torch.randint(0, 128, (3, 16))
    loss = m(x, y)
    assert loss.ndim == 0 and torch.isfinite(loss)
    logits = m(x, y, return_logits=True)
    assert logits.shape == (3, 16, 128) and logits.dtype == torch.float32
    last = m(x, return_logits=True)
    assert last.shape == (3, 1, 128)
    out = m.generate(x[:, :5], max_new_tokens=7, temperature=0.8, top_k=10)
    assert out.shape == (3, 12) and int(out.max()) < 128
    assert torch.equal(out[:, :5], x[:, :5])


def test_parameter_names_match_the_reference_layout():
    names = [n for n, _ in _model().named_parameters()]
    assert names[0] == "transformer.wte.weight" and names[-1] == "lm_head.weight"
    block = [n for n in names if n.startswith("transformer.h.0.")]
    assert block == [f"transformer.h.0.{k}.weight" for k in
                     ("attn.c_q", "attn.c_k", "attn.c_v", "attn.c_proj", "mlp.c_fc", "mlp.c_proj")]
    assert len(names) == 2 + 6 * CFG["n_layer"]          # no biases, no learnable norms


def test_functional_fallbacks_equal_the_plain_composition():
    torch.manual_seed(1)
    B, T, H, D = 2, 8, 2, 32
    C = H * D
    h = torch.randn(B, T, C)
    wq, wk, wv = (torch.randn(C, C) * C ** -0.5 for _ in range(3))
    fr = torch.outer(torch.arange(T).float(), 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D)))
    cos, sin = fr.cos().bfloat16(), fr.sin().bfloat16()
    q, k, v = Fn.qkv_rope(h, wq, wk, wv, cos, sin, H)
    q2 = torch.nn.functional.linear(h, wq).view(B, T, H, D)
    k2 = torch.nn.functional.linear(h, wk).view(B, T, H, D)
    q2, k2 = Fn.rope_qknorm(q2, k2, cos, sin)
    assert torch.allclose(q, q2) and torch.allclose(k, k2)
    assert torch.allclose(v, torch.nn.functional.linear(h, wv).view(B, T, H, D))
    wfc, wpr = torch.randn(4 * C, C) * 0.1, torch.randn(C, 4 * C) * 0.1
    assert torch.allclose(Fn.mlp_relu2(h, wfc, wpr),
                          torch.relu(h @ wfc.T).square() @ wpr.T, atol=1e-5)
    x, d = torch.randn(B, T, C), torch.randn(B, T, C)
    xn, hn = Fn.add_rms_norm(x, d)
    assert torch.allclose(xn, x + d)
    assert torch.allclose(hn, torch.nn.functional.rms_norm(x + d, (C,)), atol=1e-6)


def test_training_reduces_loss_on_a_repeated_batch():
    import dion_b200
    m = _model()
    opt = dion_b200.Muon(
        [dict(params=list(m.transformer.h.parameters())),
         dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()),
              algorithm="adamw", lr=3e-3)], lr=0.02)
    x = torch.randint(0, 128, (4, 16), generator=torch.Generator().manual_seed(2))
    y = torch.roll(x, -1, dims=1)
    first = last = None
    for _ in range(12):
        loss = m(x, y)
        loss.backward()
        opt.step()
        m.zero_grad(set_to_none=True)
        first = float(loss.detach()) if first is None else first
        last = float(loss.detach())
    assert last < first - 0.5


def test_weights_interchange_with_the_reference_model(ref_dion):
    """Same parameter names and the same function: a reference checkpoint loads into this model
    and gives the same loss and logits (and the other way round)."""
    from models.gpt_model import GPT as RefGPT, GPTConfig as RefConfig  # baseline/_ref/models
    ours = _model(3)
    torch.manual_seed(4)
    ref = RefGPT(RefConfig(**CFG))
    ref.init_weights()
    missing, unexpected = ref.load_state_dict(ours.state_dict(), strict=False)
    assert not [k for k in missing if "inv_freq" not in k] and not unexpected
    x = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(5))
    y = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(6))
    with torch.no_grad():
        assert abs(float(ours(x, y)) - float(ref(x, y))) < 1e-5
    assert torch.allclose(ours(x, y, return_logits=True), ref(x, y, return_logits=True), atol=1e-4)
    ours2 = _model(7)
    ours2.load_state_dict({k: v for k, v in ref.state_dict().items() if "inv_freq" not in k})
    assert torch.allclose(ours2(x, y, return_logits=True), ours(x, y, return_logits=True), atol=1e-6)


def test_reference_import_names_forward_to_this_package():
    """With ``compat/`` on the path, imports written against the reference package resolve to the
    classes and functions of this one (and only then: the folder is not on the default path)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import dion, dion_b200\n"
        "from dion import Muon, Dion2, Dion, NorMuon, NorDion2, Dion3, DionMixedPrecisionConfig\n"
        "from dion import DionSimple, DionReference, MuonReference\n"
        "assert Muon is dion_b200.Muon and Dion is dion_b200.Dion and Dion3 is NorDion2\n"
        "from dion.cuda_graph import CudaGraphOptimizer\n"
        "from dion.newton_schulz_triton import newton_schulz_triton, ns_line_1, ns_line_2, ns_line_3\n"
        "from dion.polar_express import polar_express\n"
        "from dion.opt_utils import AsyncRuntime, AsyncTask, to_local, pad_batch\n"
        "from dion.scalar_opts import adamw_update_foreach, lion_update_foreach\n"
        "from dion.megabatch_base import DistributedOrthoBase, megabatch_orthogonalize_async\n"
        "from dion.dion2_triton import dion2_post_orthogonalize_triton\n"
        "from models.gpt_model import GPT, GPTConfig, parallelize_gpt_model\n"
        "from models.gpt_utils import DistributedDataLoader\n"
        "import torch\n"
        "p = torch.nn.Parameter(torch.randn(8, 16)); p.grad = torch.randn(8, 16)\n"
        "Muon([p], lr=0.01).step()\n"
        "print('forwarded', dion.__file__)\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(root, "compat"), root]))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert os.path.join("compat", "dion") in out.stdout
    # Without the opt-in nothing named ``dion`` comes from this repository.
    plain = subprocess.run([sys.executable, "-c", "import dion_b200, sys; print('dion' in sys.modules)"],
                           env=dict(os.environ, PYTHONPATH=root), capture_output=True, text=True,
                           timeout=300)
    assert plain.stdout.strip() == "False"
