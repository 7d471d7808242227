"""Element-wise optimizers on the host (the arithmetic the CUDA kernels are tested against):
AdamW against torch's own, Lion and cautious weight decay against hand-computed values
(the reference keeps the same checks on its GPU path, tests/test_adamw_foreach.py)."""
import pytest
import torch

from dion_b200.ops import foreach as F


def test_adamw_follows_torch_adamw():
    torch.manual_seed(0)
    shapes = [(7,), (3, 5), (2, 3, 4)]
    ours = [torch.randn(s) for s in shapes]
    theirs = [torch.nn.Parameter(t.clone()) for t in ours]
    M = [torch.zeros_like(t) for t in ours]
    V = [torch.zeros_like(t) for t in ours]
    ref = torch.optim.AdamW(theirs, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 6):
        grads = [torch.randn(s) for s in shapes]
        for p, g in zip(theirs, grads):
            p.grad = g.clone()
        ref.step()
        F.adamw(ours, grads, M, V, 3e-3, 0.9, 0.95, 0.1, 1e-8, step=step)
        for a, b in zip(ours, theirs):
            assert torch.allclose(a, b.detach(), rtol=1e-5, atol=1e-6), step


def test_adamw_device_counter_form_equals_host_step_form():
    torch.manual_seed(1)
    x1 = [torch.randn(6, 4), torch.randn(9)]
    x2 = [t.clone() for t in x1]
    s1 = [[torch.zeros_like(t) for t in x1] for _ in range(2)]
    s2 = [[torch.zeros_like(t) for t in x1] for _ in range(2)]
    shared = torch.zeros(())                              # one counter shared by both tensors
    lr = torch.tensor(0.01)
    for step in range(1, 4):
        g = [torch.randn_like(t) for t in x1]
        F.adamw(x1, g, s1[0], s1[1], 0.01, 0.9, 0.99, 0.0, 1e-8, step=step)
        F.adamw(x2, g, s2[0], s2[1], lr, 0.9, 0.99, 0.0, 1e-8, state_steps=[shared, shared])
        assert float(shared) == step                     # advanced once, not once per tensor
        for a, b in zip(x1, x2):
            assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)
    with pytest.raises(ValueError):
        F.adamw(x1, g, s1[0], s1[1], 0.01, 0.9, 0.99, 0.0, 1e-8)
    with pytest.raises(TypeError):
        F.adamw(x1, g, s1[0], s1[1], 0.01, 0.9, 0.99, 0.0, 1e-8, state_steps=[shared, shared])


def test_lion_and_cautious_weight_decay_by_hand():
    x = torch.tensor([1.0, -2.0, 3.0, -4.0])
    g = torch.tensor([0.5, 0.5, -0.5, -0.5])
    m = torch.tensor([1.0, -1.0, 1.0, -1.0])
    lr, b1, b2, wd = 0.1, 0.9, 0.99, 0.5
    update = torch.sign(b1 * m + (1 - b1) * g)            # [+, -, +, -]
    want_x = x * (1 - lr * wd) - lr * update
    want_m = b2 * m + (1 - b2) * g
    xs, ms = [x.clone()], [m.clone()]
    F.lion(xs, [g], ms, lr, b1, b2, wd)
    assert torch.allclose(xs[0], want_x) and torch.allclose(ms[0], want_m)
    # cautious: decay only where update and weight agree in sign
    xs, ms = [torch.tensor([1.0, -2.0, 3.0, -4.0])], [torch.tensor([1.0, 1.0, -1.0, -1.0])]
    g0 = torch.zeros(4)
    F.lion(xs, [g0], ms, lr, b1, b2, wd, cautious_wd=True)
    upd = torch.tensor([1.0, 1.0, -1.0, -1.0])
    agree = torch.tensor([1.0, 0.0, 0.0, 1.0])            # sign(update) == sign(x)
    assert torch.allclose(xs[0], x * (1 - lr * wd * agree) - lr * upd)


def test_adamw_cautious_weight_decay_masks_by_momentum_sign():
    x = [torch.tensor([2.0, -2.0, 2.0, -2.0])]
    g = [torch.tensor([1.0, 1.0, -1.0, -1.0])]
    m, v = [torch.zeros(4)], [torch.zeros(4)]
    F.adamw(x, g, m, v, 0.1, 0.9, 0.999, 0.5, 1e-8, step=1, cautious_wd=True)
    # after the moment update m has the sign of g; decay applies where m * x >= 0
    decay = torch.tensor([1.0, 0.0, 0.0, 1.0])
    base = torch.tensor([2.0, -2.0, 2.0, -2.0])
    adam = 0.1 * torch.tensor([1.0, 1.0, -1.0, -1.0])     # bias-corrected m / sqrt(v) = sign(g)
    assert torch.allclose(x[0], base * (1 - 0.1 * 0.5 * decay) - adam, atol=1e-5)
