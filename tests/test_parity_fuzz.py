"""Randomly drawn configurations (shapes, options, group settings) run on this package and on the
installed reference package from the same seeds; the parameter trajectories must agree."""
import random

import pytest
import torch

import dion_b200
from tests.test_optimizers import _same_q_init


def _trajectory(pkg, name, kw, shapes, group_kw, scalar, pre=None, steps=3):
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(*s)) for s in shapes]
    v = torch.nn.Parameter(torch.randn(17))
    opt = getattr(pkg, name)([dict(params=ps, **group_kw), dict(params=[v], algorithm=scalar)],
                             lr=0.02, **kw)
    if pre is not None:
        pre(opt, ps)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        for p in ps + [v]:
            p.grad = torch.randn(p.shape, generator=g)
        opt.step()
    return [p.detach().clone() for p in ps + [v]]


def _draw_megabatch(rng):
    name = rng.choice(["Muon", "NorMuon", "Dion2", "NorDion2"])
    m, n = rng.choice([8, 12, 16, 24, 40]), rng.choice([8, 12, 16, 24, 40])
    shapes = [(m, n)] * rng.randint(1, 3) + [(n, m)] * rng.randint(0, 2)
    if rng.random() < 0.3:
        shapes.append((rng.randint(2, 3), m, n))
    kw, group_kw = {}, {}
    if rng.random() < 0.5:
        kw["cautious_wd"] = True
    if rng.random() < 0.5:
        kw["use_polar_express"] = False
    if rng.random() < 0.3:
        kw["adjust_lr"] = rng.choice(["rms_norm", None])
    if name in ("Muon", "NorMuon") and rng.random() < 0.5:
        kw["nesterov"] = True
    if name in ("Dion2", "NorDion2"):
        kw["fraction"] = rng.choice([0.25, 0.5, 1.0])
        if rng.random() < 0.4:
            kw["selection_scope"] = "global"
    if rng.random() < 0.25 and m % 4 == 0:
        shapes, group_kw = [(m, n)] * 2, dict(num_heads=rng.choice([2, 4]))
    elif rng.random() < 0.2:
        a = rng.randint(1, m - 1)
        shapes, group_kw = [(m, n)] * 2, dict(split_sizes=(a, m - a))
    return name, kw, shapes, group_kw, rng.choice(["adamw", "lion"])


@pytest.mark.parametrize("seed", range(16))
def test_random_megabatch_configuration_matches_reference(ref_dion, seed):
    name, kw, shapes, group_kw, scalar = _draw_megabatch(random.Random(seed))
    try:
        theirs = _trajectory(ref_dion, name, kw, shapes, group_kw, scalar)
    except Exception as exc:          # a combination the reference rejects must be rejected here too
        with pytest.raises(type(exc)):
            _trajectory(dion_b200, name, kw, shapes, group_kw, scalar)
        return
    ours = _trajectory(dion_b200, name, kw, shapes, group_kw, scalar)
    for a, b in zip(theirs, ours):
        assert (a - b).abs().max().item() < 1e-3, (name, kw, group_kw, shapes)


@pytest.mark.parametrize("seed", range(10))
def test_random_dion_configuration_matches_reference(ref_dion, seed):
    rng = random.Random(100 + seed)
    name = rng.choice(["Dion", "DionReference"])
    m, n = rng.choice([16, 24, 40, 64, 96]), rng.choice([16, 24, 40, 64, 96])
    shapes = [(m, n)] * rng.randint(1, 3) + [(n, m)] * rng.randint(0, 2)
    kw = dict(rank_fraction=rng.choice([0.125, 0.25, 0.5, 1.0]),
              rank_multiple_of=rng.choice([1, 4, 8]), mu=rng.choice([0.9, 0.95]),
              weight_decay=rng.choice([0.0, 0.01]))
    if name == "DionReference":
        kw.update(qr_method=rng.choice(["qr", "rcqr", "cqr"]), power_iters=rng.choice([1, 2]),
                  cqr_warmup_steps=2)
    scalar = rng.choice(["adamw", "lion"])
    theirs = _trajectory(ref_dion, name, kw, shapes, {}, scalar, pre=_same_q_init, steps=4)
    ours = _trajectory(dion_b200, name, kw, shapes, {}, scalar, pre=_same_q_init, steps=4)
    for a, b in zip(theirs, ours):
        assert (a - b).abs().max().item() < 1e-4, (name, kw, shapes)
