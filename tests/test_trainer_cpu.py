"""End-to-end checks on CPU: loss-curve parity of (our GPT + our Muon) with (reference GPT +
reference Muon) on the small configuration, the data loaders, and the trainer under torchrun with
gloo (DDP and FSDP2 + checkpoint resume)."""
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest
import torch

import dion_b200
from dion_b200.models.data import (DistributedDataLoader, SyntheticDataLoader, write_datafile)
from dion_b200.models.gpt import GPT, GPTConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = dict(sequence_len=64, vocab_size=512, n_layer=2, n_head=4, n_embd=128)


def _loss_curve(gpt_cls, cfg_cls, muon_cls, steps=6):
    torch.manual_seed(0)
    model = gpt_cls(cfg_cls(**TINY))
    model.init_weights()
    opt = muon_cls(
        [dict(params=list(model.transformer.h.parameters())),
         dict(params=list(model.transformer.wte.parameters()) + list(model.lm_head.parameters()),
              algorithm="adamw", lr=3e-3)],
        lr=0.02, mu=0.95, nesterov=True, weight_decay=0.01, use_polar_express=False)
    g = torch.Generator().manual_seed(0)
    losses = []
    for _ in range(steps):
        x = torch.randint(0, TINY["vocab_size"], (8, TINY["sequence_len"]), generator=g)
        y = torch.randint(0, TINY["vocab_size"], (8, TINY["sequence_len"]), generator=g)
        loss = model(x, y)
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        losses.append(float(loss.detach()))
    return losses


def test_loss_curve_matches_reference(ref_dion):
    from models.gpt_model import GPT as RefGPT, GPTConfig as RefConfig  # baseline/_ref/models
    ours = _loss_curve(GPT, GPTConfig, dion_b200.Muon)
    ref = _loss_curve(RefGPT, RefConfig, ref_dion.Muon)
    assert ours[0] == pytest.approx(ref[0], abs=1e-4)
    for a, b in zip(ours, ref):
        assert a == pytest.approx(b, abs=2e-2)
    assert ours[-1] < ours[0]


def test_state_dict_interchangeable_with_reference(ref_dion):
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(16, 32)), torch.nn.Parameter(torch.randn(8))]
    groups = lambda: [dict(params=[ps[0]]), dict(params=[ps[1]], algorithm="adamw")]  # noqa: E731
    ours, ref = dion_b200.NorMuon(groups(), lr=0.01), ref_dion.NorMuon(groups(), lr=0.01)
    for p in ps:
        p.grad = torch.randn_like(p)
    ours.step()
    ref.load_state_dict(ours.state_dict())     # ours -> reference
    ours.load_state_dict(ref.state_dict())     # reference -> ours
    assert set(ours.state[ps[0]]) == {"momentum", "variance_neuron"}
    assert set(ours.state[ps[1]]) == {"momentum", "variance", "step_dev"}


def test_data_loaders(tmp_path):
    toks = np.arange(5000) % 1000
    write_datafile(str(tmp_path / "fineweb_train_000000.bin"), toks)
    a = DistributedDataLoader(str(tmp_path / "fineweb_train_*.bin"), 2, 8, 0, 2)
    b = DistributedDataLoader(str(tmp_path / "fineweb_train_*.bin"), 2, 8, 1, 2)
    xa, ya = a.next_batch()
    xb, _ = b.next_batch()
    assert xa.shape == (2, 8) and torch.equal(ya[:, :-1], xa[:, 1:])
    assert int(xb[0, 0]) == 16  # rank 1 starts one device batch further
    state = a.state_dict()
    nxt = a.next_batch()[0].clone()
    a2 = DistributedDataLoader(str(tmp_path / "fineweb_train_*.bin"), 2, 8, 0, 2)
    a2.load_state_dict(state)
    assert torch.equal(a2.next_batch()[0], nxt)
    with pytest.raises(NotImplementedError):
        a2.load_state_dict({**state, "dataloader_world_size": 4})
    s1 = SyntheticDataLoader(2, 8, 100, 0, 1, seed=0)
    s2 = SyntheticDataLoader(2, 8, 100, 0, 1, seed=0)
    assert torch.equal(s1.next_batch()[0], s2.next_batch()[0])
    assert int(s1.next_batch()[0].max()) < 100


def _torchrun(args, nproc=2, timeout=900):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr",
           "127.0.0.1", "--nproc-per-node", str(nproc), os.path.join(ROOT, "train.py"),
           "--device", "cpu", "--synthetic", "--no_wandb", "--debug", "--model_dim", "64",
           "--n_layer", "2", "--n_head", "2", "--sequence_length", "32", "--batch_size", "8",
           "--device_batch_size", "4", "--val_loss_every", "0", "--scalar_opt", "adamw"] + args
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return res.stdout


def test_trainer_ddp_and_fsdp_resume(tmp_path):
    out = _torchrun(["--optimizer", "muon", "--num_iterations", "3"])
    assert out.count("train_loss=") == 3
    ck = str(tmp_path / "ckpt")
    fsdp = ["--optimizer", "normuon", "--fs_size", "2", "--checkpoint_dir", ck]
    full = _torchrun(fsdp + ["--num_iterations", "3", "--checkpoint_freq", "1"])
    assert os.path.isdir(os.path.join(ck, "step_00000001"))
    for later in ("step_00000002", "step_00000003"):
        shutil.rmtree(os.path.join(ck, later), ignore_errors=True)
    out = _torchrun(fsdp + ["--num_iterations", "3"])
    assert "Resumed from step 1" in out and "Step 0:" not in out and "Step 1:" not in out
    # The resumed run continues with the following step, on the same batches, schedule position
    # and optimizer state: its log lines repeat those of the uninterrupted run.
    line = [ln for ln in full.splitlines() if ln.startswith("Step 2:")]
    assert line and line[0] in out
    # A directory in the reference trainer's layout (one folder named "checkpoint") resumes too.
    for name in os.listdir(ck):
        if name != "step_00000001":
            shutil.rmtree(os.path.join(ck, name), ignore_errors=True)
    os.rename(os.path.join(ck, "step_00000001"), os.path.join(ck, "checkpoint"))
    out = _torchrun(fsdp + ["--num_iterations", "3"])
    assert "Resumed from step 1" in out and line[0] in out


def test_trainer_hybrid_meshes():
    """Four ranks as dp x fs (hybrid sharding, Muon and legacy Dion with compressed data-parallel
    sync) and as fs x tp (legacy Dion with tensor parallelism): the losses fall."""
    def losses(out):
        return [float(tok.split("=")[1].rstrip(",")) for tok in out.split()
                if tok.startswith("train_loss=")]
    big = ["--batch_size", "16", "--num_iterations", "3"]
    for extra in (["--optimizer", "muon", "--dp_size", "2", "--fs_size", "2"],
                  ["--optimizer", "dion", "--dp_size", "2", "--fs_size", "2",
                   "--replicate_mesh_grad_sync"],
                  ["--optimizer", "dion", "--fs_size", "2", "--tp_size", "2"]):
        ls = losses(_torchrun(extra + big, nproc=4))
        assert len(ls) == 3 and ls[-1] < ls[0], (extra, ls)


def test_trainer_on_eight_ranks_in_the_benchmark_layouts():
    """The two eight-GPU layouts named as benchmark configurations, as eight gloo processes on a
    small model: Muon with every parameter sharded eight ways (64 rows over 8 ranks), and legacy
    Dion on a dp2 x fs2 x tp2 mesh with compressed data-parallel synchronisation.  Three steps on
    random tokens say nothing about convergence (the optimizer-level tests compare eight ranks
    with a single process); here the meshes, the sharded model and the step have to work."""
    def losses(out):
        return [float(tok.split("=")[1].rstrip(",")) for tok in out.split()
                if tok.startswith("train_loss=")]
    big = ["--batch_size", "32", "--num_iterations", "3"]
    for extra in (["--optimizer", "muon", "--fs_size", "8"],
                  ["--optimizer", "dion", "--dp_size", "2", "--fs_size", "2", "--tp_size", "2",
                   "--replicate_mesh_grad_sync"]):
        ls = losses(_torchrun(extra + big, nproc=8, timeout=1500))
        assert len(ls) == 3 and all(10.0 < v < 12.5 for v in ls), (extra, ls)


def test_trace_spans_and_profile_helper():
    from dion_b200.utils import trace
    with trace.span("idle"):          # disabled (or no GPU): nothing happens
        pass
    table = trace.profile_steps(lambda: torch.ones(8).sum(), 2)
    assert "aten::sum" in table or "aten::ones" in table


def test_sectioned_and_flat_config_files_load_alike(tmp_path):
    from dion_b200.trainer import flatten_config, parse_cli_args
    assert flatten_config({"a": 1, "s": {"b": 2, "t": {"c": 3}}}) == {"a": 1, "b": 2, "c": 3}
    sectioned = tmp_path / "s.yaml"
    sectioned.write_text("model: {model_dim: 96, n_layer: 3}\noptimizer: {optimizer: muon, lr: 0.5}\n"
                         "logging: {no_wandb: true}\n")
    flat = tmp_path / "f.yaml"
    flat.write_text("model_dim: 96\nn_layer: 3\noptimizer: muon\nlr: 0.5\nno_wandb: true\n")
    a, b = parse_cli_args(["--config", str(sectioned)]), parse_cli_args(["--config", str(flat)])
    assert vars(a) | {"config": None} == vars(b) | {"config": None}
    assert a.model_dim == 96 and a.optimizer == "muon" and a.no_wandb is True
    # a flag on the command line wins over the file
    assert parse_cli_args(["--config", str(sectioned), "--lr", "0.1"]).lr == 0.1
    for name in os.listdir(os.path.join(ROOT, "configs")):
        args = parse_cli_args(["--config", os.path.join(ROOT, "configs", name)])
        assert args.optimizer and args.model_dim


def test_optimizer_factory_covers_every_choice():
    """``init_optimizer`` builds each optimizer the command line offers on a stub-free tiny model
    (no mesh, no DDP), with the matrix group first and embedding / head as scalar groups; one
    step changes the weights (reference: tests/test_dion3_alias.py:46-120 checks the alias)."""
    import argparse
    from dion_b200 import trainer
    from dion_b200.models.gpt import GPT, GPTConfig
    import dion_b200
    expected = {"muon": dion_b200.Muon, "dion2": dion_b200.Dion2, "normuon": dion_b200.NorMuon,
                "nordion2": dion_b200.NorDion2, "dion3": dion_b200.NorDion2,
                "dion": dion_b200.Dion, "dion_reference": dion_b200.DionReference,
                "dion_simple": dion_b200.DionSimple, "muon_reference": dion_b200.MuonReference,
                "adamw": torch.optim.AdamW}
    cli = argparse.Namespace()
    for name, cls in expected.items():
        torch.manual_seed(0)
        model = GPT(GPTConfig(vocab_size=64, n_layer=1, n_head=2, n_embd=16, sequence_len=8))
        model.init_weights()
        hp = trainer.Hyperparameters(optimizer=name, model_dim=16, n_layer=1, n_head=2,
                                     scalar_opt="lion" if name == "muon" else "adamw")
        opt = trainer.init_optimizer(model, None, None, hp, cli)
        assert type(opt) is cls, name
        assert len(opt.param_groups) == 3
        if name != "adamw":
            assert [g.get("algorithm") for g in opt.param_groups][1:] == [hp.scalar_opt] * 2
        idx = torch.randint(0, 64, (2, 8))
        before = [p.detach().clone() for p in model.parameters()]
        model(idx, idx).backward()
        opt.step()
        assert any(not torch.equal(a, b) for a, b in zip(before, model.parameters())), name
    with pytest.raises(ValueError):
        trainer.init_optimizer(model, None, None,
                               trainer.Hyperparameters(optimizer="sgd", model_dim=16), cli)
    with pytest.raises(ValueError):
        trainer.init_optimizer(model, None, None, trainer.Hyperparameters(
            optimizer="muon", model_dim=16, replicate_mesh_grad_sync=True), cli)


def test_trainer_runs_as_a_plain_single_process():
    """``python train.py`` without a launcher is a one-process job; validation and the
    optimizer timer report at the validation steps."""
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")}
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--device", "cpu", "--synthetic",
           "--no_wandb", "--debug", "--model_dim", "64", "--n_layer", "2", "--n_head", "2",
           "--sequence_length", "32", "--batch_size", "8", "--device_batch_size", "4",
           "--val_loss_every", "2", "--val_tokens", "512", "--scalar_opt", "lion",
           "--num_iterations", "4", "--optimizer", "dion2", "--time_optimizer"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    assert res.stdout.count("train_loss=") == 4
    assert res.stdout.count("val_loss:") == 3 and "opt_avg:" in res.stdout


def test_token_shard_loader_reads_what_the_reference_loader_reads(ref_dion, tmp_path, monkeypatch):
    """Same files, same ranks: identical batches and identical checkpoint state, across shard
    boundaries and the wrap-around to the first shard (reference: models/gpt_utils.py:40-104;
    its ``.cuda()`` calls are made no-ops so that it runs here)."""
    from models.gpt_utils import DistributedDataLoader as RefLoader   # from baseline/_ref
    monkeypatch.setattr(torch.Tensor, "cuda", lambda self, *a, **k: self)
    rng = np.random.default_rng(0)
    for i, n in enumerate((700, 450, 620)):
        write_datafile(str(tmp_path / f"fineweb_train_{i:06d}.bin"), rng.integers(0, 50000, n))
    pattern = str(tmp_path / "fineweb_train_*.bin")
    for rank in (0, 1):
        ours = DistributedDataLoader(pattern, 2, 16, rank, 2, device=torch.device("cpu"))
        ref = RefLoader(pattern, 2, 16, rank, 2)
        for step in range(40):
            (x, y), (rx, ry) = ours.next_batch(), ref.next_batch()
            assert torch.equal(x.cpu(), rx) and torch.equal(y.cpu(), ry), (rank, step)
            assert ours.state_dict() == ref.state_dict(), (rank, step)


def test_arithmetic_loader_reads_what_the_reference_loader_reads(ref_dion, tmp_path, monkeypatch):
    """Header-less uint16 files: circular strided reading (with wrap-around) and, for a file
    shorter than one batch, random windows drawn from numpy's global generator - both as the
    reference does (models/gpt_utils.py:107-168)."""
    from models.gpt_utils import ArithmeticDistributedDataLoader as RefLoader
    from dion_b200.models.data import ArithmeticDistributedDataLoader
    monkeypatch.setattr(torch.Tensor, "cuda", lambda self, *a, **k: self)
    rng = np.random.default_rng(1)
    rng.integers(0, 60000, 1000).astype(np.uint16).tofile(str(tmp_path / "train.bin"))
    rng.integers(0, 60000, 40).astype(np.uint16).tofile(str(tmp_path / "val.bin"))
    for rank in (0, 1, 2):
        ours = ArithmeticDistributedDataLoader(str(tmp_path), 2, 16, rank, 3,
                                               device=torch.device("cpu"))
        ref = RefLoader(str(tmp_path), 2, 16, rank, 3)
        for step in range(30):                                   # 30 * 96 tokens: wraps 2-3 times
            (x, y), (rx, ry) = ours.next_batch(), ref.next_batch()
            assert torch.equal(x.cpu(), rx) and torch.equal(y.cpu(), ry), (rank, step)
    ours = ArithmeticDistributedDataLoader(str(tmp_path), 4, 16, 0, 1, split="val",
                                           device=torch.device("cpu"))
    ref = RefLoader(str(tmp_path), 4, 16, 0, 1, split="val")
    np.random.seed(5)
    x, y = ours.next_batch()
    np.random.seed(5)
    rx, ry = ref.next_batch()
    assert torch.equal(x.cpu(), rx) and torch.equal(y.cpu(), ry)


def test_hyperparameter_defaults_and_flags_match_the_reference_trainer(ref_dion):
    """Field names and default values of ``Hyperparameters`` and the set of command-line flags are
    those of the reference trainer (read from its source text, train.py:35-213, not imported)."""
    import ast
    import dataclasses
    import re
    from dion_b200 import trainer
    path = os.path.join(ROOT, "baseline", "_ref", "train.py")
    if not os.path.exists(path):
        pytest.skip("reference trainer not copied beside the reference package")
    source = open(path).read()
    theirs = {}
    for node in ast.parse(source).body:
        if isinstance(node, ast.ClassDef) and node.name == "Hyperparameters":
            for st in node.body:
                if isinstance(st, ast.AnnAssign) and st.value is not None:
                    theirs[st.target.id] = eval(compile(ast.Expression(st.value), "<ref>", "eval"))
    ours = {f.name: f.default for f in dataclasses.fields(trainer.Hyperparameters)}
    assert theirs and ours == theirs
    ref_flags = set(re.findall(r'"--([a-z_0-9]+)"', source))
    our_flags = set(re.findall(r'"--([a-z_0-9]+)"', open(trainer.__file__).read()))
    assert ref_flags <= our_flags, sorted(ref_flags - our_flags)


def test_every_shipped_configuration_uses_known_flags():
    """Each key of every file under ``configs/`` is a flag of the trainer (a misspelt key would
    be ignored silently), and the files parse into usable hyper-parameters."""
    import glob
    import yaml
    from dion_b200 import trainer
    files = sorted(glob.glob(os.path.join(ROOT, "configs", "*.yaml")))
    assert len(files) >= 4
    for path in files:
        flat = trainer.flatten_config(yaml.safe_load(open(path)))
        args = trainer.parse_cli_args(["--config", path])
        unknown = [k for k in flat if not hasattr(args, k)]
        assert not unknown, (os.path.basename(path), unknown)
        hp = trainer.override_args_from_cli(trainer.Hyperparameters(), args)
        assert hp.optimizer in ("dion", "dion2", "muon", "normuon", "nordion2", "dion3")
        assert hp.batch_size % hp.device_batch_size == 0 and hp.model_dim % hp.n_head == 0


HEADLINE_CPU = dict(sequence_len=256, vocab_size=50304, n_layer=4, n_head=4, n_embd=256)


def _muon_adamw(muon_cls, model, **kw):
    return muon_cls(
        [dict(params=list(model.transformer.h.parameters())),
         dict(params=list(model.transformer.wte.parameters()) + list(model.lm_head.parameters()),
              algorithm="adamw", lr=3e-3, betas=(0.9, 0.95))],
        lr=0.02, mu=0.95, nesterov=True, weight_decay=0.01, use_polar_express=False, **kw)


def _small_gpt_curve(gpt_cls, cfg_cls, muon_cls, steps=20):
    """4 layers, d_model 256, 4 heads, vocabulary 50304, sequence 256, batch 8; fp32 weights from
    seed 0, uniform-random tokens from seed 0; Muon (momentum 0.95, Nesterov, quintic
    coefficients, lr 0.02, wd 0.01) + AdamW (lr 3e-3, betas 0.9 / 0.95) on embedding and head."""
    torch.manual_seed(0)
    model = gpt_cls(cfg_cls(**HEADLINE_CPU))
    model.init_weights()
    opt = _muon_adamw(muon_cls, model)
    g = torch.Generator().manual_seed(0)
    losses = []
    for _ in range(steps):
        x = torch.randint(0, 50304, (8, 256), generator=g)
        y = torch.randint(0, 50304, (8, 256), generator=g)
        loss = model(x, y)
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        losses.append(float(loss.detach()))
    return losses


def test_small_gpt_twenty_step_curve_matches_reference(ref_dion):
    from models.gpt_model import GPT as RefGPT, GPTConfig as RefConfig
    ours = _small_gpt_curve(GPT, GPTConfig, dion_b200.Muon)
    ref = _small_gpt_curve(RefGPT, RefConfig, ref_dion.Muon)
    assert len(ours) == 20 and ours[0] == pytest.approx(ref[0], abs=1e-5)
    assert max(abs(a - b) for a, b in zip(ours, ref)) < 2e-3


def _small_gpt_ddp_worker(rank, world, steps):
    from torch.nn.parallel import DistributedDataParallel
    import torch.distributed as dist
    torch.manual_seed(0)
    model = GPT(GPTConfig(**HEADLINE_CPU))
    model.init_weights()
    ddp = DistributedDataParallel(model)
    opt = _muon_adamw(dion_b200.Muon, model, distributed_mesh=ddp.process_group)
    g = torch.Generator().manual_seed(0)
    per = 8 // world
    losses = []
    for _ in range(steps):
        x = torch.randint(0, 50304, (8, 256), generator=g)
        y = torch.randint(0, 50304, (8, 256), generator=g)
        loss = ddp(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per])
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        mean = loss.detach().clone()
        dist.all_reduce(mean)
        losses.append(float(mean) / world)
    return losses if rank == 0 else None


def test_small_gpt_curve_under_ddp_on_two_gloo_ranks(tmp_path):
    """The same run as two data-parallel ranks (each half of every batch, Muon given the DDP
    process group) follows the single-process curve."""
    from tests.dist_utils import run_ranks
    steps = 8
    ddp = run_ranks(_small_gpt_ddp_worker, 2, "gloo", (steps,), str(tmp_path))[0]
    single = _small_gpt_curve(GPT, GPTConfig, dion_b200.Muon, steps=steps)
    assert max(abs(a - b) for a, b in zip(ddp, single)) < 2e-3
