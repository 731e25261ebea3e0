"""GPT model, data loader and training step on CPU."""

import numpy as np
import pytest
import torch

from dion_b200.models import GPT, GPTConfig
from dion_b200.models.data import (ArithmeticDistributedDataLoader, DistributedDataLoader, write_datafile,
                                   write_synthetic_shards)
from dion_b200.training import (Hyperparameters, TrainStep, build_arg_parser, init_optimizer, lr_lambda,
                                override_args_from_cli, parse_cli_args)

from _reference import load_reference

ref = load_reference()
CFG = dict(sequence_len=64, vocab_size=512, n_layer=2, n_head=4, n_embd=64)


def _model():
    torch.manual_seed(0)
    m = GPT(GPTConfig(**CFG))
    m.init_weights()
    return m


@pytest.mark.skipif(ref is None, reason="reference package not importable")
def test_gpt_matches_reference_model():
    from models.gpt_model import GPT as RGPT, GPTConfig as RCfg  # from the reference tree

    m = _model()
    r = RGPT(RCfg(**CFG))
    r.init_weights()
    r.load_state_dict(m.state_dict())  # same parameter names
    idx = torch.randint(0, 512, (3, 64))
    tgt = torch.randint(0, 512, (3, 64))
    tgt[0, :5] = -1
    l1, l2 = m(idx, tgt), r(idx, tgt)
    torch.testing.assert_close(l1, l2, rtol=1e-5, atol=1e-5)
    l1.backward()
    l2.backward()
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), r.named_parameters()):
        assert n1 == n2
        torch.testing.assert_close(p1.grad, p2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(m(idx, return_logits=True), r(idx, return_logits=True), rtol=1e-4, atol=1e-4)
    assert m(idx) is None


def test_gpt_init_statistics_and_generate():
    m = _model()
    w = m.transformer.h[0].mlp.c_fc.weight  # fan_out 256, fan_in 64 -> std 1/sqrt(64)
    assert abs(w.std().item() - 1 / 8) < 0.01
    w = m.transformer.h[0].mlp.c_proj.weight  # fan_out 64, fan_in 256 -> std 1/16 * 1/2
    assert abs(w.std().item() - 1 / 32) < 0.005
    assert abs(m.transformer.wte.weight.std().item() - 1.0) < 0.05
    out = m.generate(torch.randint(0, 512, (2, 5)), max_new_tokens=4, top_k=10)
    assert out.shape == (2, 9)


def test_data_loader_positions_and_state(tmp_path):
    toks = np.arange(10_000, dtype=np.uint16)
    write_datafile(str(tmp_path / "fineweb_train_000001.bin"), toks)
    write_datafile(str(tmp_path / "fineweb_train_000002.bin"), toks + 10_000)
    pat = str(tmp_path / "fineweb_train_*.bin")
    B, T = 2, 16
    loaders = [DistributedDataLoader(pat, B, T, r, 2, device="cpu") for r in range(2)]
    x0, y0 = loaders[0].next_batch()
    x1, _ = loaders[1].next_batch()
    assert x0.shape == (B, T) and x0.dtype == torch.long
    assert x0[0, 0] == 0 and x1[0, 0] == B * T and torch.equal(y0.view(-1)[:-1], x0.view(-1)[1:])
    x0b, _ = loaders[0].next_batch()
    assert x0b[0, 0] == 2 * B * T  # advances by B*T*world
    sd = loaders[0].state_dict()
    assert set(sd) == {"current_shard_rank_0", "current_position_rank_0", "dataloader_world_size"}
    fresh = DistributedDataLoader(pat, B, T, 0, 2, device="cpu")
    fresh.load_state_dict(sd)
    assert torch.equal(fresh.next_batch()[0], loaders[0].next_batch()[0])
    with pytest.raises(NotImplementedError):
        DistributedDataLoader(pat, B, T, 0, 4, device="cpu").load_state_dict(sd)
    # roll over into the second shard
    for _ in range(200):
        xb, _ = loaders[0].next_batch()
    assert loaders[0].current_shard in (0, 1)
    with pytest.raises(FileNotFoundError):
        DistributedDataLoader(str(tmp_path / "nothing_*.bin"), B, T, 0, 1, device="cpu")


def test_synthetic_shards_and_arithmetic_loader(tmp_path):
    write_synthetic_shards(str(tmp_path), 512, train_tokens=5000, val_tokens=1000, seed=3)
    ld = DistributedDataLoader(str(tmp_path / "fineweb_val_*.bin"), 2, 16, 0, 1, device="cpu")
    x, _ = ld.next_batch()
    assert int(x.max()) < 512
    np.arange(300, dtype=np.uint16).tofile(str(tmp_path / "train.bin"))
    al = ArithmeticDistributedDataLoader(str(tmp_path), 2, 16, 0, 1, device="cpu")
    x, y = al.next_batch()
    assert x[0, 0] == 0 and y[0, 0] == 1


def test_cli_yaml_precedence(tmp_path):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("lr: 0.5\nmodel_dim: 128\nmixed_precision: true\noversample: 2.0\nsave_every: 3\n")
    args = parse_cli_args(["--config", str(cfg), "--lr", "0.1"])
    hp = override_args_from_cli(Hyperparameters(), args)
    assert hp.lr == 0.1 and hp.model_dim == 128 and hp.mixed_precision is True
    assert hp.rcqr_oversample == 1.25 and hp.checkpoint_freq == 0  # unknown YAML keys are ignored
    assert {a.dest for a in build_arg_parser()._actions} >= {"dp_size", "fs_size", "tp_size", "fast_fsdp", "debug",
                                                             "no_triton", "inv_rank_fraction", "wandb_job_name"}


def test_lr_schedule():
    hp = Hyperparameters(num_iterations=100, warmup_ratio=0.1, warmdown_ratio=0.2)
    f = lr_lambda(hp)
    assert f(0) == pytest.approx(0.1) and f(9) == pytest.approx(1.0) and f(50) == 1.0
    assert f(80) == 1.0 and f(90) == pytest.approx(0.5) and f(100) == 0.0


@pytest.mark.parametrize("optimizer", ["dion", "muon", "dion_reference", "dion_simple", "muon_reference", "adamw"])
def test_training_reduces_loss(optimizer):
    m = _model()
    hp = Hyperparameters(model_dim=64, n_layer=2, n_head=4, sequence_length=64, optimizer=optimizer, lr=0.02,
                         rank_fraction=0.5, num_iterations=100)
    if optimizer == "adamw":
        hp.lr = 3e-3
    opt = init_optimizer(m, None, None, hp)
    step = TrainStep(m, m, opt, None, grad_accum=2)
    torch.manual_seed(1)
    x = torch.randint(0, 512, (4, 64))
    y = torch.randint(0, 512, (4, 64))
    losses = [float(step([(x[:2], y[:2]), (x[2:], y[2:])])) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.1, losses
    assert all(p.grad is None for p in m.parameters())


def test_train_step_reports_total_gradient_norm():
    m = _model()
    hp = Hyperparameters(model_dim=64, n_layer=2, n_head=4, sequence_length=64, optimizer="adamw", lr=0.0,
                         num_iterations=10)
    opt = init_optimizer(m, None, None, hp)
    step = TrainStep(m, m, opt, None, grad_accum=1, track_grad_norm=True)
    torch.manual_seed(2)
    x = torch.randint(0, 512, (2, 64))
    y = torch.randint(0, 512, (2, 64))
    step([(x, y)])
    m(x, y).backward()      # lr = 0: the same gradients again
    want = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in m.parameters()))
    torch.testing.assert_close(step.last_grad_norm, want, rtol=1e-5, atol=1e-6)
    assert TrainStep(m, m, opt, None).last_grad_norm is None
