"""The training entry point end to end: `train.py` under torchrun with two gloo ranks on synthetic
shards - data-parallel Dion with compressed gradient sync, checkpoints and an exact resume; and a
("dp", "fs", "tp") mesh with sequence-parallel tensor parallelism."""
import os
import re
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

_YAML = """
model_dim: 64
n_layer: 2
n_head: 4
sequence_length: 64
batch_size: 8
device_batch_size: 2
num_iterations: {iters}
val_loss_every: 6
val_tokens: 1024
optimizer: dion
rank_fraction: 0.5
"""


def _run(cfg, data, port, *extra):
    env = dict(os.environ)
    env.update(TORCHDYNAMO_DISABLE="1", OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "train.py"), "--config", str(cfg),
           "--data_dir", str(data), "--no_wandb", *extra]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    return out


def _val_losses(out):
    return {int(s): float(v) for s, v in re.findall(r"step:(\d+)/\d+ val_loss:([0-9.]+)", out)}


@pytest.fixture(scope="module")
def shards(tmp_path_factory):
    from dion_b200.models.data import write_synthetic_shards

    d = tmp_path_factory.mktemp("shards")
    write_synthetic_shards(str(d), 50304, train_tokens=400_000, val_tokens=66_000)
    return d


def test_ddp_training_checkpoints_and_resumes_exactly(tmp_path, shards):
    port = 29800 + os.getpid() % 100
    cfg = tmp_path / "a.yaml"
    ckpt = tmp_path / "ckpt"
    common = f"replicate_mesh_grad_sync: true\ncheckpoint_freq: 5\ncheckpoint_dir: {ckpt}\n"
    cfg.write_text(_YAML.format(iters=12) + common)
    first = _run(cfg, shards, port)
    v1 = _val_losses(first)
    assert set(v1) == {0, 6, 12} and v1[12] < v1[0], v1
    assert "Saving checkpoint" in first
    # the second run finds the checkpoint of step 10, replays steps 11-12 and goes on to 14
    cfg.write_text(_YAML.format(iters=14) + common)
    second = _run(cfg, shards, port + 1)
    assert "Resuming from step 10" in second, second[-3000:]
    v2 = _val_losses(second)
    assert v2[12] == v1[12], (v1, v2)
    assert 14 in v2


def test_mesh_training_with_sequence_parallel_tp(tmp_path, shards):
    cfg = tmp_path / "b.yaml"
    cfg.write_text(_YAML.format(iters=8))
    out = _run(cfg, shards, 29900 + os.getpid() % 100, "--dp_size", "1", "--fs_size", "1", "--tp_size", "2",
               "--sequence_parallel")
    v = _val_losses(out)
    assert set(v) == {0, 6, 8} and v[8] < v[0], v


def test_mesh_benchmark_script_smoke():
    import json

    env = dict(os.environ)
    env.update(TORCHDYNAMO_DISABLE="1", OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29950 + os.getpid() % 40),
           os.path.join(ROOT, "benchmark", "benchmark_train_mesh.py"), "--tiny", "--optimizer", "dion", "--dp", "1",
           "--fs", "1", "--tp", "2", "--sequence_parallel", "--device_batch", "2", "--steps", "2", "--warmup", "3"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, (res.stdout + res.stderr)[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["n_gpus"] == 2 and out["value"] > 0 and out["config"]["parallelism"].startswith("dp1 x fs1 x tp2")


def test_loss_curve_script_learns_the_chain(tmp_path):
    """The loss-curve comparison script: its synthetic Markov-chain tokens are learnable (the loss falls well
    below the uniform-guess level towards log(fanout)) and its comparison table prints."""
    import json

    env = dict(os.environ)
    env.update(OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    script = os.path.join(ROOT, "benchmark", "loss_curve.py")
    out_json = tmp_path / "ours.json"
    res = subprocess.run([sys.executable, script, "--tiny", "--steps", "30", "--batch", "4", "--states", "64", "--json",
                          str(out_json)], env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, (res.stdout + res.stderr)[-3000:]
    rec = json.loads(out_json.read_text())
    assert len(rec["losses"]) == 30 and rec["losses"][0] > 5.0 and rec["losses"][-1] < 2.5, rec["losses"]
    res = subprocess.run([sys.executable, script, "--compare", str(out_json), str(out_json)], env=env,
                         capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert res.returncode == 0 and "mean of the last 20 steps" in res.stdout, res.stdout + res.stderr


def test_training_on_a_dp2_fs2_tp2_mesh_with_compressed_sync(tmp_path, shards):
    """Eight gloo ranks, all three mesh dimensions active, Dion keeping the replicas in step through the
    low-rank factors: the layout of the multi-GPU benchmark, run through `train.py`."""
    env = dict(os.environ)
    env.update(TORCHDYNAMO_DISABLE="1", OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cfg = tmp_path / "c.yaml"
    cfg.write_text(_YAML.format(iters=6).replace("batch_size: 8", "batch_size: 16") + "replicate_mesh_grad_sync: true\n")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=8", "--master-addr",
           "127.0.0.1", "--master-port", str(29870 + os.getpid() % 50), os.path.join(ROOT, "train.py"), "--config",
           str(cfg), "--data_dir", str(shards), "--no_wandb", "--dp_size", "2", "--fs_size", "2", "--tp_size", "2"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    v = _val_losses(out)
    assert set(v) == {0, 6} and v[6] < v[0], v


@pytest.mark.parametrize("config", ["dion_160m", "dion_cqr_160m", "muon_160m", "dion_160m_full_rank_ddp"])
def test_shipped_configs_run_as_a_plain_python_process(tmp_path, shards, config):
    """Every recipe under configs/ parses and trains (dimensions overridden from the command line so that it runs
    on a CPU in seconds), started as `python train.py ...` without torchrun: one process, one device."""
    import yaml

    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", config + ".yaml")))
    cfg.update(val_loss_every=4, val_tokens=1024)
    path = tmp_path / "cfg.yaml"
    path.write_text(yaml.safe_dump(cfg))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    env.update(TORCHDYNAMO_DISABLE="1", OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="",
               MASTER_PORT=str(29600 + os.getpid() % 200))
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--config", str(path), "--data_dir", str(shards), "--no_wandb",
           "--model_dim", "64", "--n_layer", "2", "--n_head", "4", "--sequence_length", "64", "--batch_size", "4",
           "--device_batch_size", "2", "--num_iterations", "4"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    v = _val_losses(out)
    assert set(v) == {0, 4} and v[4] < v[0], v
