"""GPT training entry point: configuration (dataclass <- YAML <- CLI), distributed set-up
(DDP process group or a ("dp", "fs", "tp") device mesh), optimizer construction with the
matrix / embedding / lm_head parameter groups, distributed checkpointing, the learning-rate
schedule and the timed training loop.

Flags, YAML handling, parameter groups, checkpoint contents and the loop structure follow
the reference trainer (train.py:32-73 hyper-parameters, 85-235 CLI, 238-297 distributed
init, 300-473 optimizer set-up, 476-579 checkpoints, 582-959 main loop).
"""

from __future__ import annotations

import argparse
import math
import os
import shutil
import tempfile
import time
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Callable, List, Optional

import torch
import torch.distributed as dist
import yaml

from . import ops
from .models.data import DistributedDataLoader
from .models.gpt import GPT, GPTConfig, parallelize_gpt_model
from .optim import Dion, DionMixedPrecisionConfig, DionReference, DionSimple, Muon, MuonReference
from .utils.health import StepHeartbeat
from .utils.timers import PhaseTimers


@dataclass
class Hyperparameters:
    data_dir: str = "data/fineweb10B"
    # training
    batch_size: int = 8 * 64          # global batch size in sequences
    device_batch_size: int = 64       # sequences per device per micro-step
    sequence_length: int = 1024
    num_iterations: int = 5000
    warmup_ratio: float = 0.01
    warmdown_ratio: float = 0.2
    # model
    model_dim: int = 768
    n_layer: int = 12
    n_head: int = 6
    # evaluation and logging
    val_loss_every: int = 125
    val_tokens: int = 10485760
    checkpoint_freq: int = 0
    checkpoint_dir: Optional[str] = None
    wandb_project_name: str = "dion-test"
    # optimizer
    optimizer: str = "dion"
    scalar_opt: str = "lion"
    lr: float = 0.02
    mu: float = 0.95
    weight_decay: float = 0.01
    rank_fraction: float = 0.125
    qr_method: str = "rcqr"
    cqr_warmup: float = 0.05
    rcqr_oversample: float = 1.25
    replicate_mesh_grad_sync: bool = False
    mixed_precision: bool = False
    adjust_lr: str = "spectral_norm"


_MASTER = True


def print0(*args, **kwargs):
    if _MASTER:
        print(*args, **kwargs, flush=True)


_STORE_TRUE_FLAGS = ("mixed_precision", "replicate_mesh_grad_sync", "fast_fsdp", "no_wandb", "no_compile",
                     "no_triton", "debug", "sequence_parallel")


def build_arg_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Train the GPT model with Dion / Muon on B200")
    p.add_argument("--config", type=str, help="YAML file whose keys match the flags (CLI values win)")
    p.add_argument("--data_dir", type=str, default=None)
    p.add_argument("--checkpoint_dir", type=str, default=None)
    p.add_argument("--checkpoint_freq", type=int, default=None)
    p.add_argument("--optimizer", type=str, default=None)
    p.add_argument("--scalar_opt", type=str, default=None)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--adjust_lr", type=str, default=None)
    p.add_argument("--inv_rank_fraction", type=int, default=None, help="1/r rank fraction for Dion")
    p.add_argument("--qr_method", type=str, default=None, choices=["qr", "cqr", "rcqr"])
    p.add_argument("--mixed_precision", action="store_true")
    p.add_argument("--model_dim", type=int, default=None)
    p.add_argument("--n_layer", type=int, default=None)
    p.add_argument("--n_head", type=int, default=None)
    p.add_argument("--num_iterations", type=int, default=None)
    p.add_argument("--batch_size", type=int, default=None)
    p.add_argument("--device_batch_size", type=int, default=None)
    p.add_argument("--sequence_length", type=int, default=None)
    p.add_argument("--warmup_ratio", type=float, default=None)
    p.add_argument("--warmdown_ratio", type=float, default=None)
    p.add_argument("--no_wandb", action="store_true")
    p.add_argument("--wandb_project_name", type=str, default=None)
    p.add_argument("--wandb_job_name", type=str, default=None)
    p.add_argument("--dp_size", type=int, default=None)
    p.add_argument("--fs_size", type=int, default=None)
    p.add_argument("--tp_size", type=int, default=None)
    p.add_argument("--replicate_mesh_grad_sync", action="store_true")
    p.add_argument("--fast_fsdp", action="store_true")
    p.add_argument("--sequence_parallel", action="store_true",
                   help="tensor parallelism with the residual stream sharded over the tokens")
    p.add_argument("--debug", action="store_true")
    p.add_argument("--no_compile", action="store_true", help="accepted for compatibility; nothing is compiled")
    p.add_argument("--no_triton", action="store_true", help="accepted for compatibility; no Triton is used")
    return p


def parse_cli_args(argv=None) -> argparse.Namespace:
    """CLI first, then YAML fills every key the CLI left unset; store_true flags are OR-ed
    (train.py:198-224)."""
    args = build_arg_parser().parse_args(argv)
    if args.config:
        with Path(args.config).open("r") as f:
            cfg = yaml.safe_load(f) or {}
        for k, v in cfg.items():
            if getattr(args, k, None) is None:
                setattr(args, k, v)
        for flag in _STORE_TRUE_FLAGS:
            if cfg.get(flag, False):
                setattr(args, flag, True)
    return args


def override_args_from_cli(hp: Hyperparameters, cli_args: argparse.Namespace) -> Hyperparameters:
    """Only keys that are dataclass fields are applied; anything else in the YAML is ignored."""
    names = {f.name for f in fields(hp)}
    for key, value in vars(cli_args).items():
        if value is not None and key in names:
            print0(f"Setting hyperparameter {key}={value}")
            setattr(hp, key, value)
    return hp


def init_distributed(dp_size, fs_size, tp_size, backend: Optional[str] = None):
    """DDP process group when no mesh size is given, else a ("dp", "fs", "tp") device mesh."""
    global _MASTER
    if not any(v in os.environ for v in ("RANK", "LOCAL_RANK", "WORLD_SIZE")):
        # started as a plain `python train.py ...`: one process, one device (the reference insists on torchrun here)
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
    assert all(v in os.environ for v in ("RANK", "LOCAL_RANK", "WORLD_SIZE")), \
        "This script must be launched using the 'torchrun' command."
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    _MASTER = rank == 0
    cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if cuda else "gloo")
    if cuda:
        torch.cuda.set_device(local_rank)
    dims = (dp_size, fs_size, tp_size)
    if all(d is None for d in dims):
        if not dist.is_initialized():
            dist.init_process_group(backend=backend)
        print0("=" * 80)
        print0(f"Distributed training initialized with DDP, world size {world}")
        return None
    assert all(d is not None for d in dims), \
        f"All mesh dimensions (dp_size, fs_size, tp_size) must be specified, but got {dims}"
    total = dp_size * fs_size * tp_size
    assert world == total, f"World size {world} does not match expected size {total} (DP {dp_size}, FS {fs_size}, TP {tp_size})"
    from torch.distributed.device_mesh import init_device_mesh

    mesh = init_device_mesh("cuda" if cuda else "cpu", (dp_size, fs_size, tp_size), mesh_dim_names=("dp", "fs", "tp"))
    print0("=" * 80)
    print0(f"Distributed training initialized with DeviceMesh: DP {dp_size} FS {fs_size} TP {tp_size}")
    return mesh


def make_param_groups(model: GPT, hp: Hyperparameters) -> List[dict]:
    """Block matrices use the optimizer defaults; the embedding and lm_head use the scalar
    optimizer without weight decay, the lm_head with lr / sqrt(d) (train.py:312-337).  The
    ``betas`` key is carried (and ignored by Dion / Muon, which read beta1 / beta2) like in
    the reference."""
    return [
        dict(params=list(model.transformer.h.parameters())),
        dict(params=list(model.transformer.wte.parameters()), algorithm=hp.scalar_opt, lr=hp.lr, betas=(0.95, 0.98),
             weight_decay=0),
        dict(params=list(model.lm_head.parameters()), algorithm=hp.scalar_opt, lr=hp.lr / math.sqrt(hp.model_dim),
             betas=(0.95, 0.98), weight_decay=0),
    ]


def init_optimizer(model: GPT, device_mesh, replicate_group, hp: Hyperparameters, cli_args=None):
    """Build the optimizer named by ``hp.optimizer`` (train.py:300-473)."""
    if hp.scalar_opt not in ("adamw", "lion"):
        raise ValueError(f"Unrecognized scalar optimizer: {hp.scalar_opt}")
    groups = make_param_groups(model, hp)
    if device_mesh is not None:
        replicate_mesh = device_mesh["dp"]
        outer = device_mesh["fs"]
        inner = device_mesh["tp"] if device_mesh["tp"].size() > 1 else None
    else:
        replicate_mesh, outer, inner = replicate_group, None, None
    mp = DionMixedPrecisionConfig(momentum_dtype=torch.bfloat16, variance_dtype=torch.bfloat16,
                                  Q_dtype=torch.bfloat16) if hp.mixed_precision else None
    name = hp.optimizer
    if name in ("dion", "dion_reference"):
        print0(f"Dion rank fraction: {hp.rank_fraction}; mixed precision: {hp.mixed_precision}; "
               f"compressed data-parallel gradient sync: {hp.replicate_mesh_grad_sync}")
        cls = Dion if name == "dion" else DionReference
        kw = dict(replicate_mesh=replicate_mesh, outer_shard_mesh=outer, inner_shard_mesh=inner,
                  replicate_mesh_grad_sync=hp.replicate_mesh_grad_sync, rank_fraction=hp.rank_fraction, lr=hp.lr,
                  mu=hp.mu, weight_decay=hp.weight_decay,
                  cqr_warmup_steps=round(hp.cqr_warmup * hp.num_iterations), rcqr_oversample=hp.rcqr_oversample,
                  mixed_precision_config=mp)
        # the batched Dion accepts only "rcqr"; its CholeskyQR2 needs no method switch
        kw["qr_method"] = hp.qr_method if name == "dion_reference" else "rcqr"
        opt = cls(groups, **kw)
    elif name == "muon":
        if device_mesh is not None:
            if inner is not None and inner.size() > 1:
                raise ValueError("Tensor parallel is not supported by Muon.")
            mesh = outer if outer.size() > 1 else replicate_mesh
        else:
            mesh = replicate_group
        opt = Muon(groups, distributed_mesh=mesh, lr=hp.lr, mu=hp.mu, weight_decay=hp.weight_decay, nesterov=True,
                   adjust_lr=hp.adjust_lr, use_triton=not getattr(cli_args, "no_triton", False))
    elif name == "dion_simple":
        assert device_mesh is None, f"{name} does not support device mesh"
        opt = DionSimple(groups, lr=hp.lr, mu=hp.mu, weight_decay=hp.weight_decay,
                         rank=round(hp.rank_fraction * hp.model_dim))
    elif name == "muon_reference":
        opt = MuonReference(groups, lr=hp.lr, mu=hp.mu, weight_decay=hp.weight_decay, nesterov=True,
                            adjust_lr=hp.adjust_lr)
    elif name == "adamw":
        for g in groups:
            g["lr"] = hp.lr
            g["betas"] = (0.9, 0.95)
            g.pop("algorithm", None)
        opt = torch.optim.AdamW(groups, lr=hp.lr, betas=(0.9, 0.95), weight_decay=hp.weight_decay)
    else:
        raise ValueError(f"Unsupported optimizer: {name}")
    if hp.replicate_mesh_grad_sync and name not in ("dion", "dion_reference"):
        raise ValueError("replicate_mesh_grad_sync is set for non-Dion optimizer")
    if not hp.replicate_mesh_grad_sync and name in ("dion", "dion_reference"):
        print0("Warning: not using replicate_mesh_grad_sync for Dion optimizer")
    return opt


def lr_lambda(hp: Hyperparameters) -> Callable[[int], float]:
    """Trapezoid: linear warm-up, constant, linear warm-down (train.py:740-750)."""
    warmup = round(hp.warmup_ratio * hp.num_iterations)
    warmdown = round(hp.warmdown_ratio * hp.num_iterations)

    def fn(it: int) -> float:
        if it < warmup:
            return (it + 1) / warmup
        if it <= hp.num_iterations - warmdown:
            return 1.0
        return (hp.num_iterations - it) / warmdown

    return fn


class CheckpointManager:
    """torch.distributed.checkpoint directories holding model, optimizer, both data-loader
    positions, the step and the wandb id; written into a temporary directory first and moved
    into place by rank 0 (train.py:476-579)."""

    DEFAULT_NAME = "checkpoint"
    OLD_SUFFIX = ".old"  # where save() sets the previous checkpoint aside while the new one takes its name

    def __init__(self, checkpoint_dir, model, optimizer, train_loader, val_loader, wandb_id=None):
        self.checkpoint_dir = checkpoint_dir
        self.model = model
        self.optimizer = optimizer
        self.train_loader = train_loader
        self.val_loader = val_loader
        self.wandb_id = wandb_id
        self.step: Optional[int] = None

    def _state(self) -> dict:
        from torch.distributed.checkpoint.state_dict import get_state_dict

        model_state, opt_state = get_state_dict(self.model, self.optimizer)
        return {"model": model_state, "optimizer": opt_state, "train_loader": self.train_loader.state_dict(),
                "val_loader": self.val_loader.state_dict(), "step": self.step, "wandb_id": self.wandb_id}

    def save(self, name: Optional[str] = None, step: Optional[int] = None):
        import torch.distributed.checkpoint as dcp

        assert self.checkpoint_dir, "Checkpoint directory must be specified"
        self.step = step
        path = os.path.join(self.checkpoint_dir, name or self.DEFAULT_NAME)
        print0(f"Saving checkpoint to {path}")
        tmpdir = None
        if dist.get_rank() == 0:
            os.makedirs(self.checkpoint_dir, exist_ok=True)
            tmpdir = tempfile.mkdtemp(dir=self.checkpoint_dir)
        box = [tmpdir]
        dist.broadcast_object_list(box, src=0)
        tmpdir = box[0]
        dcp.save(self._state(), checkpoint_id=tmpdir)
        dist.barrier()
        if dist.get_rank() == 0:
            # Swap by renames, so that a complete checkpoint exists at every instant: the previous one
            # is set aside, the new one takes its name, and only then is the previous one deleted.
            # load() looks at the set-aside copy when the name itself is missing.
            old = path + self.OLD_SUFFIX
            if os.path.isdir(old):
                shutil.rmtree(old, ignore_errors=True)
            if os.path.isfile(path):
                os.remove(path)
            elif os.path.isdir(path):
                os.rename(path, old)
            os.rename(tmpdir, path)
            shutil.rmtree(old, ignore_errors=True)
        dist.barrier()

    def load(self, name: Optional[str] = None, allow_missing: bool = False):
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import set_state_dict

        assert self.checkpoint_dir, "Checkpoint directory must be specified"
        path = os.path.join(self.checkpoint_dir, name or self.DEFAULT_NAME)
        if not os.path.isdir(path) and os.path.isdir(path + self.OLD_SUFFIX):
            # a writer died between the two renames of save(): the previous checkpoint is intact
            path = path + self.OLD_SUFFIX
            print0(f"Checkpoint swap was interrupted; falling back to {path}")
        if not os.path.isdir(path):
            if allow_missing:
                print0(f"Checkpoint {path} does not exist, skipping load")
                return
            raise FileNotFoundError(f"Checkpoint {path} does not exist")
        print0(f"Loading checkpoint from {path}")
        state = self._state()
        dcp.load(state, checkpoint_id=path)
        set_state_dict(self.model, self.optimizer, model_state_dict=state["model"],
                       optim_state_dict=state["optimizer"])
        self.train_loader.load_state_dict(state["train_loader"])
        self.val_loader.load_state_dict(state["val_loader"])
        self.step = state["step"]
        self.wandb_id = state["wandb_id"]
        dist.barrier()


class TrainStep:
    """One optimizer step: ``grad_accum`` micro-batches of forward + backward, then
    ``optimizer.step()``, the scheduler and ``zero_grad``.  Returns the last micro-batch's
    loss (a device tensor; reading it is the caller's synchronisation point)."""

    def __init__(self, model, raw_model, optimizer, lr_scheduler=None, grad_accum: int = 1,
                 optimizer_owns_grad_sync: bool = False, fast_fsdp: bool = False, timers: Optional[PhaseTimers] = None,
                 track_grad_norm: bool = False):
        from torch.distributed.fsdp import FSDPModule
        from torch.nn.parallel import DistributedDataParallel as DDP

        self.model, self.raw_model, self.optimizer, self.lr_scheduler = model, raw_model, optimizer, lr_scheduler
        self.grad_accum = grad_accum
        self.is_ddp = isinstance(model, DDP)
        self.is_fsdp = isinstance(model, FSDPModule)
        self.optimizer_owns_grad_sync = optimizer_owns_grad_sync
        self.fast_fsdp = fast_fsdp
        self.timers = timers or PhaseTimers(enabled=False)
        # total gradient norm of the step (train.py:913-916), a device tensor; only when asked for
        self.track_grad_norm = track_grad_norm
        self.last_grad_norm: Optional[torch.Tensor] = None

    def __call__(self, batches) -> torch.Tensor:
        """`batches`: iterable of ``grad_accum`` (x, y) pairs."""
        model = self.model
        model.train()
        loss_out = None
        t = self.timers
        t.start("fwd_bwd")
        for i, (x, y) in enumerate(batches, start=1):
            last = i == self.grad_accum
            loss = model(x, y)
            loss_out = loss.detach()
            if self.grad_accum > 1:
                loss = loss / self.grad_accum
            if self.is_ddp and (not last or self.optimizer_owns_grad_sync):
                with model.no_sync():
                    loss.backward()
            else:
                if self.is_fsdp:
                    model.set_is_last_backward(last)
                    if self.fast_fsdp:
                        model.set_reshard_after_backward(last)
                        model.set_requires_gradient_sync(last)
                    else:
                        model.set_requires_gradient_sync(True)
                loss.backward()
        t.stop("fwd_bwd")
        t.start("optimizer")
        if self.track_grad_norm:
            self.last_grad_norm = torch.nn.utils.get_total_norm(
                [p.grad for p in self.model.parameters() if p.grad is not None])
        self.optimizer.step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.model.zero_grad(set_to_none=True)
        t.stop("optimizer")
        return loss_out


def build_model(hp: Hyperparameters, device_mesh, replicate_mesh_grad_sync: bool, fast_fsdp: bool = False,
                device: Optional[torch.device] = None, vocab_size: int = 50304, sequence_parallel: bool = False):
    """Create the GPT on the meta device, shard it, materialise and initialise it; wrap in DDP
    when there is no mesh but several ranks.  Returns (model, raw_model)."""
    from torch.nn.parallel import DistributedDataParallel as DDP

    cfg = GPTConfig(sequence_len=hp.sequence_length, vocab_size=vocab_size, n_layer=hp.n_layer, n_head=hp.n_head,
                    n_embd=hp.model_dim)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    with torch.device("meta"):
        model = GPT(cfg)
    if device_mesh is not None:
        parallelize_gpt_model(model, device_mesh=device_mesh, dp_name=(None if replicate_mesh_grad_sync else "dp"),
                              fs_name="fs", tp_name="tp", fsdp_reshard_after_forward=not fast_fsdp,
                              sequence_parallel=sequence_parallel)
    model.to_empty(device=device)
    model.init_weights()
    raw = model
    if device_mesh is None and dist.is_initialized() and dist.get_world_size() > 1:
        # gradients of fp32 parameters; buckets overlap the all-reduce with backward
        model = DDP(model, device_ids=[device.index] if device.type == "cuda" else None,
                    gradient_as_bucket_view=True, bucket_cap_mb=64)
        raw = model.module
    for i, p in enumerate(model.parameters()):
        if not p.is_contiguous():
            raise ValueError(f"Parameter {i} is not contiguous")
    return model, raw


def main(argv=None):
    cli = parse_cli_args(argv)
    hp = override_args_from_cli(Hyperparameters(), cli)
    if cli.inv_rank_fraction:
        hp.rank_fraction = 1.0 / cli.inv_rank_fraction
    if hp.checkpoint_freq > 0 and not hp.checkpoint_dir:
        raise ValueError("Must specify --checkpoint_dir to save checkpoints")

    mesh = init_distributed(cli.dp_size, cli.fs_size, cli.tp_size)
    print0("=" * 80)
    if mesh is not None:
        dp_mesh = mesh["dp", "fs"]._flatten()
        dp_world, dp_rank = dp_mesh.size(), dp_mesh.get_local_rank()
    else:
        dp_world, dp_rank = dist.get_world_size(), dist.get_rank()

    if cli.debug:
        hp.batch_size = 2 * dp_world
        hp.device_batch_size = 1
    tokens_per_global_batch = hp.device_batch_size * hp.sequence_length * dp_world
    assert hp.val_tokens % tokens_per_global_batch == 0, "Invalid val_tokens"
    val_steps = hp.val_tokens // tokens_per_global_batch
    if cli.debug:
        hp.num_iterations = 20
        val_steps = min(val_steps, 2)
    seqs_per_global_micro = hp.device_batch_size * dp_world
    assert hp.batch_size % seqs_per_global_micro == 0, "Invalid batch_size"
    grad_accum = hp.batch_size // seqs_per_global_micro
    assert grad_accum >= 1, "Invalid grad_accum_steps"
    print0(f"Global batch size: {hp.batch_size} sequences; per-device: {hp.device_batch_size}; "
           f"sequence length: {hp.sequence_length}; gradient accumulation steps: {grad_accum}")

    train_loader = DistributedDataLoader(os.path.join(hp.data_dir, "fineweb_train_*.bin"), hp.device_batch_size,
                                         hp.sequence_length, dp_rank, dp_world)
    val_loader = DistributedDataLoader(os.path.join(hp.data_dir, "fineweb_val_*.bin"), hp.device_batch_size,
                                       hp.sequence_length, dp_rank, dp_world, prefetch=False)
    print0(f"Training DataLoader: {len(train_loader.files)} files; validation DataLoader: {len(val_loader.files)} files")

    model, raw_model = build_model(hp, mesh, hp.replicate_mesh_grad_sync, fast_fsdp=cli.fast_fsdp,
                                   sequence_parallel=cli.sequence_parallel)
    print0(f"Total parameters: {sum(p.numel() for p in model.parameters())}")
    print0(model)
    print0("=" * 80)

    from torch.nn.parallel import DistributedDataParallel as DDP

    replicate_group = model.process_group if isinstance(model, DDP) else (
        dist.group.WORLD if mesh is None and dist.get_world_size() > 1 else None)
    print0(f"Optimizer: {hp.optimizer}; scalar optimizer: {hp.scalar_opt}; base learning rate: {hp.lr}")
    optimizer = init_optimizer(raw_model, mesh, replicate_group, hp, cli)
    scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda(hp))

    run_name = f"({hp.optimizer}+{hp.scalar_opt})"
    if "dion" in hp.optimizer:
        run_name += f"_sp={hp.rank_fraction}"
    if cli.dp_size is not None:
        run_name += f"_dp={cli.dp_size}_fs={cli.fs_size}_tp={cli.tp_size}_gradsync={cli.replicate_mesh_grad_sync}"
    if cli.wandb_job_name:
        run_name += f"_{cli.wandb_job_name}"

    ckpt = CheckpointManager(hp.checkpoint_dir, model, optimizer, train_loader, val_loader)
    print0(f"Run name: {run_name}; debug: {cli.debug}; checkpoint directory: {hp.checkpoint_dir}; "
           f"checkpoint frequency: {hp.checkpoint_freq if hp.checkpoint_freq > 0 else 'disabled'}")
    if hp.checkpoint_dir:
        ckpt.load(allow_missing=True)
        print0(f"Resuming from step {ckpt.step}" if ckpt.step is not None else
               "No previous checkpoint found, training model from scratch")
    else:
        print0("Training model from scratch")
    print0("=" * 80)

    use_wandb = not cli.no_wandb and not cli.debug
    wandb = None
    if use_wandb:
        try:
            import wandb  # type: ignore
        except ImportError:
            print0("wandb is not installed; continuing without it")
            use_wandb = False
    if use_wandb:
        if _MASTER:
            wandb.login(key=os.environ.get("WANDB_API_KEY"), host=os.environ.get("WANDB_HOST"), timeout=0)
            wandb.init(project=hp.wandb_project_name, name=run_name, config=hp.__dict__, id=ckpt.wandb_id,
                       resume="must" if ckpt.wandb_id else "never")
            ckpt.wandb_id = wandb.run.id
        box = [ckpt.wandb_id]
        dist.broadcast_object_list(box, src=0)
        ckpt.wandb_id = box[0]

    try:
        from tqdm import tqdm
    except ImportError:  # pragma: no cover
        tqdm = None

    step_fn = TrainStep(model, raw_model, optimizer, scheduler, grad_accum,
                        optimizer_owns_grad_sync=hp.replicate_mesh_grad_sync, fast_fsdp=cli.fast_fsdp,
                        track_grad_norm=use_wandb)
    device = next(raw_model.parameters()).device
    cuda = device.type == "cuda"
    sync = torch.cuda.synchronize if cuda else (lambda: None)

    training_time_ms = 0.0
    sync()
    t0 = time.time()
    start_step = 0 if ckpt.step is None else ckpt.step + 1
    pbar = tqdm(total=hp.num_iterations, desc="Training", disable=not _MASTER) if tqdm else None
    if pbar:
        pbar.update(start_step)
    # host-side liveness: a rank that leaves says so in the store, and nobody launches the next step
    # against it (DION_B200_HEARTBEAT=0 turns it off, any other number is the check interval in steps)
    hb_every = int(os.environ.get("DION_B200_HEARTBEAT", "10"))
    heartbeat = StepHeartbeat.from_default_group(check_every=hb_every) if hb_every > 0 else None
    try:
        for step in range(start_step, hp.num_iterations + 1):
            if step == 10:  # the first steps carry one-time set-up cost
                training_time_ms = 0.0
                sync()
                t0 = time.time()
            timed_steps = (step - 10) if step > 10 else float("nan")

            last_step = step == hp.num_iterations
            if last_step or (hp.val_loss_every > 0 and step % hp.val_loss_every == 0):
                sync()
                training_time_ms += 1000 * (time.time() - t0)
                model.eval()
                val_loader.reset()
                val_loss = torch.zeros((), device=device)
                with torch.no_grad():
                    for _ in range(val_steps):
                        xv, yv = val_loader.next_batch()
                        val_loss += model(xv, yv).float()
                dist.all_reduce(val_loss, op=dist.ReduceOp.SUM)
                val = val_loss.item() / val_steps / dist.get_world_size()
                print0(f"step:{step}/{hp.num_iterations} val_loss:{val:.4f} train_time:{training_time_ms:.0f}ms "
                       f"step_avg:{training_time_ms / timed_steps:.2f}ms")
                if _MASTER and use_wandb:
                    wandb.log({"val/loss": val, "step": step, "time/training_time_ms": training_time_ms})
                if pbar:
                    pbar.set_postfix(val_loss=f"{val:.4f}")
                sync()
                t0 = time.time()
            if last_step:
                break

            if heartbeat is not None:
                heartbeat.check(step)
            train_loss = step_fn(train_loader.next_batch() for _ in range(grad_accum))
            if heartbeat is not None:
                heartbeat.beat(step)
            approx_time = training_time_ms + 1000 * (time.time() - t0)
            if _MASTER and use_wandb:
                grads_norm = step_fn.last_grad_norm
                if hasattr(grads_norm, "full_tensor"):
                    grads_norm = grads_norm.full_tensor()
                wandb.log({"train/loss": train_loss.item(), "train/grad_norm": float(grads_norm), "step": step,
                           "time/training_time_ms": approx_time})
            if _MASTER and cli.debug:
                print0(f"Step {step}: train_loss={train_loss.item():.4f}")
            if pbar:
                pbar.update(1)
                pbar.set_postfix(train_loss=f"{train_loss.item():.4f}")
            if cuda:
                ops.check_status(device)

            if hp.checkpoint_freq > 0 and step % hp.checkpoint_freq == 0 and step > 0:
                sync()
                training_time_ms += 1000 * (time.time() - t0)  # checkpoints are not training time
                if hasattr(optimizer, "synchronize_for_checkpoint"):
                    optimizer.synchronize_for_checkpoint()
                ckpt.save(step=step)
                sync()
                t0 = time.time()
    except BaseException:
        if heartbeat is not None:
            heartbeat.leave()
        raise
    if heartbeat is not None:
        heartbeat.leave()

    if pbar:
        pbar.close()
    if cuda:
        print0(f"Peak memory consumption: {torch.cuda.max_memory_allocated() // 1024 // 1024} MiB")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
