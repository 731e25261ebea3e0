"""GPT-160M training throughput on a ("dp", "fs", "tp") device mesh: the sharded configurations next to
the data-parallel headline of `bench.py`.

    # Muon under FSDP2 over 8 GPUs (shard exchange -> Newton-Schulz -> scatter)
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29566 \
        benchmark/benchmark_train_mesh.py --optimizer muon --dp 1 --fs 8 --tp 1
    # Dion rank_fraction 0.25 on dp 2 x fs 2 x tp 2, low-rank gradient sync over dp, bf16 momentum / fp32 Q
    torchrun ... benchmark/benchmark_train_mesh.py --optimizer dion --dp 2 --fs 2 --tp 2 --rank_fraction 0.25 \
        --compressed --momentum_dtype bf16 --q_dtype fp32 [--sequence_parallel]

12 layers, d_model 768, 12 heads, MLP 3072, vocabulary 50304, sequence 1024, 64 sequences per
data-parallel rank (tensor-parallel ranks share their batch), random initialisation, uniform-random
tokens.  W >= 3 warm-up steps, then K steps between barriers; CUDA events on the launching stream, max
over ranks; forward + backward and optimizer are timed separately with events as well.  One JSON line
from rank 0.  `--tiny` shrinks the model so that the script can be smoke-tested with gloo ranks on CPUs.

`--impl reference` runs the same configuration with the unmodified reference package installed under
baseline/_ref: its GPT, its `parallelize_gpt_model` (FSDP2 / TP plan), its `Dion` / `Muon`, bf16 autocast
and `torch.compile` as its trainer sets them up (train.py:300-473, 685-737, 886-921); if the compiler
stack is unusable on the machine it runs eagerly (its `--no_compile` mode) and says so.  The JSON line
then carries `"impl": "reference"`.  Both arms report, under `comm_paths`, how many collectives of the
timed region ran as in-tree kernels and how many through the process group (the reference: all of them).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

_DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32}


def make_batches(args, dims, rank, dev, total):
    """Token batches of the run: tensor-parallel ranks see the same tokens, data-parallel ranks
    (dp x fs) different ones; the same for both implementations."""
    dp_rank = rank // args.tp
    gen = torch.Generator().manual_seed(7 + dp_rank)
    xs = torch.randint(0, dims["vocab"], (total, args.device_batch, dims["seq"]), generator=gen)
    ys = torch.randint(0, dims["vocab"], (total, args.device_batch, dims["seq"]), generator=gen)
    return [(xs[i].to(dev), ys[i].to(dev)) for i in range(total)]


def run_reference(args, dims, mesh, dev, cuda, rank, world):
    """The reference's own model, parallelisation plan, optimizer and training step on this mesh."""
    import math

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dion")) or not os.path.isdir(os.path.join(ref_dir, "models")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        dist.destroy_process_group()
        return
    from dion_b200.utils.compilers import ensure_openmp_cxx

    ensure_openmp_cxx()  # Inductor's host code needs a compiler with OpenMP
    sys.path.insert(0, ref_dir)
    for name in [m for m in sys.modules if m == "dion" or m.startswith("dion.") or m == "models" or m.startswith("models.")]:
        del sys.modules[name]
    from dion import Dion as RefDion, DionMixedPrecisionConfig as RefMP, Muon as RefMuon
    from models.gpt_model import GPT as RefGPT, GPTConfig as RefCfg, parallelize_gpt_model as ref_parallelize

    torch._dynamo.config.cache_size_limit = 100  # as the reference's trainer does (train.py:583)
    if hasattr(torch._dynamo.config, "recompile_limit"):
        torch._dynamo.config.recompile_limit = 100
    autocast = torch.amp.autocast(device_type="cuda" if cuda else "cpu", dtype=torch.bfloat16)

    def build(compiled: bool):
        torch.manual_seed(1234)
        with torch.device("meta"):
            model = RefGPT(RefCfg(sequence_len=dims["seq"], vocab_size=dims["vocab"], n_layer=dims["n_layer"],
                                  n_head=dims["n_head"], n_embd=dims["model_dim"]))
        ref_parallelize(model, device_mesh=mesh, dp_name=None if args.compressed else "dp", fs_name="fs", tp_name="tp",
                        fsdp_reshard_after_forward=True)
        model.to_empty(device=dev)
        model.init_weights()
        if compiled:
            model.compile()
        groups = [
            dict(params=list(model.transformer.h.parameters())),
            dict(params=list(model.transformer.wte.parameters()), algorithm="lion", lr=0.02, betas=(0.95, 0.98),
                 weight_decay=0),
            dict(params=list(model.lm_head.parameters()), algorithm="lion", lr=0.02 / math.sqrt(dims["model_dim"]),
                 betas=(0.95, 0.98), weight_decay=0),
        ]
        if args.optimizer == "dion":
            opt = RefDion(groups, replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"],
                          inner_shard_mesh=mesh["tp"] if args.tp > 1 else None,
                          replicate_mesh_grad_sync=args.compressed, rank_fraction=args.rank_fraction, lr=0.02, mu=0.95,
                          weight_decay=0.01,
                          mixed_precision_config=RefMP(momentum_dtype=_DTYPES[args.momentum_dtype],
                                                       Q_dtype=_DTYPES[args.q_dtype]))
        else:
            assert args.tp == 1, "Muon does not support tensor parallelism"
            opt = RefMuon(groups, distributed_mesh=mesh["fs"] if args.fs > 1 else mesh["dp"], lr=0.02, mu=0.95,
                          weight_decay=0.01, nesterov=True, adjust_lr="spectral_norm", use_triton=compiled)

        def step(x, y):
            model.train()
            with autocast:
                loss = model(x, y)
            out = loss.detach()
            loss.backward()
            opt.step()
            model.zero_grad(set_to_none=True)
            return out

        return step

    total = args.warmup + args.steps
    batches = make_batches(args, dims, rank, dev, total)
    mode = "torch.compile + Triton Newton-Schulz (reference defaults)"
    step = build(compiled=True)
    try:
        loss = step(*batches[0])
        float(loss.item())
    except Exception as e:
        msg = f"{type(e).__name__}: {str(e).splitlines()[-1] if str(e) else ''}"[:200]
        if rank == 0:
            print(f"[mesh bench] torch.compile path failed ({msg}); running the reference eagerly", file=sys.stderr,
                  flush=True)
        torch._dynamo.reset()
        torch._dynamo.config.disable = True
        mode = f"eager, dynamo disabled (torch.compile failed here: {msg})"
        step = build(compiled=False)
        loss = step(*batches[0])
    for i in range(1, args.warmup):
        loss = step(*batches[i])
    float(loss.item())
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for i in range(args.warmup, total):
        loss = step(*batches[i])
    if cuda:
        e1.record()
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        peak = torch.cuda.max_memory_allocated() // (1 << 20)
    else:
        ms, peak = 1000.0 * (time.perf_counter() - t0) / args.steps, 0
    tokens = args.device_batch * dims["seq"] * args.dp * args.fs
    if rank == 0:
        print(json.dumps({
            "metric": "GPT-160M train tokens/sec", "value": tokens / ms * 1e3, "unit": "tokens/s", "n_gpus": world,
            "impl": "reference", "reference_mode": mode, "ms_per_step": ms, "loss": float(loss.item()),
            "peak_mem_mib": peak, "steps": args.steps, "warmup": args.warmup, "dtype": "bf16",
            "data": "synthetic uniform-random tokens, random-init weights",
            "comm_paths": "process group (NCCL) for every collective",
            "config": {"model": "tiny" if args.tiny else "GPT-160M (12 layers, d_model 768, 12 heads, MLP 3072, vocab 50304)",
                       "global_batch": args.device_batch * args.dp * args.fs, "seq_len": dims["seq"],
                       "parallelism": f"dp{args.dp} x fs{args.fs} x tp{args.tp}",
                       "optimizer": (f"dion rank_fraction {args.rank_fraction}, momentum {args.momentum_dtype}, "
                                     f"Q {args.q_dtype}, " + ("low-rank sync over dp" if args.compressed else "gradient sync by FSDP")
                                     if args.optimizer == "dion" else "muon nesterov, 5-step Newton-Schulz") + " + lion"}}),
              flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizer", choices=("dion", "muon"), default="dion")
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--fs", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--rank_fraction", type=float, default=0.25)
    ap.add_argument("--compressed", action="store_true",
                    help="Dion owns the gradient sync over dp (low-rank factors); FSDP shards over fs only")
    ap.add_argument("--momentum_dtype", choices=tuple(_DTYPES), default="bf16")
    ap.add_argument("--q_dtype", choices=tuple(_DTYPES), default="fp32")
    ap.add_argument("--sequence_parallel", action="store_true")
    ap.add_argument("--device_batch", type=int, default=64)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    args = ap.parse_args()

    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert args.dp * args.fs * args.tp == world, f"mesh {args.dp} x {args.fs} x {args.tp} needs {args.dp * args.fs * args.tp} ranks"

    from torch.distributed.device_mesh import init_device_mesh

    if args.tiny:
        dims = dict(model_dim=64, n_layer=2, n_head=4, seq=64, vocab=512)
    else:
        dims = dict(model_dim=768, n_layer=12, n_head=12, seq=1024, vocab=50304)
    mesh = init_device_mesh("cuda" if cuda else "cpu", (args.dp, args.fs, args.tp), mesh_dim_names=("dp", "fs", "tp"))
    torch.manual_seed(1234)
    if args.impl == "reference":
        run_reference(args, dims, mesh, dev, cuda, rank, world)
        return

    from dion_b200 import Dion, DionMixedPrecisionConfig, Muon, ops
    from dion_b200.models.gpt import GPT, GPTConfig, parallelize_gpt_model
    from dion_b200.parallel import fsdp_comm, symm
    from dion_b200.training import Hyperparameters, TrainStep, make_param_groups
    from dion_b200.utils.timers import PhaseTimers

    with torch.device("meta"):
        model = GPT(GPTConfig(sequence_len=dims["seq"], vocab_size=dims["vocab"], n_layer=dims["n_layer"],
                              n_head=dims["n_head"], n_embd=dims["model_dim"]))
    parallelize_gpt_model(model, mesh, dp_name=None if args.compressed else "dp", fs_name="fs", tp_name="tp",
                          sequence_parallel=args.sequence_parallel)
    model.to_empty(device=dev)
    model.init_weights()

    hp = Hyperparameters(model_dim=dims["model_dim"], n_layer=dims["n_layer"], n_head=dims["n_head"],
                         sequence_length=dims["seq"], lr=0.02, scalar_opt="lion")
    groups = make_param_groups(model, hp)
    if args.optimizer == "dion":
        opt = Dion(groups, replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"],
                   inner_shard_mesh=mesh["tp"] if args.tp > 1 else None, replicate_mesh_grad_sync=args.compressed,
                   rank_fraction=args.rank_fraction, lr=0.02, mu=0.95, weight_decay=0.01,
                   mixed_precision_config=DionMixedPrecisionConfig(momentum_dtype=_DTYPES[args.momentum_dtype],
                                                                   Q_dtype=_DTYPES[args.q_dtype]))
    else:
        assert args.tp == 1, "Muon does not support tensor parallelism"
        opt = Muon(groups, distributed_mesh=mesh["fs"] if args.fs > 1 else mesh["dp"], lr=0.02, mu=0.95,
                   weight_decay=0.01, nesterov=True, adjust_lr="spectral_norm")
    timers = PhaseTimers(enabled=True)
    step_fn = TrainStep(model, model, opt, None, 1, optimizer_owns_grad_sync=args.compressed, timers=timers)

    total = args.warmup + args.steps
    batches = make_batches(args, dims, rank, dev, total)

    def sync():
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()

    for i in range(args.warmup):
        loss = step_fn([batches[i]])
    float(loss.item())
    if cuda:
        ops.check_status()
    timers.reset()
    symm.reset_stats()
    fsdp0 = {k: (ag.kernel_calls, ag.fallback_calls, rs.kernel_calls, rs.fallback_calls)
             for k, (ag, rs) in fsdp_comm._installed.items()}
    sync()
    t0 = time.perf_counter()
    n0 = ops.launch_count() if cuda else 0
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for i in range(args.warmup, total):
        loss = step_fn([batches[i]])
    if cuda:
        e1.record()
    sync()
    launches = (ops.launch_count() - n0) // max(args.steps, 1) if cuda else 0
    if cuda:
        ms = e0.elapsed_time(e1) / args.steps
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        phases = timers.max_over_ranks()
        ops.check_status()
        peak = torch.cuda.max_memory_allocated() // (1 << 20)
    else:
        ms, phases, peak = 1000.0 * (time.perf_counter() - t0) / args.steps, {}, 0
    tokens = args.device_batch * dims["seq"] * args.dp * args.fs
    comm = dict(symm.stats)
    for k, (ag, rs) in fsdp_comm._installed.items():
        a0 = fsdp0.get(k, (0, 0, 0, 0))
        comm["fsdp_all_gather.kernel"] = comm.get("fsdp_all_gather.kernel", 0) + ag.kernel_calls - a0[0]
        comm["fsdp_all_gather.library"] = comm.get("fsdp_all_gather.library", 0) + ag.fallback_calls - a0[1]
        comm["fsdp_reduce_scatter.kernel"] = comm.get("fsdp_reduce_scatter.kernel", 0) + rs.kernel_calls - a0[2]
        comm["fsdp_reduce_scatter.library"] = comm.get("fsdp_reduce_scatter.library", 0) + rs.fallback_calls - a0[3]
    if rank == 0:
        print(json.dumps({
            "metric": "GPT-160M train tokens/sec", "value": tokens / ms * 1e3, "unit": "tokens/s", "n_gpus": world,
            "impl": "ours", "ms_per_step": ms, "fwd_bwd_ms": phases.get("fwd_bwd"), "optimizer_ms": phases.get("optimizer"),
            "comm_paths": {k: v for k, v in sorted(comm.items())}, "gpu_launches": None if not cuda else launches,
            "loss": float(loss.item()), "peak_mem_mib": peak, "steps": args.steps, "warmup": args.warmup,
            "dtype": "bf16" if cuda else "fp32", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": "tiny" if args.tiny else "GPT-160M (12 layers, d_model 768, 12 heads, MLP 3072, vocab 50304)",
                       "global_batch": args.device_batch * args.dp * args.fs, "seq_len": dims["seq"],
                       "parallelism": f"dp{args.dp} x fs{args.fs} x tp{args.tp}"
                                      + (" sequence-parallel" if args.sequence_parallel else ""),
                       "optimizer": (f"dion rank_fraction {args.rank_fraction}, momentum {args.momentum_dtype}, "
                                     f"Q {args.q_dtype}, " + ("low-rank sync over dp" if args.compressed else "gradient sync by FSDP")
                                     if args.optimizer == "dion" else "muon nesterov, 5-step Newton-Schulz") + " + lion"}}),
              flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
