"""Optimizer step alone on GPT-160M-shaped parameters with random gradients, device-timed.

    python benchmark/benchmark_optimizer_step.py --optimizer dion                       # one GPU
    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \
        benchmark/benchmark_optimizer_step.py --optimizer dion --mode ddp [--rank_fraction 0.25 --compressed]
    torchrun ... benchmark/benchmark_optimizer_step.py --optimizer muon --mode fsdp

`--mode ddp`: replicated parameters, the optimizer owns the data-parallel gradient sync (full
gradients, or only the low-rank factors with `--compressed`).  `--mode fsdp`: parameters sharded by
FSDP2 over all ranks (Dion's outer mesh / Muon's distributed mesh).  `DION_B200_SYMM=0` moves every
reduction / exchange to the process group's own collectives, which gives the library baseline for
the same step.  One JSON line from rank 0; milliseconds are CUDA-event times, max over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizer", choices=("dion", "muon"), default="dion")
    ap.add_argument("--mode", choices=("single", "ddp", "fsdp"), default="single")
    ap.add_argument("--rank_fraction", type=float, default=1.0)
    ap.add_argument("--compressed", action="store_true", help="Dion syncs only the low-rank factors over dp")
    ap.add_argument("--fp32_states", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=8, help="the symmetric arenas reach their final size within the first three steps")
    ap.add_argument("--layers", type=int, default=12, help="fewer layers for a quick smoke run")
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")   # CPUs (gloo) only for smoke runs
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.mode != "single":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        if cuda:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    rank = dist.get_rank() if dist.is_initialized() else 0

    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import ops
    from dion_b200.training import Hyperparameters, init_optimizer

    hp = Hyperparameters(model_dim=768, n_layer=args.layers, n_head=12, optimizer=args.optimizer, rank_fraction=args.rank_fraction,
                         mixed_precision=not args.fp32_states, replicate_mesh_grad_sync=args.mode == "ddp" or args.compressed,
                         num_iterations=10 ** 6)
    mesh, group = None, None
    if args.mode == "fsdp":
        mesh = init_device_mesh("cuda" if cuda else "cpu", (1, world, 1), mesh_dim_names=("dp", "fs", "tp"))
    elif args.mode == "ddp" and world > 1:
        group = dist.group.WORLD
    torch.manual_seed(0)
    # no DDP wrapper: the optimizer is handed the replicate group and reduces the gradients itself
    from dion_b200.models import GPT, GPTConfig
    from dion_b200.models.gpt import parallelize_gpt_model

    with torch.device("meta"):
        model = GPT(GPTConfig(sequence_len=1024, vocab_size=50304, n_layer=args.layers, n_head=12, n_embd=768))
    if mesh is not None:
        parallelize_gpt_model(model, device_mesh=mesh, dp_name=None, fs_name="fs", tp_name="tp")
    model.to_empty(device=dev)
    model.init_weights()
    opt = init_optimizer(model, mesh, group, hp)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    import time
    grads = []
    for p in model.parameters():
        loc = p.to_local() if hasattr(p, "to_local") else p
        g = torch.randn(loc.shape, device=dev, generator=gen) * 0.01
        if hasattr(p, "to_local"):
            from torch.distributed.tensor import DTensor

            g = DTensor.from_local(g, p.device_mesh, p.placements, run_check=False)
        grads.append(g)

    def step():
        for p, g in zip(model.parameters(), grads):
            p.grad = g
        opt.step()

    for _ in range(args.warmup):
        step()
    if cuda:
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    n0 = ops.launch_count()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / args.steps], device=dev)
    else:
        t0 = time.time()
        for _ in range(args.steps):
            step()
        ms = torch.tensor([1000 * (time.time() - t0) / args.steps])
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ops.check_status()
    if rank == 0:
        print(json.dumps({"optimizer": args.optimizer, "mode": args.mode, "world": world, "rank_fraction": args.rank_fraction,
                          "compressed_sync": bool(args.compressed), "state_dtype": "fp32" if args.fp32_states else "bf16",
                          "symmetric_memory": os.environ.get("DION_B200_SYMM", "1") != "0",
                          "optimizer_step_ms": round(float(ms.item()), 3),
                          "kernel_launches_per_step": (ops.launch_count() - n0) // args.steps}), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
