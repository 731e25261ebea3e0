"""Headline benchmark: GPT-160M training throughput (tokens/s over all GPUs) with Dion.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Config (the reference's GPT-160M recipe, configs/dion_160m.yaml, with rank_fraction 1.0):
12 layers, d_model 768, 12 heads, MLP 3072, vocab 50304, sequence 1024, 64 sequences per
GPU per step, data parallel over N GPUs, bf16 compute, Dion + Lion for embedding/lm_head,
optimizer states in bf16 (``mixed_precision: true`` in that YAML), synthetic uniform-random
tokens, random-init weights.

Two numbers are measured after W warm-up steps, each over exactly K optimizer steps
bracketed by a barrier and a device synchronisation, max over ranks:
  * ``value``  - device time (CUDA events) with the token batches already resident on the GPU;
  * ``e2e``    - wall time through the public training API (``TrainStep`` fed by
                 ``DistributedDataLoader``): every step copies its batch from pinned host
                 memory and reads the loss back to the host.
``--impl reference`` runs the unmodified reference package installed under baseline/_ref
(its GPT, its Dion, its data loader, torch DDP, torch.compile) on the same config and
prints the same JSON line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(n_layer=12, model_dim=768, n_head=12, vocab_size=50304, sequence_length=1024)
DEVICE_BATCH = 64
HP = dict(lr=0.02, mu=0.95, weight_decay=0.01, rank_fraction=1.0, scalar_opt="lion")


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--optimizer", type=str, default="dion", choices=["dion", "muon"])
    p.add_argument("--fp32-states", action="store_true", help="keep optimizer states in fp32")
    p.add_argument("--device-batch", type=int, default=DEVICE_BATCH)
    p.add_argument("--layers", type=int, default=MODEL["n_layer"], help="for smoke runs only")
    p.add_argument("--no-e2e", action="store_true")
    return p.parse_args()


def init_dist(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} processes")
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1 or args.impl == "reference":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("LOCAL_RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def barrier_sync():
    import torch
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_data(args, rank, world, steps_needed):
    """Synthetic shards in the FineWeb format, written once by rank 0."""
    import torch.distributed as dist

    from dion_b200.models.data import write_synthetic_shards

    tokens_per_step = args.device_batch * MODEL["sequence_length"] * world
    box = [None]
    if rank == 0:
        d = tempfile.mkdtemp(prefix="dion_b200_bench_")
        write_synthetic_shards(d, MODEL["vocab_size"], train_tokens=tokens_per_step * (steps_needed + 2) + 1,
                               val_tokens=tokens_per_step + 1, seed=1234)
        box[0] = d
    if dist.is_initialized():
        dist.broadcast_object_list(box, src=0)
    return box[0]


def emit(args, world, tokens_per_step, dev_ms, e2e_ms, clocks, extra):
    value = tokens_per_step * 1000.0 / dev_ms
    line = {
        "metric": "GPT-160M train tokens/sec",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dev_ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init weights",
        "impl": args.impl,
        "config": {
            "model": "GPT-160M (12 layers, d_model 768, 12 heads, MLP 3072, vocab 50304)" if args.layers == 12
            else f"GPT {args.layers} layers (smoke)",
            "global_batch": args.device_batch * world,
            "seq_len": MODEL["sequence_length"],
            "parallelism": f"dp{world}",
            "optimizer": f"{args.optimizer} rank_fraction 1.0 + lion" if args.optimizer == "dion" else "muon + lion",
            "optimizer_state_dtype": "fp32" if args.fp32_states else "bf16",
            "l2": "inputs_exceed_l2 (activations and weights per step are far larger than the 126 MB L2)",
        },
        # how the arm computes attention is a property of the implementation, not of the workload: it stays out
        # of `config`, which is the same dictionary in both arms
        "attention_impl": ("reference: F.scaled_dot_product_attention" if args.impl == "reference" else
                           ("library (F.scaled_dot_product_attention)"
                            if os.environ.get("DION_B200_ATTENTION", "kernel") == "library"
                            else "in-tree tcgen05 kernels")),
        "clocks": clocks,
    }
    if e2e_ms is not None:
        line["e2e"] = {
            "value": tokens_per_step * 1000.0 / e2e_ms,
            "unit": "tokens/s",
            "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": extra.get("h2d_bytes_per_step"),
            "d2h_bytes_per_step": extra.get("d2h_bytes_per_step"),
        }
    for k in ("gpu_launches", "optimizer_ms", "fwd_bwd_ms", "peak_mem_mib", "reference_mode", "reference_modes_ms",
              "comm_paths"):
        if k in extra:
            line[k] = extra[k]
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- ours

def run_ours(args):
    import torch
    import torch.distributed as dist

    rank, local, world = init_dist(args)
    from dion_b200 import ops
    from dion_b200.models.data import DistributedDataLoader
    from dion_b200.training import Hyperparameters, TrainStep, build_model, init_optimizer
    from dion_b200.utils.clocks import ClockSampler
    from dion_b200.utils.timers import PhaseTimers

    torch.manual_seed(1234)
    hp = Hyperparameters(model_dim=MODEL["model_dim"], n_layer=args.layers, n_head=MODEL["n_head"],
                         sequence_length=MODEL["sequence_length"], device_batch_size=args.device_batch,
                         batch_size=args.device_batch * world, optimizer=args.optimizer, scalar_opt=HP["scalar_opt"],
                         lr=HP["lr"], mu=HP["mu"], weight_decay=HP["weight_decay"], rank_fraction=HP["rank_fraction"],
                         mixed_precision=not args.fp32_states, replicate_mesh_grad_sync=False, num_iterations=10 ** 6)
    model, raw = build_model(hp, None, False, vocab_size=MODEL["vocab_size"])
    from torch.nn.parallel import DistributedDataParallel as DDP

    group = model.process_group if isinstance(model, DDP) else None
    opt = init_optimizer(raw, None, group, hp)
    timers = PhaseTimers(enabled=True)
    step_fn = TrainStep(model, raw, opt, None, 1, optimizer_owns_grad_sync=False, timers=timers)

    tokens_per_step = args.device_batch * MODEL["sequence_length"] * world
    total_steps = args.warmup + 2 * args.steps + 2
    data_dir = make_data(args, rank, world, total_steps)
    loader = DistributedDataLoader(os.path.join(data_dir, "fineweb_train_*.bin"), args.device_batch,
                                   MODEL["sequence_length"], rank, world)

    # ---- warm-up (through the loader, like real training)
    for _ in range(args.warmup):
        loss = step_fn([loader.next_batch()])
    float(loss.item())
    ops.check_status()

    # ---- device-timed region: batches already on the GPU
    staged = [loader.next_batch() for _ in range(args.steps)]
    staged = [(x.clone(), y.clone()) for x, y in staged]
    timers.reset()
    from dion_b200.optim import orthogonalize
    from dion_b200.parallel import symm

    symm.reset_stats()
    launches0 = ops.launch_count()
    sampler = ClockSampler(gpu_index=local)
    barrier_sync()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    marks = []
    for x, y in staged:
        loss = step_fn([(x, y)])
        if os.environ.get("DION_BENCH_TRACE"):
            m = torch.cuda.Event(enable_timing=True)
            m.record()
            marks.append(m)
    ev1.record()
    barrier_sync()
    clocks = sampler.stop()
    if marks and rank == 0:
        prev, per_step = ev0, []
        for m in marks:
            per_step.append(round(prev.elapsed_time(m), 2))
            prev = m
        print(f"[bench] per-step device ms: {per_step}", file=sys.stderr, flush=True)
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    launches = (ops.launch_count() - launches0) // max(args.steps, 1)
    phases = timers.max_over_ranks()
    ops.check_status()
    # which implementation carried each kind of collective in the device-timed region (per step), and
    # whether the all-gather kernel for the orthonormal factors passed its first-use comparison
    comm_paths = {k: v // max(args.steps, 1) for k, v in sorted(symm.stats.items())}
    comm_paths["gradient_all_reduce"] = "torch DDP buckets (NCCL), overlapped with backward" if world > 1 else "none (one GPU)"
    gatherers = list(orthogonalize._gatherers.values())
    if gatherers:
        comm_paths["factor_all_gather"] = ("in-tree kernel (first-use comparison passed)"
                                           if all(g.fn is not None and g.checked for g in gatherers)
                                           else "process group (kernel unavailable or failed its first-use comparison)")

    # ---- end-to-end region: pinned-host batches through the loader, loss read every step
    e2e_ms = None
    if not args.no_e2e:
        barrier_sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            loss = step_fn([loader.next_batch()])
            float(loss.item())
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0 / args.steps)
    extra = {
        "gpu_launches": int(launches),
        "optimizer_ms": phases.get("optimizer"),
        "fwd_bwd_ms": phases.get("fwd_bwd"),
        "h2d_bytes_per_step": loader.h2d_bytes_per_batch,
        "d2h_bytes_per_step": 4,
        "peak_mem_mib": torch.cuda.max_memory_allocated() // (1 << 20),
        "comm_paths": comm_paths,
    }
    if rank == 0:
        emit(args, world, tokens_per_step, dev_ms, e2e_ms, clocks, extra)
    if dist.is_initialized():
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------- reference

def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dion")) or not os.path.isdir(os.path.join(ref_dir, "models")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    # Inductor compiles small host-side C++ kernels with OpenMP; the first g++ on PATH of
    # some images lacks libgomp.spec, the distribution compiler has it.
    from dion_b200.utils.compilers import ensure_openmp_cxx

    ensure_openmp_cxx()
    import torch
    import torch.distributed as dist

    rank, local, world = init_dist(args)
    sys.path.insert(0, ref_dir)
    for name in [m for m in sys.modules if m == "dion" or m.startswith("dion.")]:
        del sys.modules[name]
    try:
        from dion import Dion as RefDion, DionMixedPrecisionConfig as RefMP, Muon as RefMuon
        from models.gpt_model import GPT as RefGPT, GPTConfig as RefCfg
        from models.gpt_utils import DistributedDataLoader as RefLoader
    except Exception as e:  # pragma: no cover
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}))
        return
    import math

    from torch.nn.parallel import DistributedDataParallel as DDP

    from dion_b200.utils.clocks import ClockSampler

    torch._dynamo.config.cache_size_limit = 100  # as the reference's trainer does (train.py:583)
    if hasattr(torch._dynamo.config, "recompile_limit"):
        torch._dynamo.config.recompile_limit = 100
    autocast = torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16)

    def build(compiled: bool):
        """Model, optimizers and step functions exactly as the reference trainer sets them up
        (train.py:674-737, 886-921); `compiled=False` is its --no_compile mode with dynamo off.
        Returns {mode name: step function}.  For Dion the reference has two ways of synchronising
        gradients over the data-parallel replicas, both a matter of one constructor argument / YAML key:
        `replicate_mesh_grad_sync: true` (its Dion YAMLs; the optimizer all-reduces after a backward
        pass under DDP.no_sync) and `false` (DDP's bucketed all-reduce overlapped with the backward pass).
        Both are built on the same model - one optimizer object each - and the faster one is reported."""
        torch.manual_seed(1234)
        cfg = RefCfg(sequence_len=MODEL["sequence_length"], vocab_size=MODEL["vocab_size"], n_layer=args.layers,
                     n_head=MODEL["n_head"], n_embd=MODEL["model_dim"])
        with torch.device("meta"):
            raw = RefGPT(cfg)
        raw.to_empty(device="cuda")
        raw.init_weights()
        if compiled:
            raw.compile()
        model = DDP(raw, device_ids=[local])
        groups = [
            dict(params=list(raw.transformer.h.parameters())),
            dict(params=list(raw.transformer.wte.parameters()), algorithm=HP["scalar_opt"], lr=HP["lr"],
                 betas=(0.95, 0.98), weight_decay=0),
            dict(params=list(raw.lm_head.parameters()), algorithm=HP["scalar_opt"],
                 lr=HP["lr"] / math.sqrt(MODEL["model_dim"]), betas=(0.95, 0.98), weight_decay=0),
        ]
        def make_step(opt, sync_in_opt):
            def step(x, y):
                model.train()
                with autocast:
                    loss = model(x, y)
                out = loss.detach()
                if sync_in_opt:
                    with model.no_sync():
                        loss.backward()
                else:
                    loss.backward()
                opt.step()
                model.zero_grad(set_to_none=True)
                return out

            return step

        def copy_groups():
            return [dict(g, params=list(g["params"])) for g in groups]

        if args.optimizer == "dion":
            mp = None if args.fp32_states else RefMP(momentum_dtype=torch.bfloat16, variance_dtype=torch.bfloat16,
                                                     Q_dtype=torch.bfloat16)
            steps = {}
            for name, sync_in_opt in (("replicate_mesh_grad_sync=True under DDP.no_sync", True),
                                      ("replicate_mesh_grad_sync=False, DDP gradient all-reduce", False)):
                if world == 1 and not sync_in_opt:
                    continue  # one GPU: there is nothing to synchronise, the two modes are the same program
                opt = RefDion(copy_groups(), replicate_mesh=model.process_group, replicate_mesh_grad_sync=sync_in_opt,
                              rank_fraction=HP["rank_fraction"], lr=HP["lr"], mu=HP["mu"],
                              weight_decay=HP["weight_decay"], mixed_precision_config=mp)
                steps[name] = make_step(opt, sync_in_opt)
            return steps
        opt = RefMuon(groups, distributed_mesh=model.process_group, lr=HP["lr"], mu=HP["mu"],
                      weight_decay=HP["weight_decay"], nesterov=True, adjust_lr="spectral_norm",
                      use_triton=compiled)
        return {"DDP gradient all-reduce": make_step(opt, False)}

    tokens_per_step = args.device_batch * MODEL["sequence_length"] * world
    total_steps = 2 * args.warmup + 2 * args.steps + 10
    data_dir = make_data(args, rank, world, total_steps)
    loader = RefLoader(os.path.join(data_dir, "fineweb_train_*.bin"), args.device_batch, MODEL["sequence_length"],
                       rank, world)
    mode = "torch.compile (reference default)"
    steps = build(compiled=True)
    first = loader.next_batch()
    try:
        for fn in steps.values():
            loss = fn(*first)
            float(loss.item())
    except Exception as e:  # the compiler stack is unusable on this machine: run the reference eagerly
        msg = f"{type(e).__name__}: {str(e).splitlines()[-1] if str(e) else ''}"[:200]
        import traceback

        print(f"[bench] torch.compile path failed ({msg}); running the reference with --no_compile semantics",
              file=sys.stderr, flush=True)
        print("".join(traceback.format_exception(e))[-6000:], file=sys.stderr, flush=True)
        torch._dynamo.reset()
        torch._dynamo.config.disable = True
        mode = f"eager, dynamo disabled (torch.compile failed here: {msg})"
        steps = build(compiled=False)
        for fn in steps.values():
            loss = fn(*first)
    # every mode gets the full warm-up, then a short device-timed trial; the fastest mode is the one measured
    trial_ms = {}
    for name, fn in steps.items():
        for _ in range(max(args.warmup - 1, 0)):
            loss = fn(*loader.next_batch())
        float(loss.item())
        if len(steps) > 1:
            trial = [loader.next_batch() for _ in range(3)]
            barrier_sync()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for x, y in trial:
                loss = fn(x, y)
            t1.record()
            barrier_sync()
            trial_ms[name] = round(max_over_ranks(t0.elapsed_time(t1) / len(trial)), 2)
    best = min(trial_ms, key=trial_ms.get) if trial_ms else next(iter(steps))
    step = steps[best]
    mode = f"{mode}; gradient sync: {best}"
    staged = [loader.next_batch() for _ in range(args.steps)]
    sampler = ClockSampler(gpu_index=local)
    barrier_sync()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for x, y in staged:
        loss = step(x, y)
    ev1.record()
    barrier_sync()
    clocks = sampler.stop()
    dev_ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    e2e_ms = None
    if not args.no_e2e:
        barrier_sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            loss = step(*loader.next_batch())
            float(loss.item())
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0 / args.steps)
    extra = {"h2d_bytes_per_step": 2 * args.device_batch * MODEL["sequence_length"] * 8, "d2h_bytes_per_step": 4,
             "peak_mem_mib": torch.cuda.max_memory_allocated() // (1 << 20), "reference_mode": mode}
    if trial_ms:
        extra["reference_modes_ms"] = trial_ms
    if rank == 0:
        emit(args, world, tokens_per_step, dev_ms, e2e_ms, clocks, extra)
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
