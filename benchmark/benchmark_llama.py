"""Llama-3-8B-shaped decoder under FSDP2 with Dion (rank_fraction 0.125): step time and tokens/s.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29544 \
        benchmark/benchmark_llama.py [--layers 32] [--seq 4096] [--batch 1] [--steps 5] [--warmup 3]

32 layers, d_model 4096, 32 query / 8 kv heads, SwiGLU 14336, vocabulary 128256, sequence 4096, bf16
compute on fp32 sharded master weights, random initialisation, uniform-random tokens.  The block
matrices (4096 x 4096, 1024 x 4096, 14336 x 4096, 4096 x 14336) go to Dion over the FSDP mesh, the
norm gains, embedding and lm_head to AdamW.  The reference ships no Llama model; the same optimizer
call on a plain-PyTorch model of this shape is its counterpart.  `--tiny` shrinks every dimension so
that the script can be smoke-tested on CPUs (gloo).  One JSON line from rank 0; times are CUDA events
on the launching stream, max over ranks.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rank_fraction", type=float, default=0.125)
    ap.add_argument("--optimizer", choices=("dion", "muon"), default="dion")
    ap.add_argument("--tiny", action="store_true")
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

    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion, Muon, ops
    from dion_b200.models.llama import Llama, LlamaConfig, make_llama_param_groups, parallelize_llama_model

    if args.tiny:
        cfg = LlamaConfig(sequence_len=args.seq, vocab_size=512, n_layer=args.layers, n_head=4, n_kv_head=2, n_embd=64,
                          ffn_dim=192)
    else:
        cfg = LlamaConfig.llama3_8b(n_layer=args.layers, sequence_len=args.seq)
    torch.manual_seed(0)
    with torch.device("meta"):
        model = Llama(cfg)
    mesh = init_device_mesh("cuda" if cuda else "cpu", (world,), mesh_dim_names=("fs",))
    if world > 1:
        parallelize_llama_model(model, mesh["fs"])
    model.to_empty(device=dev)
    model.init_weights()
    groups = make_llama_param_groups(model, scalar_opt="adamw", lr=3e-4)
    if args.optimizer == "dion":
        opt = Dion(groups, outer_shard_mesh=mesh["fs"] if world > 1 else None, lr=0.01,
                   rank_fraction=args.rank_fraction, weight_decay=0.01)
    else:
        opt = Muon(groups, distributed_mesh=mesh["fs"] if world > 1 else None, lr=0.01, nesterov=True)

    gen = torch.Generator().manual_seed(1000 + rank)
    x = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=gen).to(dev)
    y = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), generator=gen).to(dev)

    def step():
        loss = model(x, y)
        loss.backward()
        t_opt = None
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            opt.step()
            e1.record()
            t_opt = (e0, e1)
        else:
            opt.step()
        model.zero_grad(set_to_none=True)
        return loss, t_opt

    for _ in range(args.warmup):
        loss, _ = step()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    t0 = time.time()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    opt_events = []
    for _ in range(args.steps):
        loss, ev = step()
        opt_events.append(ev)
    if cuda:
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        opt_ms = sum(e0.elapsed_time(e1) for e0, e1 in opt_events) / args.steps
        t = torch.tensor([ms, opt_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, opt_ms = t.tolist()
        ops.check_status()
        peak = torch.cuda.max_memory_allocated() // (1 << 20)
    else:
        ms, opt_ms, peak = 1000 * (time.time() - t0) / args.steps, float("nan"), 0
    if rank == 0:
        params = sum(p.numel() for p in model.parameters())
        print(json.dumps({"metric": "Llama-shaped decoder train tokens/sec", "value": args.batch * args.seq * world / ms * 1e3,
                          "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "optimizer_ms": opt_ms,
                          "loss": float(loss.item()), "peak_mem_mib": peak,
                          "config": {"layers": cfg.n_layer, "d_model": cfg.n_embd, "heads": cfg.n_head,
                                     "kv_heads": cfg.n_kv_head, "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size,
                                     "seq_len": args.seq, "batch_per_gpu": args.batch, "parameters": params,
                                     "optimizer": f"{args.optimizer} rank_fraction {args.rank_fraction} + adamw",
                                     "parallelism": f"fs{world}"}}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
