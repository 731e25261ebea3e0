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

`--impl reference` is that counterpart: a plain-PyTorch decoder of the same shape (nn.Linear,
F.rms_norm, F.scaled_dot_product_attention, F.silu; bf16 autocast; FSDP2 with the same shard placements)
driven by the unmodified reference `Dion` / `Muon` from baseline/_ref.  None of this package's kernels,
models or optimizers are on that path.
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


def build_plain_llama(cfg, mesh, world, dev):
    """The same decoder in plain PyTorch, sharded like parallelize_llama_model does (long dimension)."""
    import torch.nn as nn
    import torch.nn.functional as F
    from torch.distributed.tensor import Shard

    hd = cfg.n_embd // cfg.n_head

    def rope_tables(T, device):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=device).float() / hd))
        fr = torch.outer(torch.arange(T, device=device).float(), inv)
        return fr.cos()[None, :, None, :], fr.sin()[None, :, None, :]

    def rope(x, cos, sin):
        d = x.shape[-1] // 2
        x1, x2 = x[..., :d].float(), x[..., d:].float()
        return torch.cat([x1 * cos + x2 * sin, x2 * cos - x1 * sin], dim=-1).to(x.dtype)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attention_norm = nn.RMSNorm(cfg.n_embd, eps=cfg.norm_eps)
            self.ffn_norm = nn.RMSNorm(cfg.n_embd, eps=cfg.norm_eps)
            self.wq = nn.Linear(cfg.n_embd, cfg.n_head * hd, bias=False)
            self.wk = nn.Linear(cfg.n_embd, cfg.n_kv_head * hd, bias=False)
            self.wv = nn.Linear(cfg.n_embd, cfg.n_kv_head * hd, bias=False)
            self.wo = nn.Linear(cfg.n_head * hd, cfg.n_embd, bias=False)
            self.w_gate = nn.Linear(cfg.n_embd, cfg.ffn_dim, bias=False)
            self.w_up = nn.Linear(cfg.n_embd, cfg.ffn_dim, bias=False)
            self.w_down = nn.Linear(cfg.ffn_dim, cfg.n_embd, bias=False)

        def forward(self, x, cos, sin):
            B, T, _ = x.shape
            h = self.attention_norm(x)
            q = rope(self.wq(h).view(B, T, cfg.n_head, hd), cos, sin)
            k = rope(self.wk(h).view(B, T, cfg.n_kv_head, hd), cos, sin)
            v = self.wv(h).view(B, T, cfg.n_kv_head, hd)
            y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=True)
            x = x + self.wo(y.transpose(1, 2).reshape(B, T, -1))
            h = self.ffn_norm(x)
            return x + self.w_down(F.silu(self.w_gate(h)) * self.w_up(h))

    class Plain(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.n_embd)
            self.layers = nn.ModuleList([Block() for _ in range(cfg.n_layer)])
            self.norm = nn.RMSNorm(cfg.n_embd, eps=cfg.norm_eps)
            self.output = nn.Linear(cfg.n_embd, cfg.vocab_size, bias=False)

        def forward(self, idx, targets):
            cos, sin = rope_tables(idx.shape[1], idx.device)
            x = self.tok_embeddings(idx)
            for layer in self.layers:
                x = layer(x, cos, sin)
            logits = self.output(self.norm(x)).float()
            return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1))

    with torch.device("meta"):
        model = Plain()
    if world > 1:
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for b in model.layers:
            shard = {b.w_gate.weight: Shard(0), b.w_up.weight: Shard(0), b.w_down.weight: Shard(1), b.wq.weight: Shard(1),
                     b.wk.weight: Shard(1), b.wv.weight: Shard(1), b.wo.weight: Shard(0)}
            fully_shard(b, mesh=mesh, mp_policy=mp, shard_placement_fn=lambda p, m=shard: m.get(p))
        top = {model.tok_embeddings.weight: Shard(1), model.output.weight: Shard(1)}
        fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=False, shard_placement_fn=lambda p, m=top: m.get(p))
    model.to_empty(device=dev)
    for m in model.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=1.0)
        elif isinstance(m, nn.RMSNorm):
            nn.init.ones_(m.weight)
    matrices = [p for b in model.layers for p in b.parameters() if p.ndim == 2]
    gains = [p for p in model.parameters() if p.ndim == 1]
    import math

    groups = [dict(params=matrices),
              dict(params=gains, algorithm="adamw", lr=3e-4, weight_decay=0),
              dict(params=list(model.tok_embeddings.parameters()), algorithm="adamw", lr=3e-4, weight_decay=0),
              dict(params=list(model.output.parameters()), algorithm="adamw", lr=3e-4 / math.sqrt(cfg.n_embd),
                   weight_decay=0)]
    return model, groups


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

    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion, Muon, ops
    from dion_b200.models.llama import Llama, LlamaConfig, make_llama_param_groups, parallelize_llama_model

    if args.tiny:
        cfg = LlamaConfig(sequence_len=args.seq, vocab_size=512, n_layer=args.layers, n_head=4, n_kv_head=2, n_embd=64,
                          ffn_dim=192)
    else:
        cfg = LlamaConfig.llama3_8b(n_layer=args.layers, sequence_len=args.seq)
    torch.manual_seed(0)
    mesh = init_device_mesh("cuda" if cuda else "cpu", (world,), mesh_dim_names=("fs",))
    reference = args.impl == "reference"
    if reference:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        ref_dir = os.path.join(root, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "dion")):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
            dist.destroy_process_group()
            return
        from dion_b200.utils.compilers import ensure_openmp_cxx

        ensure_openmp_cxx()  # Inductor's host code needs a compiler with OpenMP
        sys.path.insert(0, ref_dir)
        for name in [m for m in sys.modules if m == "dion" or m.startswith("dion.")]:
            del sys.modules[name]
        from dion import Dion as RefDion, Muon as RefMuon

        # the reference's trainer raises dynamo's cache limit because its compiled helpers recompile for
        # every new shape / hyper-parameter combination (train.py:583); a decoder with seven weight shapes needs it too
        torch._dynamo.config.cache_size_limit = 100
        if hasattr(torch._dynamo.config, "recompile_limit"):
            torch._dynamo.config.recompile_limit = 100

        model, groups = build_plain_llama(cfg, mesh["fs"], world, dev)
        if args.optimizer == "dion":
            opt = RefDion(groups, outer_shard_mesh=mesh["fs"] if world > 1 else None, lr=0.01,
                          rank_fraction=args.rank_fraction, weight_decay=0.01)
        else:
            opt = RefMuon(groups, distributed_mesh=mesh["fs"] if world > 1 else None, lr=0.01, nesterov=True)
        plain, autocast = model, torch.amp.autocast(device_type="cuda" if cuda else "cpu", dtype=torch.bfloat16)

        def model(x, y):  # noqa: F811 - the training step below calls model(x, y)
            with autocast:
                return plain(x, y)

        model.zero_grad = plain.zero_grad
        model.parameters = plain.parameters
    else:
        with torch.device("meta"):
            model = Llama(cfg)
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
        if not reference:
            ops.check_status()
        peak = torch.cuda.max_memory_allocated() // (1 << 20)
    else:
        ms, opt_ms, peak = 1000 * (time.time() - t0) / args.steps, float("nan"), 0
    if rank == 0:
        params = sum(p.numel() for p in model.parameters())
        print(json.dumps({"metric": "Llama-shaped decoder train tokens/sec", "value": args.batch * args.seq * world / ms * 1e3,
                          "unit": "tokens/s", "n_gpus": world, "impl": args.impl, "ms_per_step": ms, "optimizer_ms": opt_ms,
                          "loss": float(loss.item()), "peak_mem_mib": peak,
                          "config": {"layers": cfg.n_layer, "d_model": cfg.n_embd, "heads": cfg.n_head,
                                     "kv_heads": cfg.n_kv_head, "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size,
                                     "seq_len": args.seq, "batch_per_gpu": args.batch, "parameters": params,
                                     "optimizer": f"{args.optimizer} rank_fraction {args.rank_fraction} + adamw",
                                     "parallelism": f"fs{world}"}}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
