"""In-tree collectives against the process group's own (NCCL), device-timed, max over ranks.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        benchmark/benchmark_collectives.py [--iters 20]

Cases: the symmetric-memory all-reduce kernel, the all-gather and reduce-scatter kernels behind the
FSDP2 hooks, and the tensor-parallel row-parallel product (GEMM with peer-store scatter epilogue +
reduce + all-gather kernel) against GEMM + all-reduce.  Every line gives the time of both variants
and, for the in-tree one, the fraction of the NVLink roofline: bytes that have to leave each GPU
divided by the measured peer-copy bandwidth of 770 GB/s per direction (for the fused product the
roofline is the slower of that and the GEMM at the measured bf16 peak).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peak_tflops() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0))
    return 1590.0


def timed(fn, iters: int) -> float:
    """Milliseconds per call: events on the current stream, barrier on both sides, max over ranks."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD

    from dion_b200 import ops
    from dion_b200.parallel import symm
    from dion_b200.parallel import tp as TP
    from dion_b200.parallel.fsdp_comm import SymmAllGather, SymmReduceScatter

    def report(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    # ---- all-reduce (fp32, in place), the optimizer's reduction of P / R / Gram matrices
    for mb in (1, 16, 256):
        n = mb * (1 << 20) // 4
        symm.begin_step([g], dev)
        t = symm.empty(g, (n,), torch.float32, dev)
        if symm.arena_for(g) is None or symm.arena_for(g).offset_of(t) is None:
            symm.begin_step([g], dev)          # the arena grows at the next step boundary
            t = symm.empty(g, (n,), torch.float32, dev)
        t.normal_()
        u = torch.randn(n, device=dev)
        ms_k = timed(lambda: symm.all_reduce(t, g, average=True), args.iters)
        ms_l = timed(lambda: dist.all_reduce(u, op=dist.ReduceOp.AVG, group=g), args.iters)
        out_bytes = 2 * n * 4 * (world - 1) / world  # reduce-scatter + all-gather halves, per GPU and direction
        report(case="all_reduce", mbytes=mb, world=world, kernel_ms=round(ms_k, 4), nccl_ms=round(ms_l, 4),
               kernel_busbw_gbs=round(out_bytes / ms_k / 1e6, 1), nvlink_roofline_frac=round(out_bytes / ms_k / 1e6 / NVLINK_GBS, 3))

    # ---- all-gather / reduce-scatter of one GPT-160M block (7.08 M parameters) and of a 64 MB shard set
    ag, rs = SymmAllGather(g, dev), SymmReduceScatter(g, dev)
    for numel in (7077888, 32 << 20):
        per = numel // world // 8 * 8
        out = ag.allocate((per * world,), dtype=torch.bfloat16, device=dev)
        inp = out.narrow(0, rank * per, per)
        inp.normal_()
        ms_k = timed(lambda: ag(out, inp, g), args.iters)
        ms_l = timed(lambda: dist.all_gather_into_tensor(out, inp, group=g), args.iters)
        nbytes = per * 2 * (world - 1)           # received by each GPU
        report(case="all_gather_bf16", params=per * world, world=world, kernel_ms=round(ms_k, 4), nccl_ms=round(ms_l, 4),
               kernel_gbs_in=round(nbytes / ms_k / 1e6, 1), nvlink_roofline_frac=round(nbytes / ms_k / 1e6 / NVLINK_GBS, 3))
        rin = rs.allocate((per * world,), dtype=torch.float32, device=dev)
        rin.normal_()
        rout = rs.allocate((per,), dtype=torch.float32, device=dev)
        lin, lout = torch.randn(per * world, device=dev), torch.empty(per, device=dev)
        ms_k = timed(lambda: rs(rout, rin, g, dist.ReduceOp.AVG), args.iters)
        ms_l = timed(lambda: dist.reduce_scatter_tensor(lout, lin, op=dist.ReduceOp.AVG, group=g), args.iters)
        nbytes = per * 4 * (world - 1)
        report(case="reduce_scatter_fp32", params=per * world, world=world, kernel_ms=round(ms_k, 4),
               nccl_ms=round(ms_l, 4), kernel_gbs_in=round(nbytes / ms_k / 1e6, 1),
               nvlink_roofline_frac=round(nbytes / ms_k / 1e6 / NVLINK_GBS, 3))

    # ---- tensor-parallel row-parallel product: mlp.c_proj of GPT-160M, 32 x 1024 tokens
    T, K, N = 32768, 3072 // world, 768
    x = torch.randn(T, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)

    def unfused():
        y = ops.gemm(x, w.t())
        dist.all_reduce(y, group=g)
        return y

    ms_k = timed(lambda: TP._matmul_all_reduce(x, w.t(), g), args.iters)
    ms_l = timed(unfused, args.iters)
    ya, yb = TP._matmul_all_reduce(x, w.t(), g), unfused()
    err = ((ya.float() - yb.float()).abs().max() / yb.float().abs().max()).item()
    link_ms = 2 * T * N * 2 * (world - 1) / world / (NVLINK_GBS * 1e6)   # scatter out + gather in, bf16
    gemm_ms = 2.0 * T * K * N / (_peak_tflops() * 1e9)
    report(case="tp_row_parallel_product", T=T, K_local=K, N=N, world=world, fused_ms=round(ms_k, 4),
           gemm_plus_nccl_ms=round(ms_l, 4), roofline_ms=round(max(link_ms, gemm_ms), 4),
           roofline_frac=round(max(link_ms, gemm_ms) / ms_k, 3), max_rel_diff=round(err, 5))
    ops.check_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
