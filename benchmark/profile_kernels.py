"""Small, self-contained cases of the hot kernels for profiling and roofline numbers.

    python benchmark/profile_kernels.py <case> [--iters N]

Every case allocates well under 4 GB, uses inputs larger than the 126 MB L2 (where the op
is bandwidth-bound), warms up, then times `iters` launches with CUDA events (L2 flushed in
between) and prints achieved FLOP/s or bytes/s next to the measured peaks of
MEASURED_PEAKS.json when that file is present.  Under `ncu --clock-control none -k regex:<kernel> -c 1`
the same command yields one capture of the named kernel (never profile without `--clock-control none`:
ncu would lock the GPU's clocks, and that setting outlasts the process).

`--ref` times cuBLAS (torch.matmul / torch.bmm) on the operands of gemm_fwd, gemm_dx, gemm_dw
and gemm_sym for comparison.

Cases: gemm_fwd, gemm_dx, gemm_dw, gemm_sym, gemm_tf32_mn, gram3x, gram3x_k, apply3x, gemm_scatter, chol, cross_entropy,
rope, rope_bwd, rmsnorm, lion, adamw, muon_pre, dion_accum, all_reduce (single rank loop-back over
symmetric memory).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from dion_b200 import ops
from dion_b200.ops import nn as K


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def case(name: str, ref: bool = False):
    from dion_b200.ops import _ext

    _ext.load(required=True)  # the raw torch.ops calls below need the library in the process
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    r = lambda *s, dt=bf: torch.randn(*s, device=dev, dtype=torch.float32).to(dt)
    if name == "gemm_fwd":        # Linear forward: [T, K] x [N, K]^T, both K-major
        T, N, Kd = 32768, 3072, 768
        x, w, y = r(T, Kd), r(N, Kd), torch.empty(T, N, device=dev, dtype=bf)
        if ref:
            return (lambda: torch.matmul(x, w.t(), out=y)), 2.0 * T * N * Kd, (T * Kd + N * Kd + T * N) * 2
        return (lambda: ops.gemm(x, w.t(), out=y)), 2.0 * T * N * Kd, (T * Kd + N * Kd + T * N) * 2
    if name == "gemm_dx":         # input gradient: [T, N] x [N, K], B is MN-major
        T, N, Kd = 32768, 3072, 768
        dy, w, dx = r(T, N), r(N, Kd), torch.empty(T, Kd, device=dev, dtype=bf)
        if ref:
            return (lambda: torch.matmul(dy, w, out=dx)), 2.0 * T * N * Kd, (T * N + N * Kd + T * Kd) * 2
        return (lambda: ops.gemm(dy, w, out=dx)), 2.0 * T * N * Kd, (T * N + N * Kd + T * Kd) * 2
    if name == "gemm_dw":         # weight gradient: [N, T] x [T, K], both MN-major, split-K atomics
        T, N, Kd = 65536, 768, 768
        dy, x, dw = r(T, N), r(T, Kd), torch.zeros(N, Kd, device=dev)
        if ref:
            dyb, dwb = dy.t(), torch.empty(N, Kd, device=dev, dtype=bf)
            return (lambda: torch.matmul(dyb, x, out=dwb)), 2.0 * T * N * Kd, (T * N + T * Kd) * 2
        return (lambda: ops.gemm(dy.t(), x, out=dw, accumulate=True, split_k=16)), 2.0 * T * N * Kd, (T * N + T * Kd) * 2
    if name == "gemm_sym":        # Newton-Schulz X X^T, upper-triangular tiles + mirror
        B, m, n = 24, 768, 3072
        x, a = r(B, m, n), torch.empty(B, m, m, device=dev, dtype=bf)
        if ref:
            return (lambda: torch.bmm(x, x.transpose(1, 2), out=a)), 2.0 * B * m * m * n, B * (m * n + m * m) * 2
        return (lambda: ops.gemm(x, x.transpose(1, 2), out=a, symmetric=True)), 2.0 * B * m * m * n, B * (m * n + m * m) * 2
    if name == "gemm_tf32_mn":    # Dion R = A^T P on fp32 state: A MN-major (32-byte-atom swizzle)
        B, a, b_, rr = 12, 3072, 768, 768
        A, P, R = r(B, a, b_, dt=f32), r(B, a, rr, dt=f32), torch.empty(B, b_, rr, device=dev)
        return (lambda: ops.gemm(A.transpose(1, 2), P, out=R)), 2.0 * B * a * b_ * rr, B * (a * b_ + a * rr + b_ * rr) * 4
    if name in ("gram3x", "gram3x_k", "apply3x"):
        # the 3xTF32 products of Dion's orthonormalisation, fp32 operands split inside the kernel:
        #   gram3x   P^T P (symmetric, both operands MN-major)     gram3x_k  X X^T (symmetric, K-major)
        #   apply3x  P Z^T (K-major operands)
        B, a, rr = 64, 768, 768
        P, Z = r(B, a, rr, dt=f32), r(B, rr, rr, dt=f32)
        G, X = torch.empty(B, rr, rr, device=dev), torch.empty(B, a, rr, device=dev)
        if name == "gram3x":
            fn = lambda: ops.gemm(P.transpose(1, 2), P, out=G, symmetric=True, split3=True)
            return fn, 3 * 2.0 * B * rr * rr * a / 2, B * (a * rr + rr * rr) * 4
        if name == "gram3x_k":
            fn = lambda: ops.gemm(P, P.transpose(1, 2), out=G, symmetric=True, split3=True)
            return fn, 3 * 2.0 * B * rr * rr * a / 2, B * (a * rr + rr * rr) * 4
        fn = lambda: ops.gemm(P, Z.transpose(1, 2), out=X, split3=True)
        return fn, 3 * 2.0 * B * a * rr * rr, B * (2 * a * rr + rr * rr) * 4
    if name == "gemm_scatter":    # last Newton-Schulz product with the scatter epilogue (8 row blocks)
        B, m, n, W = 24, 768, 3072, 8
        bm, x = r(B, m, m), r(B, m, n)
        out = torch.empty(B, W, m // W, n, device=dev, dtype=bf)
        ptrs = torch.tensor([[out[i, s].data_ptr() for s in range(W)] for i in range(B)], dtype=torch.int64,
                            device=dev).view(-1)
        st = ops.runtime.status_tensor(torch.device(dev, 0))
        fn = lambda: torch.ops.dion_b200.gemm_scatter(bm, x, x, out[0, 0], ptrs, 1, m // W, W, 1.0, 2.8, st)
        return fn, 2.0 * B * m * m * n, B * (m * m + 3 * m * n) * 2
    if name == "chol":            # all Dion Gram matrices of GPT-160M in one launch
        B, rr = int(os.environ.get("CHOL_BATCH", "72")), 768
        P = r(B, 1024, rr, dt=f32)
        G = P.transpose(1, 2) @ P
        Z, W_, info = torch.empty_like(G), torch.empty_like(G), torch.empty(B, dtype=torch.int32, device=dev)
        return (lambda: ops.chol_inverse(G, out=Z, work=W_, info=info)), B * (2.0 / 3.0) * rr ** 3, B * rr * rr * 4 * 3
    if name == "cross_entropy":
        T, V = 8192, 50304
        logits, tgt = r(T, V), torch.randint(0, V, (T,), device=dev)
        loss = torch.empty(T, device=dev)
        fn = lambda: torch.ops.dion_b200.cross_entropy_fwd_bwd(logits, tgt, loss, None, 1.0 / T, -1, True)
        return fn, 0.0, T * V * 2 * 2
    if name == "rope":
        T, H, Dh = 65536, 12, 64
        q, k = r(T, H * Dh), r(T, H * Dh)
        qo, ko = torch.empty_like(q), torch.empty_like(k)
        cos, sin = K.rotary_tables(1024, Dh, dev)
        fn = lambda: torch.ops.dion_b200.rope_qknorm_fwd(q, k, qo, ko, cos, sin, 1024, H, Dh, K.RMS_EPS)
        return fn, 0.0, T * H * Dh * 2 * 4
    if name == "rope_bwd":
        T, H, Dh = 65536, 12, 64
        q, k, gq, gk = r(T, H * Dh), r(T, H * Dh), r(T, H * Dh), r(T, H * Dh)
        dq, dk = torch.empty_like(q), torch.empty_like(k)
        cos, sin = K.rotary_tables(1024, Dh, dev)
        fn = lambda: torch.ops.dion_b200.rope_qknorm_bwd(gq, gk, q, k, dq, dk, cos, sin, 1024, H, Dh, K.RMS_EPS)
        return fn, 0.0, T * H * Dh * 2 * 6
    if name == "rmsnorm":
        T, D = 131072, 768
        x, y, rs = r(T, D), torch.empty(T, D, device=dev, dtype=bf), torch.empty(T, device=dev)
        return (lambda: torch.ops.dion_b200.rmsnorm_fwd(x, None, None, y, rs, K.RMS_EPS)), 0.0, T * D * 2 * 2
    if name in ("lion", "adamw", "muon_pre", "dion_accum"):
        shapes = [(50304, 768)] + [(768, 768)] * 24 + [(3072, 768)] * 6
        X = [r(*s, dt=f32) for s in shapes]
        G = [r(*s, dt=f32) for s in shapes]
        M = [torch.zeros_like(x) for x in X]
        n = sum(x.numel() for x in X)
        if name == "lion":
            return (lambda: ops.lion_update(X, G, M, lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.0)), 0.0, n * 4 * 5
        if name == "adamw":
            V = [torch.zeros_like(x) for x in X]
            fn = lambda: ops.adamw_update(X, G, M, V, lr=1e-3, beta1=0.9, beta2=0.95, weight_decay=0.0, step=3, epsilon=1e-8)
            return fn, 0.0, n * 4 * 7
        if name == "muon_pre":
            U = [torch.empty_like(x, dtype=bf) for x in X]
            return (lambda: ops.muon_momentum(G, M, mu=0.95, nesterov=True, U=U)), 0.0, n * (4 * 3 + 2)
        return (lambda: ops.dion_accumulate(G, M)), 0.0, n * 4 * 3
    if name == "all_reduce":      # symmetric-memory all-reduce kernel, one rank talking to itself
        import torch.distributed as dist

        from dion_b200.parallel import symm

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(dev, 0))
        n = 64 << 20
        arena = symm.SymmetricArena(dist.group.WORLD, n * 4 + 4096, torch.device(dev, 0))
        t = arena.alloc((n,), f32)
        t.normal_()
        off = arena.offset_of(t)
        return (lambda: arena.all_reduce(t, off, average=True)), 0.0, n * 4 * 2
    raise SystemExit(f"unknown case {name}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ref", action="store_true",
                    help="time the library routine (cuBLAS through torch.matmul) on the same operands instead; "
                         "GEMM cases only")
    a = ap.parse_args()
    fn, flops, nbytes = case(a.case, a.ref)
    ms = _time(fn, a.iters)
    hbm, tf, src = _peaks()
    line = {"case": a.case + (" (library)" if a.ref else ""), "ms": round(ms, 4)}
    if flops:
        line["tflops"] = round(flops / ms / 1e9, 1)
        line[f"frac_of_{src}_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    line["gbs"] = round(nbytes / ms / 1e6, 1)
    line[f"frac_of_{src}_hbm"] = round(nbytes / ms / 1e6 / hbm, 3)
    print(json.dumps(line))
    ops.check_status()


if __name__ == "__main__":
    main()
