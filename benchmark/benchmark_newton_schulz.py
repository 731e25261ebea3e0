"""Newton-Schulz micro-benchmark: the tcgen05 implementation against the plain bf16-matmul
one (three library GEMMs per iteration), the comparison the reference makes for its Triton
kernels (benchmark/benchmark_newton_shultz.py:33-101, 173).

    python benchmark/benchmark_newton_schulz.py --single --m 4096 --n 14336
    python benchmark/benchmark_newton_schulz.py --grid            # 512 ... 8192, square
    python benchmark/benchmark_newton_schulz.py --batch_size 12 --m 768 --n 3072

FLOPs per iteration are counted as ``4 m^2 n + 2 m^3`` (m <= n), i.e. without crediting the
symmetric products, so both implementations are measured against the same amount of work.
Timing: CUDA events on the launching stream, after warm-up, L2 flushed between iterations.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from dion_b200.optim.newton_schulz import NS_COEFFS, newton_schulz, newton_schulz_torch
from dion_b200.utils.timers import cuda_time_ms


def ns_flops(m: int, n: int, batch: int = 1, iters: int = len(NS_COEFFS)) -> float:
    if m > n:
        m, n = n, m
    return float(batch) * iters * (4.0 * m * m * n + 2.0 * m ** 3)


def bench_one(m: int, n: int, batch: int, iters: int = 10):
    shape = (batch, m, n) if batch > 1 else (m, n)
    G = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
    ours = cuda_time_ms(lambda: newton_schulz(G), iters=iters, warmup=3, flush_l2=True)
    ref = cuda_time_ms(lambda: newton_schulz_torch(G), iters=iters, warmup=3, flush_l2=True)
    fl = ns_flops(m, n, batch)
    e = max(m, n) / min(m, n)
    err = (newton_schulz(G).float() - newton_schulz_torch(G).float()).abs().max().item()
    return {
        "m": m, "n": n, "batch": batch,
        "tcgen05_ms": ours, "tcgen05_tflops": fl / ours / 1e9,
        "torch_ms": ref, "torch_tflops": fl / ref / 1e9,
        "speedup": ref / ours,
        "max_theoretical_speedup_from_symmetry": (4 * e + 2) / (3 * e + 1),
        "max_abs_diff": err,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--single", action="store_true", help="one (m, n) point")
    ap.add_argument("--grid", action="store_true", help="square sizes 512 ... 8192")
    ap.add_argument("--expansion", type=int, default=1, help="n = expansion * m for --grid")
    ap.add_argument("--json", type=str, default=None, help="write the rows to this file")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required")
    rows = []
    if a.grid:
        for m in (512, 1024, 2048, 4096, 8192):
            rows.append(bench_one(m, m * a.expansion, a.batch_size))
    else:
        rows.append(bench_one(a.m, a.n, a.batch_size))
    for r in rows:
        print(f"{r['batch']:3d} x {r['m']:5d} x {r['n']:5d} | tcgen05 {r['tcgen05_ms']:8.3f} ms {r['tcgen05_tflops']:7.1f} TF"
              f" | torch {r['torch_ms']:8.3f} ms {r['torch_tflops']:7.1f} TF | x{r['speedup']:.2f}"
              f" (symmetry bound x{r['max_theoretical_speedup_from_symmetry']:.2f}) | max diff {r['max_abs_diff']:.3e}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
