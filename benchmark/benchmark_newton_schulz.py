"""Newton-Schulz micro-benchmark: the tcgen05 implementation against the plain bf16-matmul
one (three library GEMMs per iteration), the comparison the reference makes for its Triton
kernels (benchmark/benchmark_newton_shultz.py:33-101, 173).

    python benchmark/benchmark_newton_schulz.py --single --m 4096 --n 14336
    python benchmark/benchmark_newton_schulz.py --grid            # 512 ... 8192, square
    python benchmark/benchmark_newton_schulz.py --batch_size 12 --m 768 --n 3072

`--triton_ref` adds a third arm: the reference's own Triton kernels (``newton_schulz_triton`` of the
unmodified reference package installed under baseline/_ref, dion/newton_schulz_triton.py:337-374,
timed like benchmark/benchmark_newton_shultz.py:49-101 does), on the same inputs and the same box.

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


_triton_fn = None
_triton_why = None


def reference_triton_newton_schulz():
    """The reference's ``newton_schulz_triton`` (imported from baseline/_ref, unmodified), or None with
    the reason in ``_triton_why`` when it cannot be used on this machine."""
    global _triton_fn, _triton_why
    if _triton_fn is not None or _triton_why is not None:
        return _triton_fn
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dion")):
        _triton_why = "baseline/_ref is not installed"
        return None
    # Inductor's host-side code needs a C++ compiler with OpenMP; some images put one first on PATH that lacks it
    from dion_b200.utils.compilers import ensure_openmp_cxx

    ensure_openmp_cxx()
    sys.path.insert(0, ref_dir)
    for name in [m for m in sys.modules if m == "dion" or m.startswith("dion.")]:
        del sys.modules[name]
    try:
        from dion.newton_schulz_triton import newton_schulz_triton

        _triton_fn = newton_schulz_triton
    except Exception as e:
        _triton_why = f"import failed: {type(e).__name__}: {e}"[:200]
    finally:
        sys.path.remove(ref_dir)
    return _triton_fn


def bench_one(m: int, n: int, batch: int, iters: int = 10, triton_ref: bool = False):
    global _triton_fn, _triton_why
    shape = (batch, m, n) if batch > 1 else (m, n)
    G = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
    ours = cuda_time_ms(lambda: newton_schulz(G), iters=iters, warmup=3, flush_l2=True)
    ref = cuda_time_ms(lambda: newton_schulz_torch(G), iters=iters, warmup=3, flush_l2=True)
    fl = ns_flops(m, n, batch)
    e = max(m, n) / min(m, n)
    err = (newton_schulz(G).float() - newton_schulz_torch(G).float()).abs().max().item()
    row = {
        "m": m, "n": n, "batch": batch,
        "tcgen05_ms": ours, "tcgen05_tflops": fl / ours / 1e9,
        "torch_ms": ref, "torch_tflops": fl / ref / 1e9,
        "speedup": ref / ours,
        "max_theoretical_speedup_from_symmetry": (4 * e + 2) / (3 * e + 1),
        "max_abs_diff": err,
    }
    if triton_ref:
        fn = reference_triton_newton_schulz()
        if fn is not None:
            try:
                fn(G)  # compile + autotune
                tri = cuda_time_ms(lambda: fn(G), iters=iters, warmup=3, flush_l2=True)
                row.update(triton_ref_ms=tri, triton_ref_tflops=fl / tri / 1e9, speedup_vs_triton_ref=tri / ours)
            except Exception as ex:  # the compiler stack may be unusable on a machine
                _triton_fn, _triton_why = None, f"{type(ex).__name__}: {str(ex).splitlines()[-1] if str(ex) else ''}"[:200]
        if _triton_why is not None:
            row["triton_ref_unavailable"] = _triton_why
    return row


def write_plot(rows, path: str) -> None:
    """TFLOPS over the matrix size for every arm, as the reference's `--plot` draws it
    (benchmark/benchmark_newton_shultz.py:104-170) - written as a plain SVG file, no plotting library needed."""
    arms = [("tcgen05_tflops", "tcgen05 (this package)", "#d62728"), ("torch_tflops", "PyTorch", "#1f77b4"),
            ("triton_ref_tflops", "reference Triton", "#2ca02c")]
    arms = [a for a in arms if any(a[0] in r for r in rows)]
    xs = [r["m"] for r in rows]
    top = max(r.get(k, 0.0) for r in rows for k, _, _ in arms) * 1.1 or 1.0
    W, H, L, B = 640, 400, 70, 50
    px = lambda i: L + (W - L - 20) * (i / max(len(xs) - 1, 1))
    py = lambda v: H - B - (H - B - 20) * (v / top)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="12">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<line x1="{L}" y1="{H - B}" x2="{W - 20}" y2="{H - B}" stroke="black"/>',
           f'<line x1="{L}" y1="20" x2="{L}" y2="{H - B}" stroke="black"/>',
           f'<text x="{W / 2}" y="{H - 10}" text-anchor="middle">matrix dimension m (n = expansion x m)</text>',
           f'<text x="15" y="{H / 2}" transform="rotate(-90 15 {H / 2})" text-anchor="middle">TFLOPS (4 m^2 n + 2 m^3 per step)</text>']
    for i, x in enumerate(xs):
        out.append(f'<text x="{px(i)}" y="{H - B + 18}" text-anchor="middle">{x}</text>')
    for t in range(5):
        v = top * t / 4
        out.append(f'<text x="{L - 6}" y="{py(v) + 4}" text-anchor="end">{v:.0f}</text>')
        out.append(f'<line x1="{L}" y1="{py(v)}" x2="{W - 20}" y2="{py(v)}" stroke="#dddddd"/>')
    for j, (key, label, colour) in enumerate(arms):
        pts = " ".join(f"{px(i)},{py(r[key])}" for i, r in enumerate(rows) if key in r)
        out.append(f'<polyline points="{pts}" fill="none" stroke="{colour}" stroke-width="2"/>')
        out.append(f'<rect x="{L + 15}" y="{28 + 16 * j}" width="12" height="3" fill="{colour}"/>')
        out.append(f'<text x="{L + 32}" y="{34 + 16 * j}">{label}</text>')
    out.append("</svg>")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--single", action="store_true", help="one (m, n) point")
    ap.add_argument("--grid", action="store_true", help="square sizes 512 ... 8192")
    ap.add_argument("--expansion", type=int, default=1, help="n = expansion * m for --grid")
    ap.add_argument("--json", type=str, default=None, help="write the rows to this file")
    ap.add_argument("--triton_ref", action="store_true", help="also time the reference's Triton kernels (baseline/_ref)")
    ap.add_argument("--plot", type=str, default=None, metavar="FILE.svg",
                    help="draw TFLOPS over the size for every arm (use with --grid)")
    ap.add_argument("--shapes", type=str, default=None,
                    help="several points in one run: comma-separated batch x m x n, e.g. 1x4096x4096,12x768x3072")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required")
    rows = []
    if a.shapes:
        for item in a.shapes.split(","):
            b, m, n = (int(v) for v in item.lower().split("x"))
            rows.append(bench_one(m, n, b, triton_ref=a.triton_ref))
    elif a.grid:
        for m in (512, 1024, 2048, 4096, 8192):
            rows.append(bench_one(m, m * a.expansion, a.batch_size, triton_ref=a.triton_ref))
    else:
        rows.append(bench_one(a.m, a.n, a.batch_size, triton_ref=a.triton_ref))
    for r in rows:
        tri = ""
        if "triton_ref_ms" in r:
            tri = f" | reference Triton {r['triton_ref_ms']:8.3f} ms {r['triton_ref_tflops']:7.1f} TF (x{r['speedup_vs_triton_ref']:.2f})"
        elif "triton_ref_unavailable" in r:
            tri = f" | reference Triton unavailable: {r['triton_ref_unavailable']}"
        print(f"{r['batch']:3d} x {r['m']:5d} x {r['n']:5d} | tcgen05 {r['tcgen05_ms']:8.3f} ms {r['tcgen05_tflops']:7.1f} TF"
              f" | torch {r['torch_ms']:8.3f} ms {r['torch_tflops']:7.1f} TF | x{r['speedup']:.2f}"
              f" (symmetry bound x{r['max_theoretical_speedup_from_symmetry']:.2f}) | max diff {r['max_abs_diff']:.3e}{tri}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    if a.plot:
        write_plot(rows, a.plot)


if __name__ == "__main__":
    main()
