"""Host-side utilities: the clock sampler against a stand-in `nvidia-smi`, the phase timers without a GPU."""
import os
import stat
import time

import pytest
import torch

from dion_b200.utils.clocks import ClockSampler
from dion_b200.utils.timers import PhaseTimers

_FAKE = """#!/bin/sh
# prints what `nvidia-smi --query-gpu=... --format=csv,noheader,nounits -lms N` prints, forever
i=0
while true; do
  if [ $i -lt 2 ]; then echo "0, 345, 1965, 180.5, Not Active, Not Active, Not Active, Not Active";
  else echo "0, 1650, 1965, 951.2, Not Active, Not Active, Not Active, Active"; fi
  i=$((i+1))
  sleep 0.02
done
"""


def test_clock_sampler_reports_clocks_under_load_and_reasons(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(_FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    s = ClockSampler(gpu_index=0, period_ms=20)
    s.start()
    time.sleep(0.5)
    out = s.stop()
    assert out["samples"] >= 5
    assert out["sm_mhz"] == 1650.0            # the idle samples (low power) do not count
    assert out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert out["power_w_max"] == 951.2


def test_clock_sampler_without_the_tool(monkeypatch, tmp_path):
    monkeypatch.setenv("PATH", str(tmp_path))
    s = ClockSampler()
    s.start()
    assert s.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="describes the machine without a GPU")
def test_phase_timers_are_inert_without_a_gpu():
    t = PhaseTimers(enabled=True)
    t.start("a")
    t.stop("a")
    assert t.summary() == {} and t.max_over_ranks() == {}


@pytest.mark.parametrize("M,N,K,rows,world", [(512, 96, 64, 256, 2), (2048, 1536, 768, 1024, 2), (8192, 2304, 768, 4096, 2),
                                              (4096, 4096, 1024, 2048, 2), (32768, 1536, 768, 16384, 2),
                                              (65536, 384, 768, 8192, 8), (32768, 768, 768, 4096, 8)])
def test_gather_gemm_plan_invariants(M, N, K, rows, world):
    """Host-side plan of the GEMM that all-gathers its first operand: every tile's rows sit inside one
    readiness chunk of one source rank, tiles are visited own rows first and then in ring order (the order
    in which the copier warps fetch), the copy units tile every chunk exactly, and the counter buffer the
    Python side allocates is large enough."""
    from dion_b200.ops import _ext

    if not _ext.load(required=False):
        pytest.skip("extension not built")
    unit = 64 * 1024
    for rank in range(world):
        plan = list(torch.ops.dion_b200.gemm_gather_plan(M, N, K, rows, world, rank))
        assert plan, "shapes were rejected"
        tile_m, bn, pair, chunk_rows, units_per_chunk, m_rot, tiles_m, tiles_n = plan
        assert tile_m == (256 if pair else 128) and bn in (128, 256)
        assert rows % chunk_rows == 0 and chunk_rows % tile_m == 0 and tiles_m * tile_m == M
        assert 2 + M // chunk_rows <= 2 + M // 128
        ring_seen = []
        for t in range(tiles_m * tiles_n):
            m_blk = (t // tiles_n + m_rot) % tiles_m
            row0 = m_blk * tile_m
            assert row0 % chunk_rows + tile_m <= chunk_rows          # one chunk per tile (both CTAs of a pair)
            src = row0 // rows
            assert (row0 + tile_m - 1) // rows == src                # one source rank per tile
            ring = (src - rank) % world
            if not ring_seen or ring_seen[-1] != ring:
                ring_seen.append(ring)
        assert ring_seen == list(range(world))                       # own rows first, then ring order, each once
        chunk_bytes = chunk_rows * K * 2
        assert units_per_chunk == -(-chunk_bytes // unit)
        covered = 0
        for u in range(units_per_chunk):
            lo, hi = u * unit, min((u + 1) * unit, chunk_bytes)
            assert lo < hi and lo % 16 == 0 and (hi - lo) % 16 == 0
            covered += hi - lo
        assert covered == chunk_bytes


def test_gather_gemm_plan_rejects_ragged_row_blocks():
    from dion_b200.ops import _ext

    if not _ext.load(required=False):
        pytest.skip("extension not built")
    assert list(torch.ops.dion_b200.gemm_gather_plan(400, 96, 64, 200, 2, 0)) == []      # rows not a multiple of 128
    assert list(torch.ops.dion_b200.gemm_gather_plan(512, 96, 64, 256, 3, 0)) == []      # world * rows != M


def _load_benchmark_module(name):
    import importlib.util

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, "benchmark", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_newton_schulz_benchmark_flop_count_and_plot(tmp_path):
    """FLOP accounting of the Newton-Schulz benchmark (4 m^2 n + 2 m^3 per step, the smaller dimension as m,
    as in the reference's script) and its SVG plot writer, which needs no plotting library."""
    bench = _load_benchmark_module("benchmark_newton_schulz")
    assert bench.ns_flops(4, 8, iters=1) == 4 * 16 * 8 + 2 * 64
    assert bench.ns_flops(8, 4, iters=1) == bench.ns_flops(4, 8, iters=1)
    assert bench.ns_flops(4, 8, batch=3, iters=5) == 15 * bench.ns_flops(4, 8, iters=1)
    rows = [{"m": 512, "tcgen05_tflops": 100.0, "torch_tflops": 80.0},
            {"m": 1024, "tcgen05_tflops": 400.0, "torch_tflops": 300.0, "triton_ref_tflops": 350.0}]
    path = tmp_path / "sub" / "ns.svg"
    bench.write_plot(rows, str(path))
    svg = path.read_text()
    assert svg.startswith("<svg") and svg.rstrip().endswith("</svg>")
    assert svg.count("<polyline") == 3 and "reference Triton" in svg and ">1024<" in svg


def test_loss_curve_markov_batches_are_reproducible_and_follow_the_chain():
    lc = _load_benchmark_module("loss_curve")
    a = lc.markov_batches(2, 3, 16, states=8, fanout=2, vocab=50, seed=5)
    b = lc.markov_batches(2, 3, 16, states=8, fanout=2, vocab=50, seed=5)
    assert all(torch.equal(x1, x2) and torch.equal(y1, y2) for (x1, y1), (x2, y2) in zip(a, b))
    x, y = a[0]
    assert x.shape == (3, 16) and torch.equal(x[:, 1:], y[:, :-1])     # targets are the inputs shifted by one
    assert len(torch.unique(torch.cat([x.flatten(), y.flatten()]))) <= 8
    # every token has at most `fanout` distinct successors over all batches
    succ = {}
    for x, y in a:
        for s, t in zip(x.flatten().tolist(), y.flatten().tolist()):
            succ.setdefault(s, set()).add(t)
    assert max(len(v) for v in succ.values()) <= 2


def test_openmp_compiler_selection(tmp_path, monkeypatch):
    """`ensure_openmp_cxx` keeps a compiler that can build OpenMP code and replaces one that cannot."""
    from dion_b200.utils import compilers

    assert compilers.can_openmp("/nonexistent/compiler") is False
    broken = tmp_path / "g++"
    broken.write_text("#!/bin/sh\nexit 1\n")
    broken.chmod(broken.stat().st_mode | stat.S_IEXEC)
    assert compilers.can_openmp(str(broken)) is False
    monkeypatch.setenv("CXX", str(broken))
    chosen = compilers.ensure_openmp_cxx()
    if chosen:                                   # a working compiler exists on this machine
        assert chosen != str(broken) and os.environ["CXX"] == chosen and compilers.can_openmp(chosen)
        monkeypatch.setenv("CXX", chosen)
        assert compilers.ensure_openmp_cxx() == chosen
