"""The free functions and import paths that mirror the reference's module-level helpers
(dion/opt_utils.py, dion/scalar_opts.py, dion/dion.py:1165-1602, dion/muon.py:489-593): same results as the
reference's own functions where the reference is installed, and the documented contracts everywhere."""
import importlib

import pytest
import torch

from _reference import load_reference

ref_pkg = load_reference()
needs_ref = pytest.mark.skipif(ref_pkg is None, reason="reference package not installed under baseline/_ref")


def _ref(module):
    return importlib.import_module(f"dion.{module}")


def test_reference_import_paths_resolve():
    import dion_b200
    from dion_b200.dion import Dion, DionMixedPrecisionConfig, orthogonalize  # noqa: F401
    from dion_b200.dion_reference import Dion as RefDion
    from dion_b200.dion_simple import Dion as SimpleDion, dion_update  # noqa: F401
    from dion_b200.muon import Muon, adjust_lr_spectral_norm, zeropower_via_newtonschulz5  # noqa: F401
    from dion_b200.muon_reference import Muon as RefMuon, MuonKellerJordan  # noqa: F401
    from dion_b200.newton_schulz_triton import newton_schulz_triton, ns_line_1, ns_line_2  # noqa: F401
    from dion_b200.opt_utils import AsyncRuntime, AsyncTask, create_param_batches, dtensor_from_local, pad_batch, to_local  # noqa: F401
    from dion_b200.scalar_opts import adamw_update, adamw_update_foreach, lion_update, lion_update_foreach  # noqa: F401

    assert RefDion is dion_b200.DionReference and SimpleDion is dion_b200.DionSimple and RefMuon is dion_b200.MuonReference
    assert Dion is dion_b200.Dion and Muon is dion_b200.Muon


@needs_ref
def test_every_module_level_name_of_the_reference_has_a_counterpart():
    """Public functions and classes defined in the reference's modules exist under the same name in the module
    of the same name here (Triton kernel bodies and the per-topology update generators excepted: their work is
    done by CUDA kernels and by the optimizer classes' phases)."""
    import inspect

    internal = {"dion": {"dion_update_ddp", "dion_update_fsdp", "dion_update_fsdp_tp"},
                "muon": {"muon_update_batch_async"},
                "newton_schulz_triton": {"ns_line_1_kernel", "ns_line_2_kernel"},
                "dion_reference": {"generate_random_sketch_dtensor"}}
    missing = []
    for name in ("opt_utils", "scalar_opts", "dion", "muon", "newton_schulz_triton", "dion_reference", "dion_simple",
                 "muon_reference"):
        theirs = _ref(name)
        ours = importlib.import_module(f"dion_b200.{name}")
        for sym, obj in vars(theirs).items():
            if sym.startswith("_") or sym in internal.get(name, ()):
                continue
            defined_there = getattr(obj, "__module__", None) == theirs.__name__ or (
                hasattr(obj, "_torchdynamo_orig_callable") or hasattr(obj, "__wrapped__"))
            if not (inspect.isfunction(obj) or inspect.isclass(obj) or callable(obj)) or not defined_there:
                continue
            if inspect.ismodule(obj) or getattr(obj, "__module__", "").startswith(("torch", "typing", "triton")):
                continue
            if not hasattr(ours, sym):
                missing.append(f"{name}.{sym}")
    assert not missing, missing


def test_async_runtime_interleaves_tasks_like_an_event_loop():
    from dion_b200.opt_utils import AsyncRuntime, AsyncTask

    trace = []

    def work(tag, steps):
        for i in range(steps):
            trace.append((tag, i))
            yield

    def tasks():
        for tag, steps in (("a", 3), ("b", 1), ("c", 2)):
            yield AsyncTask(work(tag, steps))

    AsyncRuntime(tasks(), max_concurrent_tasks=2).run()
    assert sorted(trace) == [("a", 0), ("a", 1), ("a", 2), ("b", 0), ("c", 0), ("c", 1)]
    assert trace.index(("b", 0)) < trace.index(("a", 2))       # b started while a was still running
    assert trace.index(("c", 0)) > trace.index(("b", 0))       # never more than two alive
    with pytest.raises(ValueError):
        AsyncRuntime(tasks(), max_concurrent_tasks=0)


@needs_ref
def test_async_runtime_matches_the_reference_schedule():
    ours = importlib.import_module("dion_b200.opt_utils")
    theirs = _ref("opt_utils")
    traces = []
    for mod in (ours, theirs):
        trace = []

        def work(tag, steps, trace=trace):
            for i in range(steps):
                trace.append((tag, i))
                yield

        def tasks(mod=mod):
            for tag, steps in (("a", 4), ("b", 2), ("c", 5), ("d", 1), ("e", 3)):
                yield mod.AsyncTask(work(tag, steps))

        mod.AsyncRuntime(tasks(), max_concurrent_tasks=3).run()
        traces.append(trace)
    assert traces[0] == traces[1]


def test_param_batches_and_padding():
    from dion_b200.opt_utils import create_param_batches, pad_batch

    ps = [torch.zeros(4, 3), torch.zeros(4, 3), torch.zeros(2, 3), torch.zeros(4, 3), torch.zeros(4, 3, dtype=torch.bfloat16)]
    batches = list(create_param_batches(ps, 2))
    assert [len(b) for b in batches] == [2, 1, 1, 1]
    assert all(len({(tuple(t.shape), t.dtype) for t in b}) == 1 for b in batches)
    padded = pad_batch(list(batches[1]), 3)
    assert len(padded) == 3 and all(t.shape == padded[0].shape for t in padded)
    with pytest.raises(ValueError):
        pad_batch([], 2)


@needs_ref
@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_scalar_updates_match_the_reference_functions(state_dtype):
    ours = importlib.import_module("dion_b200.scalar_opts")
    theirs = _ref("scalar_opts")
    torch.manual_seed(0)
    shapes = [(7, 5), (33,), (4, 4, 2)]
    X0 = [torch.randn(s) for s in shapes]
    G = [torch.randn(s) for s in shapes]
    hp = dict(lr=torch.tensor(0.01), beta1=torch.tensor(0.9), beta2=torch.tensor(0.95), weight_decay=torch.tensor(0.1))
    res = []
    for mod in (ours, theirs):
        X = [x.clone() for x in X0]
        M = [torch.zeros_like(x, dtype=state_dtype) for x in X]
        V = [torch.zeros_like(x, dtype=state_dtype) for x in X]
        for step in (1, 2, 3):
            mod.adamw_update_foreach(X, G, M, V, hp["lr"], hp["beta1"], hp["beta2"], hp["weight_decay"], step, 1e-8)
        X2 = [x.clone() for x in X0]
        M2 = [torch.zeros_like(x, dtype=state_dtype) for x in X]
        for _ in range(3):
            mod.lion_update_foreach(X2, G, M2, hp["lr"], hp["beta1"], hp["beta2"], hp["weight_decay"])
        mod.lion_update(X2[0], G[0], M2[0], hp["lr"], hp["beta1"], hp["beta2"], hp["weight_decay"])
        mod.adamw_update(X[0], G[0], M[0], V[0], hp["lr"], hp["beta1"], hp["beta2"], hp["weight_decay"], 4, 1e-8)
        res.append((X, M, V, X2, M2))
    tol = dict(rtol=1e-5, atol=1e-6) if state_dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
    for a, b in zip(res[0], res[1]):
        for x, y in zip(a, b):
            torch.testing.assert_close(x.float(), y.float(), **tol)


@needs_ref
@pytest.mark.parametrize("nesterov", [False, True])
def test_muon_pre_and_post_match_the_reference_functions(nesterov):
    ours = importlib.import_module("dion_b200.muon")
    theirs = _ref("muon")
    torch.manual_seed(1)
    G = [torch.randn(6, 4), torch.randn(3, 9)]
    res = []
    for mod in (ours, theirs):
        M = [torch.full_like(g, 0.25) for g in G]
        X = [torch.ones_like(g) for g in G]
        U = mod.muon_update_pre_orthogonalize(G, M, torch.tensor(0.95), nesterov)
        assert all(u.dtype == torch.bfloat16 for u in U)
        mod.muon_update_post_orthogonalize(X, U, torch.tensor(0.02), torch.tensor(0.01), torch.tensor(0.1))
        res.append((M, U, X))
    for a, b in zip(res[0], res[1]):
        for x, y in zip(a, b):
            torch.testing.assert_close(x.float(), y.float(), rtol=1e-2, atol=1e-3)
    # shapes with more than two dimensions go through the flatten rules
    X4 = torch.randn(2, 3, 8, 4)
    f = lambda x, epsilon: x * 2
    for flatten in (False, True):
        torch.testing.assert_close(ours.muon_update_newton_schulz(X4, f, flatten, 1e-7),
                                   theirs.muon_update_newton_schulz(X4, f, flatten, 1e-7))


@needs_ref
def test_dion_building_blocks_match_the_reference_functions():
    ours = importlib.import_module("dion_b200.dion")
    theirs = _ref("dion")
    torch.manual_seed(2)
    B, m, n, r = 3, 10, 6, 4
    Mlist = [torch.randn(m, n) for _ in range(B)]
    Qlist = [torch.randn(n, r).bfloat16() for _ in range(B)]
    for transposed in (False, True):
        a = ours.tensor_list_to_batch(Mlist, [q if not transposed else torch.randn(m, r).bfloat16() for q in Qlist], transposed)
        assert a[0].shape == ((B, n, m) if transposed else (B, m, n)) and a[1].dtype == a[0].dtype
    Mb, Qb = ours.tensor_list_to_batch(Mlist, Qlist, False)
    Mt, Qt = theirs.tensor_list_to_batch(Mlist, Qlist, False)
    assert torch.equal(Mb, Mt) and torch.equal(Qb, Qt)

    P = torch.randn(B, m, r)
    R = torch.randn(B, n, r)
    P[1] = float("nan")
    Bz = torch.randn(B, m, n)
    Bz[1] = 0
    Pa, Ra = ours.fix_all_zero_or_nan(P, R, Qb, Bz)
    Pb, Rb = theirs.fix_all_zero_or_nan(P, R, Qb, Bz)
    torch.testing.assert_close(Pa, Pb)
    torch.testing.assert_close(Ra, Rb)
    assert torch.equal(Pa[1], torch.zeros(m, r)) and torch.equal(Ra[1], Qb[1])

    torch.testing.assert_close(ours.local_column_sum_sq(R), theirs.local_column_sum_sq(R))
    torch.testing.assert_close(ours.column_normalize(R), theirs.column_normalize(R))
    ss = theirs.local_column_sum_sq(R) * 2
    torch.testing.assert_close(ours.column_normalize(R.bfloat16(), ss, 1e-6).float(),
                               theirs.column_normalize(R.bfloat16(), ss, 1e-6).float())

    for transpose in (False, True):
        Xa = [torch.randn(m, n) if not transpose else torch.randn(n, m) for _ in range(B)]
        Xb = [x.clone() for x in Xa]
        ours.foreach_baddbmm_(Xa, P.nan_to_num(), R, alpha=-0.3, beta=0.9, transpose=transpose)
        theirs.foreach_baddbmm_(Xb, P.nan_to_num(), R, alpha=-0.3, beta=0.9, transpose=transpose)
        for x, y in zip(Xa, Xb):
            torch.testing.assert_close(x, y, rtol=1e-5, atol=1e-5)

    Qa = [q.clone() for q in Qlist]
    Qc = [q.clone() for q in Qlist]
    ours.update_Q_matrix_(Qa, R)
    theirs.update_Q_matrix_(Qc, R)
    assert all(torch.equal(x, y) for x, y in zip(Qa, Qc))

    S = ours.generate_random_sketch_matrix(P, oversample=1.25)
    assert S.shape == (B, 128, m) and abs(float(S.std()) - (1 / 128) ** 0.5) < 0.01


@pytest.mark.parametrize("shape", [(3, 40, 8), (2, 2, 16, 16)])
def test_orthogonalize_returns_the_qr_factor(shape):
    from dion_b200.dion import orthogonalize

    torch.manual_seed(3)
    P = torch.randn(*shape)
    Q = orthogonalize(P)
    assert Q.shape == P.shape and Q.dtype == P.dtype
    r = shape[-1]
    torch.testing.assert_close(Q.mT @ Q, torch.eye(r).expand(*shape[:-2], r, r), rtol=1e-4, atol=1e-4)
    # same column spans, nested like a QR factorisation with positive diagonal: Q^T P is upper triangular
    Rm = Q.mT @ P
    assert float(torch.tril(Rm, -1).abs().max()) < 1e-3 * float(Rm.abs().max())
    assert bool((torch.diagonal(Rm, dim1=-2, dim2=-1) > 0).all())
    with pytest.raises(ValueError):
        orthogonalize(torch.randn(4, 4))


def test_orthogonalize_of_a_wide_matrix_is_the_householder_factor():
    """More columns than rows: the reduced QR factor [m, m], as the reference returns it."""
    from dion_b200.dion import orthogonalize

    torch.manual_seed(5)
    P = torch.randn(2, 6, 12)
    torch.testing.assert_close(orthogonalize(P), torch.linalg.qr(P)[0])


@needs_ref
def test_power_iteration_and_dion_update_match_the_reference_oracle():
    ours = importlib.import_module("dion_b200.dion_reference")
    theirs = _ref("dion_reference")
    torch.manual_seed(4)
    m, n, r = 24, 16, 4
    Bm = torch.randn(m, 3) @ torch.randn(3, n) + 0.01 * torch.randn(m, n)
    Q0 = torch.randn(n, r)
    Pa, Qa = ours.power_iteration(Bm, Q0, 2, "qr", 1.25, False)
    Pb, Qb = theirs.power_iteration(Bm, Q0, power_iters=2, qr_method="qr", oversample=1.25, compressed_all_reduce=False)
    torch.testing.assert_close(Pa, Pb, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(Qa, Qb, rtol=1e-4, atol=1e-4)

    for transpose in (False, True):
        X0, G = torch.randn(m, n), torch.randn(m, n)
        Qi = torch.randn(m if transpose else n, r)
        outs = []
        for mod in (ours, theirs):
            X, M = X0.clone(), torch.zeros(m, n)
            Q = Qi.clone()
            for _ in range(2):
                Q = mod.dion_update(X, G, M, Q, torch.tensor(0.01), torch.tensor(0.95), torch.tensor(0.1), 1e-8, transpose,
                                    1, "qr", 1.25, False, None)
            outs.append((X, M, Q))
        for x, y in zip(outs[0], outs[1]):
            torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)


def test_model_import_paths_of_the_reference(tmp_path):
    from dion_b200.models import gpt_model, gpt_utils
    from dion_b200.models.data import write_datafile

    assert gpt_model.GPT is importlib.import_module("dion_b200.models").GPT
    for name in ("GPTConfig", "Rotary", "CausalSelfAttention", "MLP", "Block", "parallelize_gpt_model", "_apply_tp",
                 "_apply_fsdp", "apply_rotary_emb"):
        assert hasattr(gpt_model, name), name
    toks = (torch.arange(1000) % 50000).numpy().astype("uint16")
    path = str(tmp_path / "shard.bin")
    write_datafile(path, toks)
    assert gpt_utils._peek_data_shard(path) == 1000
    assert (gpt_utils._load_data_shard(path) == toks).all()


@needs_ref
def test_apply_rotary_emb_and_shard_readers_match_the_reference(tmp_path):
    import sys

    from dion_b200.models import gpt_model, gpt_utils
    from dion_b200.models.data import write_datafile

    ref_root = [p for p in sys.path if p.endswith("_ref") or p == __import__("os").environ.get("DION_REFERENCE_PATH")][0]
    sys.path.insert(0, ref_root)
    for m in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
        del sys.modules[m]
    ref_model = importlib.import_module("models.gpt_model")
    ref_utils = importlib.import_module("models.gpt_utils")
    torch.manual_seed(6)
    x = torch.randn(2, 9, 3, 16)
    rot = ref_model.Rotary(16)
    rot.init_inv_freq()
    cos, sin = rot(x)
    torch.testing.assert_close(gpt_model.apply_rotary_emb(x, cos.float(), sin.float()),
                               ref_model.apply_rotary_emb(x, cos.float(), sin.float()), rtol=1e-5, atol=1e-5)
    toks = (torch.arange(777) * 13 % 50000).numpy().astype("uint16")
    path = str(tmp_path / "shard.bin")
    write_datafile(path, toks)
    assert gpt_utils._peek_data_shard(path) == ref_utils._peek_data_shard(path)
    assert (gpt_utils._load_data_shard(path) == ref_utils._load_data_shard(path)).all()
