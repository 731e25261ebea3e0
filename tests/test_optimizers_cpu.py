"""Optimizers on CPU against the reference implementations (state injected so that one
step is comparable) and against their own contracts."""
import copy

import pytest
import torch

import dion_b200
from dion_b200 import Dion, DionMixedPrecisionConfig, DionReference, DionSimple, Muon, MuonReference
from dion_b200.optim.newton_schulz import newton_schulz_torch

from _reference import load_reference

ref = load_reference()
needs_ref = pytest.mark.skipif(ref is None, reason="reference package not importable")

SHAPES = [(64, 32), (32, 64), (48, 48), (64, 32), (96, 24)]


def _params(shapes=SHAPES):
    return [torch.nn.Parameter(torch.randn(s)) for s in shapes]


def _clone(ps):
    return [torch.nn.Parameter(p.detach().clone()) for p in ps]


def _set_grads(a, b, scale=1.0):
    for p, q in zip(a, b):
        g = torch.randn_like(p) * scale
        p.grad = g.clone()
        q.grad = g.clone()


def _inject_q(opt, opt_ref, P, Pr):
    for g in opt.param_groups:
        for p in g["params"]:
            if g["algorithm"] == "dion":
                opt._get_or_initialize_state(p, g)
    for p, pr in zip(P, Pr):
        if "Q" in opt.state[p]:
            opt_ref.state[pr] = {"momentum": torch.zeros_like(pr), "Q": opt.state[p]["Q"].clone()}


def test_public_names():
    for name in ("Dion", "DionMixedPrecisionConfig", "DionSimple", "DionReference", "Muon", "MuonReference"):
        assert hasattr(dion_b200, name)


@needs_ref
@pytest.mark.parametrize("rank_fraction", [1.0, 0.5, 0.25])
def test_dion_matches_reference_qr(rank_fraction):
    P = _params()
    Pr = _clone(P)
    opt = Dion(P, lr=0.02, rank_fraction=rank_fraction, weight_decay=0.1)
    opt_ref = ref.DionReference(Pr, lr=0.02, rank_fraction=rank_fraction, weight_decay=0.1, qr_method="qr")
    _inject_q(opt, opt_ref, P, Pr)
    for _ in range(4):
        _set_grads(P, Pr)
        opt.step()
        opt_ref.step()
        for p, pr in zip(P, Pr):
            torch.testing.assert_close(p, pr, rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(opt.state[p]["momentum"], opt_ref.state[pr]["momentum"], rtol=1e-4, atol=1e-4)
            q, qr = opt.state[p]["Q"], opt_ref.state[pr]["Q"]
            sign = torch.sign((q * qr).sum(0, keepdim=True))
            torch.testing.assert_close(q * sign, qr, rtol=1e-3, atol=1e-4)


@needs_ref
def test_dion_matches_reference_async_dion_with_scalar_groups():
    P = _params()
    e = torch.nn.Parameter(torch.randn(100, 16))
    h = torch.nn.Parameter(torch.randn(16, 100))
    Pr, er, hr = _clone(P), _clone([e])[0], _clone([h])[0]
    groups = lambda ps, a, b: [dict(params=ps), dict(params=[a], algorithm="lion", lr=0.01, weight_decay=0),
                               dict(params=[b], algorithm="adamw", lr=0.003, betas=(0.95, 0.98))]
    opt = Dion(groups(P, e, h), lr=0.02, rank_fraction=0.5)
    opt_ref = ref.Dion(groups(Pr, er, hr), lr=0.02, rank_fraction=0.5)
    _inject_q(opt, opt_ref, P, Pr)
    for _ in range(3):
        _set_grads(P + [e, h], Pr + [er, hr])
        opt.step()
        opt_ref.step()
    for p, pr in zip(P + [e, h], Pr + [er, hr]):
        torch.testing.assert_close(p, pr, rtol=1e-4, atol=2e-5)
    # parameter-group keys and state keys are the reference's
    assert set(opt.param_groups[0].keys()) == set(opt_ref.param_groups[0].keys())
    assert set(opt.state[P[0]].keys()) == {"momentum", "Q"}
    assert set(opt.state[e].keys()) == {"momentum"}
    assert set(opt.state[h].keys()) == {"momentum", "variance"}
    assert [g["step"] for g in opt.param_groups] == [3, 3, 3]


@needs_ref
@pytest.mark.parametrize("qr_method", ["qr", "cqr", "rcqr"])
def test_dion_reference_matches_reference(qr_method):
    P = _params()
    Pr = _clone(P)
    kw = dict(lr=0.02, rank_fraction=0.5, qr_method=qr_method, cqr_warmup_steps=1, power_iters=2)
    opt = DionReference(P, **kw)
    opt_ref = ref.DionReference(Pr, **kw)
    _inject_q(opt, opt_ref, P, Pr)
    for _ in range(3):
        _set_grads(P, Pr)
        opt.step()
        opt_ref.step()
    # the sketch is random, so rcqr agrees only up to the basis it spans; X and M are basis independent
    for p, pr in zip(P, Pr):
        torch.testing.assert_close(p, pr, rtol=2e-3, atol=2e-4)


@needs_ref
def test_dion_simple_matches_reference():
    P = _params([(64, 32), (48, 48)])
    Pr = _clone(P)
    opt = DionSimple(P, lr=0.02, rank=16)
    opt_ref = ref.DionSimple(Pr, lr=0.02, rank=16)
    for g in opt.param_groups:
        for p in g["params"]:
            opt._init_state(p, opt.state[p], "dion")
    for p, pr in zip(P, Pr):
        opt_ref.state[pr] = {"momentum": torch.zeros_like(pr), "Q": opt.state[p]["Q"].clone()}
    for _ in range(3):
        _set_grads(P, Pr)
        opt.step()
        opt_ref.step()
    for p, pr in zip(P, Pr):
        torch.testing.assert_close(p, pr, rtol=1e-4, atol=1e-5)


@needs_ref
@pytest.mark.parametrize("nesterov", [False, True])
@pytest.mark.parametrize("adjust_lr", ["spectral_norm", "rms_norm", "keller_muon", None])
def test_muon_matches_reference(nesterov, adjust_lr):
    P = _params()
    Pr = _clone(P)
    opt = Muon(P, lr=0.02, nesterov=nesterov, adjust_lr=adjust_lr)
    opt_ref = ref.Muon(Pr, lr=0.02, nesterov=nesterov, adjust_lr=adjust_lr)
    for _ in range(3):
        _set_grads(P, Pr)
        opt.step()
        opt_ref.step()
    for p, pr in zip(P, Pr):
        # bf16 Newton-Schulz: compare updates at bf16 accuracy
        assert (p - pr).abs().max() < 2e-3
    assert set(opt.param_groups[0].keys()) == set(opt_ref.param_groups[0].keys())
    assert set(opt.state[P[0]].keys()) == {"momentum"}


@needs_ref
def test_muon_reference_matches_reference():
    P = _params([(64, 32), (32, 64)])
    e = torch.nn.Parameter(torch.randn(50, 8))
    Pr, er = _clone(P), _clone([e])[0]
    mk = lambda ps, x: [dict(params=ps), dict(params=[x], algorithm="adamw", lr=0.01)]
    opt = MuonReference(mk(P, e), lr=0.02)
    opt_ref = ref.MuonReference(mk(Pr, er), lr=0.02)
    for _ in range(3):
        _set_grads(P + [e], Pr + [er])
        opt.step()
        opt_ref.step()
    for p, pr in zip(P + [e], Pr + [er]):
        assert (p - pr).abs().max() < 2e-3
    assert set(opt.state[P[0]].keys()) == set(opt_ref.state[Pr[0]].keys())
    assert set(opt.state[e].keys()) == set(opt_ref.state[er].keys())


def test_dion_argument_validation():
    p = _params([(8, 8)])
    for bad in (dict(lr=-1), dict(mu=-1), dict(betas=(0.9,)), dict(weight_decay=-1), dict(rank_fraction=0),
                dict(rank_fraction=1.5), dict(rank_multiple_of=0), dict(power_iters=2), dict(qr_method="qr")):
        with pytest.raises(ValueError):
            Dion(p, **bad)
    with pytest.raises(TypeError):
        Dion(p, replicate_mesh="mesh")
    with pytest.raises(ValueError):
        Muon(p, adjust_lr="bogus")
    with pytest.raises(TypeError):
        Muon(p, distributed_mesh=3)
    opt = Dion([torch.nn.Parameter(torch.randn(4, 4, 4))])
    opt.param_groups[0]["params"][0].grad = torch.randn(4, 4, 4)
    with pytest.raises((NotImplementedError, ValueError)):
        opt.step()


def test_dion_rank_rounding_and_transposition():
    p1 = torch.nn.Parameter(torch.randn(100, 40))
    p2 = torch.nn.Parameter(torch.randn(40, 100))
    opt = Dion([p1, p2], rank_fraction=0.3, rank_multiple_of=8)
    for p in (p1, p2):
        p.grad = torch.randn_like(p)
    opt.step()
    assert opt.state[p1]["Q"].shape == (40, 16)   # 0.3 * 40 = 12 -> 16; Q is (n, r) for tall
    assert opt.state[p2]["Q"].shape == (40, 16)   # transposed: Q is (m, r)
    assert opt._param_config[p2].is_transposed and not opt._param_config[p1].is_transposed


def test_dion_zero_gradient_zero_lr_step_is_noop_on_weights():
    """What distributed checkpoint loading does to create states: grads = 0, lr = 0, step()."""
    P = _params()
    before = [p.detach().clone() for p in P]
    e = torch.nn.Parameter(torch.randn(10, 4))
    opt = Dion([dict(params=P), dict(params=[e], algorithm="adamw")], lr=0.02, rank_fraction=0.5)
    for g in opt.param_groups:
        g["lr"] = 0.0
    for p in P + [e]:
        p.grad = torch.zeros_like(p)
    opt.step()
    for p, b in zip(P, before):
        assert torch.equal(p, b)
        st = opt.state[p]
        assert torch.isfinite(st["Q"]).all() and torch.isfinite(st["momentum"]).all()
        assert st["momentum"].abs().max() == 0
    m = Muon(_params([(16, 8)]), lr=0.0)
    q = m.param_groups[0]["params"][0]
    q.grad = torch.zeros_like(q)
    w = q.detach().clone()
    m.step()
    assert torch.equal(q, w)


def test_dion_mixed_precision_state_dtypes_and_state_dict_roundtrip():
    P = _params()
    e = torch.nn.Parameter(torch.randn(10, 4))
    cfg = DionMixedPrecisionConfig(momentum_dtype=torch.bfloat16, Q_dtype=torch.float32, variance_dtype=torch.bfloat16)
    mk = lambda ps, x: Dion([dict(params=ps), dict(params=[x], algorithm="adamw")], lr=0.02, rank_fraction=0.5,
                            mixed_precision_config=cfg)
    opt = mk(P, e)
    for _ in range(2):
        for p in P + [e]:
            p.grad = torch.randn_like(p)
        opt.step()
    assert opt.state[P[0]]["momentum"].dtype == torch.bfloat16
    assert opt.state[P[0]]["Q"].dtype == torch.float32
    assert opt.state[e]["variance"].dtype == torch.bfloat16
    sd = copy.deepcopy(opt.state_dict())
    P2, e2 = _clone(P), _clone([e])[0]
    opt2 = mk(P2, e2)
    opt2.load_state_dict(sd)
    g = [torch.randn_like(p) for p in P + [e]]
    for p, q, gg in zip(P + [e], P2 + [e2], g):
        p.grad = gg.clone()
        q.grad = gg.clone()
    opt.step()
    opt2.step()
    for p, q in zip(P + [e], P2 + [e2]):
        torch.testing.assert_close(p, q)


def test_newton_schulz_orthogonalises():
    G = torch.randn(3, 32, 64)
    X = newton_schulz_torch(G).float()
    s = torch.linalg.svdvals(X)
    assert s.max() < 1.3 and s.min() > 0.5


def test_muon_custom_newton_schulz_and_flatten():
    calls = []

    def ns(x, epsilon):
        calls.append(tuple(x.shape))
        return newton_schulz_torch(x, epsilon)

    p = torch.nn.Parameter(torch.randn(4, 6, 5))
    opt = Muon([p], lr=0.01, newton_schulz_func=ns, flatten=True)
    p.grad = torch.randn_like(p)
    opt.step()
    assert calls and calls[0][-2:] == (4, 30)


def test_scheduler_admits_one_task_per_turn_and_bounds_tasks_in_flight():
    from dion_b200.optim.common import Scheduler

    log, alive, peak = [], set(), [0]

    def make(i, yields):
        def gen():
            alive.add(i)
            peak[0] = max(peak[0], len(alive))
            log.append(("start", i))
            for k in range(yields):
                yield
                log.append(("resume", i, k))
            alive.discard(i)
            log.append(("end", i))
        return gen

    Scheduler((make(i, 3) for i in range(6)), max_in_flight=2).run()
    assert peak[0] == 2
    assert [e[1] for e in log if e[0] == "start"] == list(range(6))      # tasks are created lazily, in order
    assert sum(1 for e in log if e[0] == "end") == 6
    # task 1 starts before task 0 has finished: their steps interleave
    assert log.index(("start", 1)) < log.index(("end", 0))
    # a task without any yield finishes inside its admission turn and never counts as in flight
    log.clear()
    Scheduler((make(i, 0) for i in range(3)), max_in_flight=1).run()
    assert [e for e in log if e[0] == "end"] == [("end", 0), ("end", 1), ("end", 2)]
    with pytest.raises(ValueError):
        Scheduler(iter(()), max_in_flight=0)


def test_muon_keller_jordan_single_rank_step(monkeypatch):
    from dion_b200.optim.muon_reference import MuonKellerJordan, zeropower_fixed_coeffs

    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("RANK", "0")
    P = _params([(64, 32), (32, 64)])
    before = [p.detach().clone() for p in P]
    for p in P:
        p.grad = torch.randn_like(p)
    opt = MuonKellerJordan(P, lr=0.05, momentum=0.9, nesterov=True)
    opt.step()
    for p, b in zip(P, before):
        g = p.grad
        upd = g + 0.9 * g                       # momentum buffer starts at zero: buf = g, nesterov adds 0.9 * buf
        u = zeropower_fixed_coeffs(upd, steps=5) * (g.size(0) / g.size(1)) ** 0.5
        want = b - 0.05 * u.to(torch.bfloat16).to(b.dtype)
        torch.testing.assert_close(p.detach(), want, rtol=0, atol=1e-6)
        assert set(opt.state[p].keys()) == {"momentum_buffer"}


def test_muon_state_dict_roundtrip_continues_identically():
    P = _params()
    opt = Muon([dict(params=P[:3]), dict(params=P[3:], algorithm="adamw", lr=0.01)], lr=0.02, nesterov=True)
    grads = [[torch.randn_like(p) for p in P] for _ in range(4)]
    for step in range(2):
        for p, g in zip(P, grads[step]):
            p.grad = g.clone()
        opt.step()
    Q = _clone(P)
    opt2 = Muon([dict(params=Q[:3]), dict(params=Q[3:], algorithm="adamw", lr=0.01)], lr=0.02, nesterov=True)
    opt2.load_state_dict(copy.deepcopy(opt.state_dict()))
    for step in range(2, 4):
        for p, q, g in zip(P, Q, grads[step]):
            p.grad = g.clone()
            q.grad = g.clone()
        opt.step()
        opt2.step()
    for p, q in zip(P, Q):
        torch.testing.assert_close(p, q, rtol=0, atol=0)


def _with_condition(k, m=192, n=96, batch=2):
    out = []
    for _ in range(batch):
        U = torch.linalg.qr(torch.randn(m, n))[0]
        V = torch.linalg.qr(torch.randn(n, n))[0]
        out.append((U * torch.logspace(0, -k, n)) @ V)
    return torch.stack(out)


def _orth_err(X):
    G = X.transpose(-1, -2) @ X
    return (G - torch.eye(G.shape[-1])).abs().max().item()


def test_orthonormalisation_of_ill_conditioned_batches():
    from dion_b200.optim.orthogonalize import orthonormalize_many

    torch.manual_seed(0)
    easy, hard = _with_condition(2), _with_condition(5)
    # well conditioned: both treatments agree and report nothing
    infos = []
    a = orthonormalize_many([easy], infos=infos)[0]
    assert int(infos[0].sum()) == 0 and _orth_err(a) < 1e-5
    infos = []
    b = orthonormalize_many([easy], robust=[True], infos=infos)[0]
    assert int(infos[0].sum()) == 0
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    # condition 1e5: the plain path gives up on pivots, says so, and degrades to unit or dropped columns
    infos = []
    c = orthonormalize_many([hard], infos=infos)[0]
    assert (infos[0] > 0).all()
    assert torch.isfinite(c).all()
    norms = c.norm(dim=-2)
    assert ((norms - 1).abs() < 1e-3).logical_or(norms == 0).all(), norms
    # ... the shifted two-pass treatment orthonormalises it, and reports that it is still needed
    infos = []
    d = orthonormalize_many([hard], robust=[True], infos=infos)[0]
    assert _orth_err(d) < 1e-4 and (infos[0] > 0).all()
    Q, _ = torch.linalg.qr(hard.double())
    assert (d.double().abs() - Q.abs()).abs().max() < 5e-2          # the basis of a QR factorisation, up to signs
    # mixed request: only the flagged batch takes the second pass, the other result is unchanged
    e, f = orthonormalize_many([easy, hard], robust=[False, True])
    torch.testing.assert_close(e, a, rtol=0, atol=0)
    torch.testing.assert_close(f, d, rtol=0, atol=0)


def test_dion_survives_rank_deficient_momentum_and_switches_treatment():
    torch.manual_seed(0)
    P = _params([(64, 32), (64, 32), (48, 48)])
    before = [p.detach().clone() for p in P]
    opt = Dion(P, lr=0.02, rank_fraction=1.0, weight_decay=0.0)
    grads = [torch.randn(p.shape[0], 2) @ torch.randn(2, p.shape[1]) for p in P]   # rank 2, every step the same
    for _ in range(6):
        for p, g in zip(P, grads):
            p.grad = g.clone()
        opt.step()
        for p in P:
            assert torch.isfinite(p).all()
    assert opt.robust_switches >= 1
    for p, b in zip(P, before):
        r = min(p.shape)
        # six steps of at most lr * sqrt(fan_out / fan_in) * ||P Q^T||_F, with unit columns in P and Q
        bound = 6 * 0.02 * (p.shape[0] / p.shape[1]) ** 0.5 * r
        assert (p.detach() - b).norm() <= bound
    for st in opt.state.values():
        assert torch.isfinite(st["Q"]).all() and torch.isfinite(st["momentum"]).all()
        assert (st["Q"].norm(dim=0) > 0).all()        # no column of Q has died


def _structured_run(opt_cls, device, steps=24, **kw):
    from dion_b200.models import GPT, GPTConfig

    torch.manual_seed(0)
    m = GPT(GPTConfig(sequence_len=64, vocab_size=512, n_layer=2, n_head=4, n_embd=64))
    m.init_weights()
    m = m.to(device)
    groups = [dict(params=list(m.transformer.h.parameters())),
              dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()), algorithm="lion",
                   lr=0.002)]
    opt = opt_cls(groups, lr=0.02, rank_fraction=1.0, **kw)
    base = (torch.arange(65) * 7) % 23
    losses = []
    for s in range(steps):
        x = torch.stack([(base + i + s) % 23 for i in range(8)]).to(device)
        loss = m(x[:, :-1].contiguous(), x[:, 1:].contiguous())
        loss.backward()
        opt.step()
        m.zero_grad(set_to_none=True)
        losses.append(loss.item())
    return losses, opt


def test_dion_trains_on_structured_data_like_the_qr_oracle():
    """Periodic token sequences give low-rank gradients, so P = M Q is ill conditioned from the first
    step on - the regime in which a plain Cholesky-QR breaks down.  The loss must follow the oracle that
    orthonormalises with Householder QR."""
    ours, opt = _structured_run(Dion, "cpu")
    oracle, _ = _structured_run(DionReference, "cpu", qr_method="qr")
    assert opt.robust_switches >= 1
    assert ours[-1] < 0.5 and oracle[-1] < 0.5
    for a, b in zip(ours[4:], oracle[4:]):
        assert abs(a - b) < 0.05 * max(b, 0.1), (ours, oracle)


@pytest.mark.gpu
def test_dion_trains_on_structured_data_gpu():
    """The same regime through the CUDA kernels (bf16 activations): the ill-conditioned treatment comes
    on and the loss falls like the oracle's."""
    ours, opt = _structured_run(Dion, "cuda")
    oracle, _ = _structured_run(DionReference, "cuda", qr_method="qr")
    assert opt.robust_switches >= 1
    assert all(l == l for l in ours)
    assert ours[-1] < 0.6 and oracle[-1] < 0.6, (ours, oracle)
    assert abs(ours[-1] - oracle[-1]) < 0.25 * max(oracle[-1], 0.2), (ours, oracle)


def _groups(mats, emb, head):
    return [dict(params=mats),
            dict(params=[emb], algorithm="lion", lr=0.002, weight_decay=0.0),
            dict(params=[head], algorithm="adamw", lr=0.003, weight_decay=0.01)]


@needs_ref
@pytest.mark.parametrize("direction", ["reference_to_ours", "ours_to_reference"])
@pytest.mark.parametrize("kind", ["dion", "muon"])
def test_optimizer_state_dicts_interchange_with_the_reference(kind, direction):
    """A state_dict written by the reference's optimizer loads into this package's optimizer (and the other way
    round) and training continues as if nothing had happened: same keys, same tensors, same group entries."""
    torch.manual_seed(11)
    shapes = [(48, 32), (32, 48), (48, 32)]
    base = [torch.randn(s) for s in shapes] + [torch.randn(50, 16), torch.randn(16, 50)]

    def build(module, which):
        ps = [torch.nn.Parameter(t.clone()) for t in base]
        groups = _groups(ps[:3], ps[3], ps[4])
        if which == "dion":
            opt = module.Dion(groups, lr=0.02, rank_fraction=0.5, weight_decay=0.05)
        else:
            opt = module.Muon(groups, lr=0.02, mu=0.95, weight_decay=0.05, nesterov=True, adjust_lr="spectral_norm")
        return ps, opt

    def run(ps, opt, steps, seed):
        g = torch.Generator().manual_seed(seed)
        for _ in range(steps):
            for p in ps:
                p.grad = torch.randn(p.shape, generator=g)
            opt.step()

    src_mod, dst_mod = (ref, dion_b200) if direction == "reference_to_ours" else (dion_b200, ref)
    # the writer trains three steps and keeps going; the reader loads the writer's state and takes the same steps
    ps_w, opt_w = build(src_mod, kind)
    run(ps_w, opt_w, 3, seed=1)
    sd = copy.deepcopy(opt_w.state_dict())
    ps_r, opt_r = build(dst_mod, kind)
    with torch.no_grad():
        for a, b in zip(ps_r, ps_w):
            a.copy_(b)
    opt_r.load_state_dict(sd)
    assert opt_r.state_dict()["param_groups"][0].keys() == sd["param_groups"][0].keys()
    for sw, sr in zip(sd["state"].values(), opt_r.state_dict()["state"].values()):
        assert sw.keys() == sr.keys()
    run(ps_w, opt_w, 2, seed=2)
    run(ps_r, opt_r, 2, seed=2)
    tol = dict(rtol=2e-3, atol=2e-4) if kind == "dion" else dict(rtol=2e-2, atol=2e-3)   # Muon: bf16 Newton-Schulz
    for a, b in zip(ps_w, ps_r):
        torch.testing.assert_close(a, b, **tol)


@needs_ref
@pytest.mark.parametrize("missing", [False, True])
def test_dion_edge_cases_follow_the_reference(missing):
    """Parameters without a gradient in some steps, an all-zero gradient, and groups that override the learning
    rate, rank fraction and weight decay for matrices of the same shape."""
    torch.manual_seed(0)
    P = [torch.nn.Parameter(torch.randn(32, 16)) for _ in range(4)] + [torch.nn.Parameter(torch.randn(16, 32)) for _ in range(2)]
    A, B = _clone(P), _clone(P)
    groups = lambda ps: [dict(params=ps[:3]), dict(params=ps[3:], lr=0.005, rank_fraction=0.25, weight_decay=0.0)]
    oa = Dion(groups(A), lr=0.02, rank_fraction=0.5, rank_multiple_of=1)
    ob = ref.DionReference(groups(B), lr=0.02, rank_fraction=0.5, rank_multiple_of=1, qr_method="qr")
    _inject_q(oa, ob, A, B)
    for step in range(3):
        gen = torch.Generator().manual_seed(step)
        for i, (p, q) in enumerate(zip(A, B)):
            if missing and (i + step) % 3 == 0:
                p.grad = q.grad = None
                continue
            g = torch.zeros(p.shape) if i == 1 else torch.randn(p.shape, generator=gen)
            p.grad, q.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for p, q in zip(A, B):
        assert torch.isfinite(p).all()
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


@needs_ref
@pytest.mark.parametrize("kw", [dict(nesterov=False, adjust_lr="spectral_norm", flatten=True),
                                dict(nesterov=True, adjust_lr="rms_norm", flatten=True),
                                dict(nesterov=True, adjust_lr=None, flatten=False),
                                dict(nesterov=True, adjust_lr="keller_muon", flatten=True)])
def test_muon_options_follow_the_reference_on_higher_rank_parameters(kw):
    """Convolution-shaped (4-D) and batched (3-D) parameters with and without `flatten`, every learning-rate
    scaling, parameters without a gradient in some steps."""
    torch.manual_seed(0)
    P = ([torch.nn.Parameter(torch.randn(32, 16)) for _ in range(3)] + [torch.nn.Parameter(torch.randn(8, 4, 3, 3))]
         + [torch.nn.Parameter(torch.randn(2, 16, 8))])
    A, B = _clone(P), _clone(P)
    oa = Muon(A, lr=0.02, weight_decay=0.05, **kw)
    ob = ref.Muon(B, lr=0.02, weight_decay=0.05, use_triton=False, **kw)
    for step in range(3):
        gen = torch.Generator().manual_seed(step)
        for i, (p, q) in enumerate(zip(A, B)):
            if (i + step) % 4 == 0:
                p.grad = q.grad = None
                continue
            g = torch.randn(p.shape, generator=gen)
            p.grad, q.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for p, q in zip(A, B):
        torch.testing.assert_close(p, q, rtol=2e-3, atol=2e-4)
