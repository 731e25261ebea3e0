"""Multi-tensor optimizer kernels against the PyTorch statement of the same update."""
import pytest
import torch

from dion_b200 import ops

SHAPES = [(768, 768), (50, 77), (3, 5), (1, 1), (4099,), (128, 96)]


def _lists(device, dtype=torch.float32, n=None):
    shapes = SHAPES if n is None else (SHAPES * ((n + len(SHAPES) - 1) // len(SHAPES)))[:n]
    return [torch.randn(s, device=device).to(dtype) for s in shapes]


def test_adamw_reference_matches_torch_adamw_cpu():
    x = [torch.randn(7, 5)]
    g = [torch.randn(7, 5)]
    p = torch.nn.Parameter(x[0].clone())
    p.grad = g[0].clone()
    opt = torch.optim.AdamW([p], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    m, v = [torch.zeros(7, 5)], [torch.zeros(7, 5)]
    for step in (1, 2, 3):
        opt.step()
        ops.adamw_update(x, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1, step=step, epsilon=1e-8)
    torch.testing.assert_close(x[0], p.data, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_adamw_kernel(state_dtype, grad_dtype):
    X = _lists("cuda", n=50)
    G = [g.to(grad_dtype) for g in _lists("cuda", n=50)]
    M = [m.to(state_dtype) * 0.1 for m in _lists("cuda", n=50)]
    V = [v.abs().to(state_dtype) * 0.1 for v in _lists("cuda", n=50)]
    S = [torch.empty_like(x, dtype=torch.bfloat16) for x in X]
    Xr, Mr, Vr = [x.clone() for x in X], [m.clone() for m in M], [v.clone() for v in V]
    kw = dict(lr=3e-3, beta1=0.9, beta2=0.95, weight_decay=0.01, step=3, epsilon=1e-8)
    ops.adamw_update(X, G, M, V, shadow=S, **kw)
    ops.adamw_update_reference(Xr, G, Mr, Vr, **kw)
    tol = dict(rtol=1e-5, atol=1e-6) if state_dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
    for a, b in zip(X, Xr):
        torch.testing.assert_close(a, b, **(dict(rtol=1e-4, atol=1e-5) if state_dtype == torch.float32 else tol))
    for a, b in zip(M, Mr):
        torch.testing.assert_close(a, b, **tol)
    for a, b in zip(V, Vr):
        torch.testing.assert_close(a, b, **tol)
    for s, x in zip(S, X):
        assert torch.equal(s, x.to(torch.bfloat16))


@pytest.mark.gpu
@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_lion_kernel(state_dtype):
    X = _lists("cuda", n=45)
    G = _lists("cuda", n=45)
    M = [m.to(state_dtype) for m in _lists("cuda", n=45)]
    Xr, Mr = [x.clone() for x in X], [m.clone() for m in M]
    kw = dict(lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.1)
    ops.lion_update(X, G, M, **kw)
    ops.lion_update_reference(Xr, G, Mr, **kw)
    for a, b in zip(M, Mr):
        torch.testing.assert_close(a, b, rtol=1e-2 if state_dtype == torch.bfloat16 else 1e-6, atol=1e-2 if state_dtype == torch.bfloat16 else 1e-6)
    # sign() may flip where the interpolated value is within rounding of zero
    for a, b in zip(X, Xr):
        frac = ((a - b).abs() > 1e-6).float().mean().item()
        assert frac < 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("nesterov", [False, True])
def test_muon_momentum_and_apply_kernels(nesterov):
    G = _lists("cuda", n=44)
    M = _lists("cuda", n=44)
    Mr = [m.clone() for m in M]
    ss = torch.zeros(len(G), device="cuda")
    U = ops.muon_momentum(G, M, mu=0.95, nesterov=nesterov, sumsq=ss)
    for g, m, mr, u, s in zip(G, M, Mr, U, ss):
        mr.mul_(0.95).add_(g)
        ur = (mr * 0.95 + g) if nesterov else mr
        torch.testing.assert_close(m, mr, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(u.float(), ur.bfloat16().float(), rtol=1e-2, atol=1e-6)
        torch.testing.assert_close(s, u.float().square().sum(), rtol=1e-4, atol=1e-6)
    X = _lists("cuda", n=44)
    Xr = [x.clone() for x in X]
    S = [torch.empty_like(x, dtype=torch.bfloat16) for x in X]
    ops.muon_apply(X, U, decay=0.999, step=0.02, shadow=S)
    for x, xr, u, s in zip(X, Xr, U, S):
        torch.testing.assert_close(x, xr * 0.999 - 0.02 * u.float(), rtol=1e-6, atol=1e-6)
        assert torch.equal(s, x.to(torch.bfloat16))


@pytest.mark.gpu
@pytest.mark.parametrize("m_dtype", [torch.float32, torch.bfloat16])
def test_dion_accumulate_kernel(m_dtype):
    G = _lists("cuda", n=43)
    M = [m.to(m_dtype) for m in _lists("cuda", n=43)]
    M[3].zero_(); G[3].zero_()
    Mr = [m.clone() for m in M]
    nz = torch.zeros(len(G), dtype=torch.int32, device="cuda")
    ops.dion_accumulate(G, M, nz)
    for i, (g, m, mr) in enumerate(zip(G, M, Mr)):
        torch.testing.assert_close(m, (mr.float() + g).to(m_dtype))
        assert int(nz[i]) == (0 if i == 3 else 1)


@pytest.mark.gpu
def test_cast_copy_kernel():
    src = _lists("cuda", n=41)
    dst = [torch.empty_like(s, dtype=torch.bfloat16) for s in src]
    ops.cast_copy(src, dst)
    for s, d in zip(src, dst):
        assert torch.equal(d, s.to(torch.bfloat16))
