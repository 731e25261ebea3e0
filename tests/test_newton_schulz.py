"""Newton-Schulz orthogonalisation: the tcgen05 path (symmetric X X^T tiles, fused b A + c A A and
a X + B X epilogues) against the plain PyTorch iteration of the same coefficients, as the reference
checks its Triton kernels against torch (tests/test_newton_shultz.py)."""
import pytest
import torch

from dion_b200.optim.newton_schulz import NS_COEFFS, newton_schulz, newton_schulz_torch


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_torch_iteration_orthogonalises_on_cpu():
    torch.manual_seed(0)
    for shape in [(48, 96), (96, 48), (3, 64, 64)]:
        X = newton_schulz_torch(torch.randn(shape)).float()
        m = min(shape[-2:])
        gram = X @ X.transpose(-1, -2) if shape[-2] <= shape[-1] else X.transpose(-1, -2) @ X
        # the quintic iteration drives singular values into a band around 1, not to 1 exactly
        assert (gram - torch.eye(m)).abs().max() < 0.45
    assert len(NS_COEFFS) == 5 and all(len(c) == 3 for c in NS_COEFFS)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(768, 768), (768, 3072), (3072, 768), (4, 256, 512), (3, 512, 256), (2, 200, 328)])
def test_kernel_matches_torch_iteration(shape):
    torch.manual_seed(1)
    G = torch.randn(shape, device="cuda")
    ours = newton_schulz(G)
    ref = newton_schulz_torch(G)
    assert ours.shape == G.shape and ours.dtype == torch.bfloat16
    # both run five bf16 iterations; rounding differs, the result agrees to bf16 accuracy
    assert _rel(ours, ref) < 3e-2
    # and it is an approximate orthogonal factor
    X = ours.float()
    small_first = shape[-2] <= shape[-1]
    gram = X @ X.transpose(-1, -2) if small_first else X.transpose(-1, -2) @ X
    eye = torch.eye(gram.shape[-1], device="cuda")
    assert (gram - eye).abs().max() < 0.5


@pytest.mark.gpu
def test_kernel_handles_zero_and_tiny_inputs():
    Z = torch.zeros(2, 128, 256, device="cuda")
    out = newton_schulz(Z)
    assert torch.isfinite(out).all() and out.abs().max() == 0
    T = torch.randn(128, 256, device="cuda") * 1e-20
    assert torch.isfinite(newton_schulz(T)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n", [(256, 256), (256, 1024), (200, 328)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_symmetric_gram_and_poly_match_torch(m, n, dtype):
    from dion_b200.optim.newton_schulz import ns_line_1, ns_line_2

    tol = 5e-2
    for batch in (None, 4):
        shape = (m, n) if batch is None else (batch, m, n)
        A = torch.randn(shape, dtype=dtype, device="cuda")
        got, want = ns_line_1(A), A @ A.mT
        assert got.dtype == dtype and got.shape == want.shape
        assert (got.float() - want.float()).abs().max() <= tol * want.float().abs().max()
        S = torch.randn(shape[:-1] + (m,), dtype=dtype, device="cuda")
        S = (S + S.mT) / 2
        alpha, beta = 0.7, -1.3
        got, want = ns_line_2(S, alpha, beta), alpha * (S @ S.mT) + beta * S
        assert (got.float() - want.float()).abs().max() <= tol * want.float().abs().max()


def test_symmetric_helpers_on_cpu():
    from dion_b200.optim.newton_schulz import ns_line_1, ns_line_2

    A = torch.randn(3, 16, 24)
    torch.testing.assert_close(ns_line_1(A), A @ A.mT)
    S = torch.randn(16, 16)
    S = S + S.T
    torch.testing.assert_close(ns_line_2(S, 0.5, 2.0), 0.5 * (S @ S.T) + 2.0 * S)
