"""Batched Cholesky-inverse kernel and column norms against PyTorch references."""
import pytest
import torch

from dion_b200 import ops


def _gram(batch, m, r, device, cond=None):
    P = torch.randn(batch, m, r, device=device)
    if cond is not None:
        scale = torch.logspace(0, -cond, r, device=device)
        P = P * scale
    return P, P.transpose(-1, -2) @ P


def test_chol_inverse_reference_orthonormalises_cpu():
    P, G = _gram(2, 64, 24, "cpu", cond=2)
    Z, info = ops.chol_inverse(G)
    Q = P @ Z.transpose(-1, -2)
    eye = torch.eye(24).expand(2, 24, 24)
    assert (Q.transpose(-1, -2) @ Q - eye).abs().max() < 1e-3
    assert int(info.sum()) == 0
    # same basis as Householder QR up to column signs
    Qh, _ = torch.linalg.qr(P)
    assert ((Q.abs() - Qh.abs()).abs().max()) < 1e-3


def test_chol_inverse_reference_zero_matrix_cpu():
    Z, info = ops.chol_inverse(torch.zeros(1, 8, 8))
    assert torch.isfinite(Z).all()
    assert int(info[0]) == 8


@pytest.mark.gpu
@pytest.mark.parametrize("r", [32, 96, 192, 200, 768, 1024])
def test_chol_inverse_kernel(r):
    batch = 3
    P, G = _gram(batch, 4 * r, r, "cuda", cond=1.5)
    Z, info = ops.chol_inverse(G)
    torch.cuda.synchronize()
    assert int(info.sum()) == 0
    assert torch.equal(Z, torch.tril(Z))
    Q = P @ Z.transpose(-1, -2)
    eye = torch.eye(r, device="cuda")
    err = (Q.transpose(-1, -2) @ Q - eye).abs().max().item()
    assert err < 5e-3, err
    Zr, _ = ops.chol_inverse_reference(G.double())
    rel = ((Z.double() - Zr.double()).norm() / Zr.double().norm()).item()
    assert rel < 1e-2, rel


@pytest.mark.gpu
@pytest.mark.parametrize("r,batch", [(768, 80), (200, 7)])
def test_chol_inverse_kernel_is_deterministic(r, batch):
    """The two CTAs that share a matrix exchange their updates through global memory; whichever of them
    runs ahead, the result must be the same to the last bit.  More matrices than CTA pairs fit on the
    GPU, a second stream keeping the SMs busy, and a comparison with the single-CTA kernel's accuracy."""
    P, G = _gram(batch, 2 * r, r, "cuda", cond=1.0)
    Z0, _ = ops.chol_inverse(G)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    noise = torch.randn(4096, 4096, device="cuda")
    for _ in range(3):
        with torch.cuda.stream(side):
            for _ in range(4):
                noise = noise @ noise * 1e-3
        Z, _ = ops.chol_inverse(G)
        torch.cuda.synchronize()
        assert torch.equal(Z, Z0)
    Zr, _ = ops.chol_inverse_reference(G[:2].double())
    rel = ((Z0[:2].double() - Zr.double()).norm() / Zr.double().norm()).item()
    assert rel < 1e-2, rel


@pytest.mark.gpu
def test_chol_inverse_kernel_rank_deficient_and_zero():
    P = torch.randn(2, 512, 64, device="cuda")
    P[0, :, 10] = 0          # a zero column
    P[0, :, 20] = P[0, :, 5]  # a duplicated column
    P[1] = 0                 # an all-zero matrix
    G = P.transpose(-1, -2) @ P
    Z, info = ops.chol_inverse(G)
    assert torch.isfinite(Z).all()
    assert int(info[0]) >= 2 and int(info[1]) == 64
    Q = P @ Z.transpose(-1, -2)
    assert torch.isfinite(Q).all()
    assert Q[1].abs().max() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_col_sumsq_kernel(dtype):
    X = torch.randn(5, 333, 200, device="cuda").to(dtype)
    out = ops.col_sumsq(X)
    torch.testing.assert_close(out, X.float().square().sum(-2), rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
def test_split_tf32_and_refine_prep_match_torch():
    from dion_b200.ops.linalg import refine_prep, split_tf32

    x = torch.randn(3, 130, 77, device="cuda") * 10
    hi, lo = split_tf32(x)
    ref_hi = (x.view(torch.int32) & -8192).view(torch.float32)
    assert torch.equal(hi, ref_hi) and torch.equal(lo, x - ref_hi)
    a = torch.randn(5, 200, 72, device="cuda")
    a[2, :, 7] = 0  # a vanishing column: d = 0, its row and column of C are zero
    G = a.transpose(1, 2) @ a
    C, d = refine_prep(G)
    Cr, dr = refine_prep(G.cpu())
    torch.testing.assert_close(d.cpu(), dr, rtol=1e-5, atol=0)
    torch.testing.assert_close(C.cpu(), Cr, rtol=1e-5, atol=1e-7)
    assert d[2, 7] == 0 and C[2, 7].abs().max() == 0 and C[2, :, 7].abs().max() == 0


@pytest.mark.gpu
def test_orthonormalisation_of_ill_conditioned_batch_gpu():
    """Condition number 1e5: the plain path reports the pivots it gave up on and returns bounded columns,
    the shifted two-pass treatment orthonormalises."""
    from dion_b200.optim.orthogonalize import orthonormalize_many

    torch.manual_seed(0)
    m, n = 512, 256
    U = torch.linalg.qr(torch.randn(2, m, n, device="cuda"))[0]
    V = torch.linalg.qr(torch.randn(2, n, n, device="cuda"))[0]
    P = (U * torch.logspace(0, -5, n, device="cuda")) @ V
    infos = []
    X = orthonormalize_many([P], infos=infos)[0]
    assert (infos[0] > 0).all()
    assert torch.isfinite(X).all() and X.norm(dim=-2).max() < 1.5
    infos = []
    Y = orthonormalize_many([P], robust=[True], infos=infos)[0]
    eye = torch.eye(n, device="cuda")
    assert (Y.transpose(-1, -2) @ Y - eye).abs().max() < 1e-3
    assert (infos[0] > 0).all()


def _refine_prep_case(device):
    G = torch.randn(3, 40, 40, device=device)
    G = G @ G.transpose(-1, -2) + 40 * torch.eye(40, device=device)
    G[1, 5, 5] = 1e-9      # a dead column: d = 0 there
    skip = torch.tensor([0, 0, 1], dtype=torch.int32, device=device)
    C, d = ops.refine_prep(G, 1e-4, skip)
    C2, d2 = ops.refine_prep(G, 1e-4, skip, fold=True)
    torch.testing.assert_close(d2, d)
    torch.testing.assert_close(C2, C * d.unsqueeze(-2))
    assert d[1, 5] == 0 and (C[2] == 0).all() and torch.equal(C, torch.tril(C, -1))
    return C, d


def test_refine_prep_fold_cpu():
    _refine_prep_case("cpu")


@pytest.mark.gpu
def test_refine_prep_kernel_with_folded_column_scale():
    C, d = _refine_prep_case("cuda")
    Cr, dr = _refine_prep_case("cpu")


def _blocked_case(device, r, block):
    torch.manual_seed(r)
    P = torch.randn(3, 3 * r, r, device=device) * torch.logspace(0, -1.5, r, device=device)
    P[0, :, 10] = 0               # a zero column
    P[0, :, r - 7] = P[0, :, 5]   # a duplicated column, in a later block than its twin
    P[2] = 0                      # an all-zero matrix
    G = P.transpose(-1, -2) @ P if device == "cpu" else (P.double().transpose(-1, -2) @ P.double()).float()
    Zr, info_r = ops.chol_inverse_reference(G.cpu())
    Zb, info_b = ops.linalg.chol_inverse_blocked(G, block=block)
    assert torch.equal(Zb, torch.tril(Zb)) and torch.isfinite(Zb).all()
    if device == "cpu":
        assert info_b.tolist() == info_r.tolist()
        rel = ((Zb - Zr).norm() / Zr.norm()).item()
        assert rel < 1e-5, rel
    else:
        # The trailing updates run as 3xTF32 products, whose rounding noise (a few 1e-6 of the unit diagonal)
        # may leave the twin of a duplicated column a pivot just above the floor: such a column then carries
        # a bounded noise direction instead of being dropped, and the count is one lower.
        got, want = info_b.cpu().tolist(), info_r.tolist()
        assert got[1:] == want[1:] and got[0] in (want[0], want[0] - 1), (got, want)
        rel = ((Zb[1].cpu() - Zr[1]).norm() / Zr[1].norm()).item()
        assert rel < 1e-4, rel
    Q = P[1].double() @ Zb[1].double().T
    err = (Q.T @ Q - torch.eye(r, device=device, dtype=torch.float64)).abs().max().item()
    assert err < 1e-4, err


@pytest.mark.parametrize("r,block", [(96, 32), (200, 64), (130, 64)])
def test_chol_inverse_blocked_matches_the_unblocked_reference_cpu(r, block):
    _blocked_case("cpu", r, block)


@pytest.mark.gpu
@pytest.mark.parametrize("r,block", [(520, 256), (768, 256), (1024, 256), (384, 128)])
def test_chol_inverse_blocked_kernels(r, block):
    """Diagonal blocks through the Cholesky-inverse kernel, everything else as 3xTF32 tensor-core products."""
    _blocked_case("cuda", r, block)


@pytest.mark.gpu
def test_chol_inverse_takes_the_blocked_path_for_large_ranks():
    P, G = _gram(4, 1536, 768, "cuda", cond=1.5)
    n0 = ops.launch_count()
    Z, info = ops.chol_inverse(G)
    assert ops.launch_count() - n0 > 5            # several kernels, not the one-launch factorisation
    Zr, _ = ops.chol_inverse_reference(G.double())
    assert ((Z.double() - Zr.double()).norm() / Zr.double().norm()).item() < 1e-4
    assert int(info.sum()) == 0
