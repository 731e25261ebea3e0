"""Kernels that fuse Dion's reductions with the arithmetic after them, against PyTorch statements of the
same operations (CPU: the statements themselves through the front ends; GPU: the kernels)."""
import pytest
import torch

from dion_b200 import ops


def _case(device, dtype, B=5, n=70, r=45, m=52, nslots=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    slots = torch.randn(nslots, B, n, r, generator=g).to(device)
    Qm = torch.randn(B, n, r, generator=g).to(device=device, dtype=dtype)
    P = torch.randn(B, m, r, generator=g).to(device=device, dtype=dtype)
    nonzero = torch.ones(B, dtype=torch.int32, device=device)
    nonzero[1] = 0                       # an all-zero momentum: R <- previous Q, P <- 0
    slots[0, 2, 3, 4] = float("nan")     # NaN and inf are replaced
    slots[1, 2, 5, 6] = float("inf")
    P[3, 7, 8] = float("nan")
    slots[:, 4, :, 9] = 0.0              # a zero column keeps its previous Q
    return slots, Qm, P, nonzero


def _run(device, dtype, finish, qs_cols, qs_col0, r=45):
    slots, Qm, P, nonzero = _case(device, dtype, r=r)
    nsl, B, n, r = slots.shape
    scale, eps = 0.5, 1e-8
    Rr, Pr, ssr, Qr = ops.dion_r_post_reference(slots, scale, nonzero, Qm, P.clone(), eps, finish=True)
    R32 = torch.empty(B, n, r, device=device)
    Rm = torch.empty(B, n, r, device=device, dtype=dtype)
    ss = torch.empty(B, r, device=device)
    Qn = torch.full((B, n, r), -7.0, device=device, dtype=dtype)
    Qs = torch.full((B, n, qs_cols), -7.0, device=device, dtype=torch.float32)
    Pw = P.clone()
    ops.dion_r_post(slots, scale, nonzero, Qm, Pw, R32, Rm, ss, finish, eps, Qn, Qs, qs_col0)
    if not finish:
        assert (Qn == -7.0).all() and (Qs == -7.0).all()
        ops.dion_q_norm(R32, ss, Qm, eps, Qn, Qs, qs_col0)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    big = Rr.abs() > 1e30   # the inf that became the largest finite number
    torch.testing.assert_close(R32.masked_fill(big, 0), Rr.masked_fill(big, 0), rtol=1e-5, atol=1e-5)
    assert (R32[big] > 1e30).all()
    torch.testing.assert_close(Rm.float().masked_fill(big, 0), Rr.masked_fill(big, 0), rtol=tol, atol=tol)
    torch.testing.assert_close(Pw.float(), Pr.float(), rtol=0, atol=0)
    col_big = big.any(dim=1)
    torch.testing.assert_close(ss.masked_fill(col_big, 0), ssr.masked_fill(col_big, 0), rtol=1e-4, atol=1e-4)
    Qr = Qr.masked_fill(col_big.unsqueeze(1), 0)
    torch.testing.assert_close(Qn.float().masked_fill(col_big.unsqueeze(1), 0), Qr, rtol=tol, atol=tol)
    torch.testing.assert_close(Qs.masked_fill(col_big.unsqueeze(1)[:, :, qs_col0:qs_col0 + qs_cols], 0),
                               Qr[:, :, qs_col0:qs_col0 + qs_cols], rtol=tol, atol=tol)
    # the all-zero matrix kept (a normalised copy of) its previous Q, the zero column its previous values
    assert (Pw[1] == 0).all()
    torch.testing.assert_close(Qn[4, :, 9].float(), Qm[4, :, 9].float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("finish", [True, False])
def test_r_post_front_end_cpu(finish):
    _run("cpu", torch.float32, finish, qs_cols=15, qs_col0=30)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("finish,qs_cols,qs_col0", [(True, 45, 0), (True, 15, 30), (False, 15, 15), (False, 45, 0)])
def test_r_post_kernel(dtype, finish, qs_cols, qs_col0):
    _run("cuda", dtype, finish, qs_cols, qs_col0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("finish,qs_cols,qs_col0,r", [(True, 200, 0, 200), (True, 48, 96, 192), (False, 64, 64, 192),
                                                      (False, 136, 0, 136), (True, 16, 20, 48)])
def test_r_post_kernel_wide_strips(dtype, finish, qs_cols, qs_col0, r):
    """Ranks that are multiples of four take the 128-column strips with 16-byte accesses (several strips,
    a ragged last one, and a Q slice whose offset is not a multiple of four, which falls back)."""
    _run("cuda", dtype, finish, qs_cols, qs_col0, r=r)


@pytest.mark.gpu
def test_r_post_kernel_may_write_the_new_q_over_the_previous_one():
    """Qs may be the very tensor Qm is (no tensor parallelism, same dtype): every element is read before
    the thread that owns it overwrites it."""
    slots, Qm, P, nonzero = _case("cuda", torch.float32)
    _, _, _, Qr = ops.dion_r_post_reference(slots, 1.0, nonzero, Qm, None, 1e-8)
    Q = Qm.clone()
    ops.dion_r_post(slots, 1.0, nonzero, Q, None, None, None, None, True, 1e-8, None, Q, 0)
    ok = ~torch.isnan(Qr) & (Qr.abs() < 1e30)
    torch.testing.assert_close(Q[ok], Qr[ok], rtol=1e-5, atol=1e-5)


def _slot_reduce_case(device, nslots=4, shape=(3, 40, 24)):
    g = torch.Generator().manual_seed(1)
    slots = torch.randn(nslots, *shape, generator=g).to(device)
    out, hi, lo = (torch.empty(shape, device=device) for _ in range(3))
    ops.slot_reduce(slots, out, hi, lo, [], 0.25)
    want = slots[0].clone()
    for s in range(1, nslots):
        want += slots[s]
    want *= 0.25
    assert torch.equal(out, want)                       # same order of additions: same bits
    assert torch.equal(hi + lo, out)
    assert (hi.view(torch.int32) & 8191).eq(0).all()    # hi is exactly representable in tf32
    # a leading part of every slot (what a rank with fewer matrices than its peers reduces)
    part = torch.empty((2, *shape[1:]), device=device)
    ops.slot_reduce(slots[:, :2], part, None, None, [], 1.0)
    want = slots[0, :2].clone()
    for s in range(1, nslots):
        want += slots[s, :2]
    assert torch.equal(part, want)


def test_slot_reduce_front_end_cpu():
    _slot_reduce_case("cpu")


@pytest.mark.gpu
def test_slot_reduce_kernel():
    _slot_reduce_case("cuda")


@pytest.mark.gpu
def test_slot_reduce_kernel_hands_the_sum_on_to_other_buffers():
    slots = torch.randn(2, 4, 32, 16, device="cuda")
    a, b = torch.zeros(4, 32, 16, device="cuda"), torch.zeros(4, 32, 16, device="cuda")
    ops.slot_reduce(slots, None, None, None, [a.data_ptr(), b.data_ptr()], 1.0)
    assert torch.equal(a, slots[0] + slots[1]) and torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_stores_every_batch_element_to_several_destinations(dtype):
    B, M, N, K, dup = 3, 192, 160, 128, 3
    a = torch.randn(B, M, K, device="cuda").to(dtype)
    b = torch.randn(B, K, N, device="cuda").to(dtype)
    bufs = [torch.zeros(B, M, N, device="cuda") for _ in range(dup)]
    table = torch.tensor([bufs[k][i].data_ptr() for i in range(B) for k in range(dup)], dtype=torch.int64, device="cuda")
    ops.gemm(a, b, out=bufs[0][0], out_ptrs=table, out_dup=dup)
    ref = ops.gemm(a, b, out_dtype=torch.float32)
    for k in range(dup):
        assert torch.equal(bufs[k], ref)
    ops.check_status()
