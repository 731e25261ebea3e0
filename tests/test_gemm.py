"""tcgen05 GEMM against a plain fp32 PyTorch reference of the same op."""
import pytest
import torch

from dion_b200.ops.gemm import gemm


def _operand(rows, cols, dtype, transposed, batch=None, device="cuda"):
    """Logical [rows, cols] matrix, stored row-major or as the transpose of a row-major one."""
    shape = (cols, rows) if transposed else (rows, cols)
    if batch is not None:
        shape = (batch, *shape)
    t = torch.randn(shape, device=device, dtype=torch.float32).to(dtype)
    return t.transpose(-1, -2) if transposed else t


def _rel_err(x, ref):
    return ((x.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-20)).item()


def test_reference_semantics_cpu():
    a = torch.randn(5, 7)
    b = torch.randn(7, 3)
    c = torch.randn(5, 3)
    out = gemm(a, b, c=c, alpha=0.5, beta=2.0)
    torch.testing.assert_close(out, 0.5 * a @ b + 2.0 * c)
    out2 = torch.ones(5, 3)
    gemm(a, b, out=out2, accumulate=True)
    torch.testing.assert_close(out2, 1 + a @ b)
    out3 = gemm(a, b, act="relu2")
    torch.testing.assert_close(out3, torch.relu(a @ b) ** 2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape", [(256, 256, 256), (384, 200, 328), (128, 64, 64), (1000, 520, 72)])
def test_gemm_layouts(dtype, ta, tb, shape):
    M, N, K = shape
    a = _operand(M, K, dtype, ta)
    b = _operand(K, N, dtype, tb)
    out = gemm(a, b, out_dtype=torch.float32)
    ref = a.float() @ b.float()
    tol = 2e-5 if dtype == torch.bfloat16 else 4e-3
    assert _rel_err(out, ref) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_block_n_and_batch(block_n, dtype):
    a = _operand(300, 192, dtype, False, batch=3)
    b = _operand(192, 520, dtype, True, batch=3)
    out = gemm(a, b, out_dtype=torch.float32, block_n=block_n)
    ref = torch.matmul(a.float(), b.float())
    assert _rel_err(out, ref) < (2e-5 if dtype == torch.bfloat16 else 4e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_epilogue_alpha_beta(c_dtype, out_dtype):
    a = _operand(520, 256, torch.bfloat16, False)
    b = _operand(256, 392, torch.bfloat16, False)
    c = torch.randn(520, 392, device="cuda").to(c_dtype)
    shadow = torch.empty(520, 392, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, c=c, alpha=-0.25, beta=0.75, out_dtype=out_dtype, shadow=shadow)
    ref = -0.25 * (a.float() @ b.float()) + 0.75 * c.float()
    assert _rel_err(out, ref) < (1e-2 if out_dtype == torch.bfloat16 else 2e-5)
    assert torch.equal(shadow, out.to(torch.bfloat16))


@pytest.mark.gpu
def test_gemm_inplace_accumulate_into_c():
    a = _operand(256, 128, torch.float32, False)
    b = _operand(128, 256, torch.float32, True)
    m = torch.randn(256, 256, device="cuda")
    ref = m - 0.05 * (a @ b)
    gemm(a, b, c=m, out=m, alpha=-0.05, beta=1.0)
    assert _rel_err(m, ref) < 1e-3


@pytest.mark.gpu
def test_gemm_relu2():
    a = _operand(256, 128, torch.bfloat16, False)
    b = _operand(128, 512, torch.bfloat16, True)
    out = gemm(a, b, act="relu2", out_dtype=torch.float32)
    ref = torch.relu(a.float() @ b.float()) ** 2
    assert _rel_err(out, ref) < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_symmetric(dtype):
    x = _operand(640, 328, dtype, False, batch=2)
    out = gemm(x, x.transpose(-1, -2), out_dtype=torch.float32, symmetric=True)
    ref = torch.matmul(x.float(), x.float().transpose(-1, -2))
    assert _rel_err(out, ref) < (2e-5 if dtype == torch.bfloat16 else 4e-3)
    assert torch.equal(out, out.transpose(-1, -2))


@pytest.mark.gpu
@pytest.mark.parametrize("split_k", [1, 3, 8])
def test_gemm_split_k_atomic(split_k):
    a = _operand(256, 4096, torch.bfloat16, True)
    b = _operand(4096, 384, torch.bfloat16, False)
    out = torch.ones(256, 384, device="cuda")
    gemm(a, b, out=out, accumulate=True, split_k=split_k, alpha=0.5)
    ref = 1 + 0.5 * (a.float() @ b.float())
    assert _rel_err(out, ref) < 1e-4


@pytest.mark.gpu
def test_gemm_pointer_array_outputs():
    B = 5
    a = _operand(256, 96, torch.float32, False, batch=B)
    b = _operand(96, 384, torch.float32, True, batch=B)
    xs = [torch.randn(256, 384, device="cuda") for _ in range(B)]
    sh = [torch.empty(256, 384, device="cuda", dtype=torch.bfloat16) for _ in range(B)]
    refs = [0.9 * x - 0.1 * (a[i] @ b[i]) for i, x in enumerate(xs)]
    ptrs = torch.tensor([x.data_ptr() for x in xs], dtype=torch.int64, device="cuda")
    sptrs = torch.tensor([x.data_ptr() for x in sh], dtype=torch.int64, device="cuda")
    gemm(a, b, c=xs[0], out=xs[0], c_ptrs=ptrs, out_ptrs=ptrs, shadow=sh[0], shadow_ptrs=sptrs, alpha=-0.1, beta=0.9)
    for x, r, s in zip(xs, refs, sh):
        assert _rel_err(x, r) < 2e-3
        assert torch.equal(s, x.to(torch.bfloat16))


@pytest.mark.gpu
def test_gemm_unaligned_falls_back_to_library():
    a = torch.randn(33, 17, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(17, 9, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, out_dtype=torch.float32)
    assert _rel_err(out, a.float() @ b.float()) < 2e-2


@pytest.mark.gpu
def test_gemm_status_word_stays_clear():
    from dion_b200.ops import runtime

    a = _operand(512, 512, torch.bfloat16, False)
    gemm(a, a)
    runtime.check_status()


@pytest.mark.gpu
def test_gemm_relu2_save_pre_and_backward_multiplier():
    a = _operand(300, 128, torch.bfloat16, False)
    b = _operand(128, 520, torch.bfloat16, True)
    h = torch.empty(300, 520, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty_like(h)
    gemm(a, b, out=h, shadow=pre, act="relu2_save_pre")
    ref_pre = a.float() @ b.float()
    assert _rel_err(pre, ref_pre) < 1e-2
    assert _rel_err(h, torch.relu(ref_pre) ** 2) < 1e-2
    dy = _operand(300, 64, torch.bfloat16, False)
    w = _operand(64, 520, torch.bfloat16, False)
    dpre = torch.empty(300, 520, device="cuda", dtype=torch.bfloat16)
    gemm(dy, w, c=pre, out=dpre, act="mul_relu2_grad")
    ref = (dy.float() @ w.float()) * 2 * torch.relu(pre.float())
    assert _rel_err(dpre, ref) < 1e-2
    # the same multiplier recovered from the stored activation h = relu(pre)^2
    dpre2 = torch.empty_like(dpre)
    gemm(dy, w, c=h, out=dpre2, act="mul_relu2_grad_sq")
    assert _rel_err(dpre2, ref) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape", [(512, 512, 256), (640, 296, 200), (200, 1000, 72)])
def test_gemm_cta_pair_layouts(dtype, ta, tb, shape):
    """256-row tiles computed by two CTAs of a cluster (tcgen05 cta_group::2), forced on small shapes."""
    M, N, K = shape
    a = _operand(M, K, dtype, ta)
    b = _operand(K, N, dtype, tb)
    out = gemm(a, b, out_dtype=torch.float32, pair=1)
    ref = a.float() @ b.float()
    assert _rel_err(out, ref) < (2e-5 if dtype == torch.bfloat16 else 4e-3)


@pytest.mark.gpu
def test_gemm_cta_pair_epilogues_batch_and_many_tiles():
    # batched, with C / alpha / beta and the second output; more tiles than CTA pairs so that the
    # persistent loop and both accumulator buffers wrap around several times
    a = _operand(1100, 320, torch.bfloat16, False, batch=5)
    b = _operand(320, 2100, torch.bfloat16, True, batch=5)
    c = torch.randn(5, 1100, 2100, device="cuda").to(torch.bfloat16)
    shadow = torch.empty(5, 1100, 2100, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, c=c, alpha=0.5, beta=1.0, out_dtype=torch.float32, shadow=shadow, pair=1)
    ref = 0.5 * torch.matmul(a.float(), b.float()) + c.float()
    assert _rel_err(out, ref) < 2e-5
    assert torch.equal(shadow, out.to(torch.bfloat16))
    y = gemm(a, b, act="relu2", pair=1)
    assert _rel_err(y, torch.relu(torch.matmul(a.float(), b.float())) ** 2) < 1e-2
    # split-K accumulation with atomics
    acc = torch.zeros(5, 1100, 2100, device="cuda")
    gemm(a, b, out=acc, accumulate=True, split_k=3, pair=1)
    assert _rel_err(acc, torch.matmul(a.float(), b.float())) < 2e-5


@pytest.mark.gpu
def test_gemm_cta_pair_matches_single_cta_bitwise():
    a = _operand(4096, 768, torch.bfloat16, False)
    b = _operand(768, 3072, torch.bfloat16, True)
    y1 = gemm(a, b, pair=1)
    y0 = gemm(a, b, pair=-1)
    assert torch.equal(y0, y1)


def _split(x):
    hi = (x.contiguous().view(torch.int32) & -8192).view(torch.float32)
    return hi, x - hi


def test_gemm_hi_lo_operands_and_column_scale_cpu():
    a, b, c = torch.randn(2, 9, 12), torch.randn(2, 12, 5), torch.randn(2, 9, 5)
    a_hi, a_lo = _split(a)
    b_hi, b_lo = _split(b)
    out = gemm(a_hi, b_hi, a_lo=a_lo, b_lo=b_lo)
    torch.testing.assert_close(out, a_hi @ b_hi + a_lo @ b_hi + a_hi @ b_lo)
    s = torch.rand(2, 5)
    out = gemm(a, b, c=c, alpha=-1.0, beta=1.0, c_col_scale=s)
    torch.testing.assert_close(out, c * s.unsqueeze(1) - a @ b)


@pytest.mark.gpu
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape,symmetric", [((384, 200, 328), False), ((512, 512, 1000), False), ((256, 256, 520), True)])
def test_gemm_hi_lo_operands_reach_fp32_accuracy_in_one_launch(ta, tb, shape, symmetric):
    """A product of split operands (three K-segments into one accumulator) against fp64: a single tf32
    pass is about 1e-3 off, the three-segment product is close to fp32 rounding."""
    M, N, K = shape
    B = 3
    if symmetric:
        if ta != tb:
            pytest.skip("a symmetric product multiplies an operand with its own transpose")
        x = _operand(M, K, torch.float32, ta, batch=B)
        a, b = x, x.transpose(-1, -2)
    else:
        a = _operand(M, K, torch.float32, ta, batch=B)
        b = _operand(K, N, torch.float32, tb, batch=B)

    def split_like(t):  # halves with the memory layout of t
        base = t.transpose(-1, -2) if t.stride(-1) != 1 else t
        hi, lo = _split(base)
        return (hi.transpose(-1, -2), lo.transpose(-1, -2)) if t.stride(-1) != 1 else (hi, lo)

    a_hi, a_lo = split_like(a)
    b_hi, b_lo = split_like(b)
    ref = a.double() @ b.double()
    one = gemm(a_hi, b_hi, symmetric=symmetric)
    three = gemm(a_hi, b_hi, a_lo=a_lo, b_lo=b_lo, symmetric=symmetric)
    e1, e3 = _rel_err(one, ref), _rel_err(three, ref)
    assert e3 < 2e-5, (e1, e3)
    assert e1 > 10 * e3, (e1, e3)  # the segments really were added
    if symmetric:
        # mirrored tiles are exact copies; inside a diagonal tile the two cross terms of an element and of its
        # mirror image are added in opposite order, which may differ in the last bit
        torch.testing.assert_close(three, three.transpose(-1, -2), rtol=0, atol=2e-6 * ref.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_column_scale_on_the_addend(out_dtype):
    B, M, N, K = 2, 300, 200, 96
    a = torch.randn(B, M, K, device="cuda")
    b = torch.randn(B, K, N, device="cuda") * 0.05
    c = torch.randn(B, M, N, device="cuda")
    s = torch.rand(B, N, device="cuda") + 0.5
    out = gemm(a, b, c=c, alpha=-1.0, beta=1.0, c_col_scale=s, out_dtype=out_dtype)
    ref = c * s.unsqueeze(1) - a @ b
    assert _rel_err(out, ref) < (2e-2 if out_dtype == torch.bfloat16 else 3e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,k,batch", [(1024, 1024, 2), (768, 3072, 6), (520, 1032, 5), (512, 2048, 3)])
def test_gemm_symmetric_long_k_on_cta_pairs_with_staged_mirror(dtype, n, k, batch):
    """Symmetric products with K >= 1024 take 256 x 256 tiles on CTA pairs; off-diagonal tiles are stored a
    second time transposed, through shared memory.  The result must be exactly symmetric and match the
    plain product, also with an addend (b A + c A A) and ragged edges."""
    x = torch.randn(batch, n, k, device="cuda").to(dtype) * 0.05
    out = gemm(x, x.transpose(1, 2), symmetric=True)
    ref = x.float() @ x.float().transpose(1, 2)
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
    assert _rel_err(out, ref) < tol
    assert torch.equal(out, out.transpose(1, 2))
    a = out.clone()
    if n * 4 % 16 == 0 and a.shape[-1] >= 1024:
        poly = gemm(a, a.transpose(1, 2), c=a, alpha=0.5, beta=-1.5, symmetric=True)
        ref2 = 0.5 * a.float() @ a.float().transpose(1, 2) - 1.5 * a.float()
        assert _rel_err(poly, ref2) < tol
        assert torch.equal(poly, poly.transpose(1, 2))


@pytest.mark.gpu
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("shape,symmetric", [((384, 200, 328), False), ((512, 512, 1000), False), ((200, 64, 72), False),
                                             ((256, 256, 520), True), ((768, 768, 768), True)])
def test_gemm_split3_splits_fp32_operands_in_shared_memory(ta, tb, shape, symmetric):
    """3xTF32 product of plain fp32 operands: the kernel forms the tf32 halves of every tile itself.
    Against fp64, and against the product of operands that were split beforehand."""
    M, N, K = shape
    B = 3
    if symmetric:
        if ta != tb:
            pytest.skip("a symmetric product multiplies an operand with its own transpose")
        x = _operand(M, K, torch.float32, ta, batch=B)
        a, b = x, x.transpose(-1, -2)
    else:
        a = _operand(M, K, torch.float32, ta, batch=B)
        b = _operand(K, N, torch.float32, tb, batch=B)
    ref = a.double() @ b.double()
    one = gemm(a, b, symmetric=symmetric)
    three = gemm(a, b, symmetric=symmetric, split3=True)
    e1, e3 = _rel_err(one, ref), _rel_err(three, ref)
    assert e3 < 2e-5 and e1 > 10 * e3, (e1, e3)
    # epilogue options ride along: addend with column scale, alpha / beta, strided views as operands
    c = torch.randn(B, M, N, device="cuda")
    s = torch.rand(B, N, device="cuda") + 0.5
    if not symmetric:
        out = gemm(a, b, c=c, alpha=-1.0, beta=1.0, c_col_scale=s, split3=True)
        assert _rel_err(out, c.double() * s.unsqueeze(1).double() - ref) < 2e-5
        big = torch.randn(B, M + 40, K + 24, device="cuda")
        av = big[:, 8:8 + M, 16:16 + K]
        out = gemm(av, b, split3=True)
        assert _rel_err(out, av.double() @ b.double()) < 2e-5
    from dion_b200 import ops

    ops.check_status()
