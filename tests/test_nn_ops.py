"""Model kernels (norms, rotary, ReLU^2, embedding, fused lm_head + cross-entropy, Linear)
against fp32 PyTorch references, forward and backward."""
import pytest
import torch
import torch.nn.functional as F

from dion_b200.ops import nn as N


def _close(x, ref, tol):
    """max |x - ref| relative to the scale of ref (bf16 intermediates make per-element
    relative checks meaningless near zero)."""
    err = ((x.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-20)).item()
    assert err < tol, f"scaled max error {err:.3e} >= {tol}"


def _ref_rms(x, eps=N.RMS_EPS):
    xf = x.float()
    return xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)


def test_cpu_paths_are_differentiable():
    x = torch.randn(2, 5, 16, requires_grad=True)
    w = torch.randn(24, 16, requires_grad=True)
    y = N.linear(N.rms_norm(x), w, act="relu2")
    y.sum().backward()
    assert x.grad is not None and w.grad is not None
    cos, sin = N.rotary_tables(5, 8, "cpu")
    q = torch.randn(2, 5, 2, 8)
    qo, ko = N.rope_qknorm(q, q.clone(), cos, sin)
    assert qo.shape == q.shape
    torch.testing.assert_close(qo.square().mean(-1), torch.ones(2, 5, 2), rtol=1e-3, atol=1e-3)
    t = torch.randint(0, 24, (2, 5))
    loss = N.linear_cross_entropy(torch.randn(2, 5, 16), w, t)
    assert loss.ndim == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [768, 64, 4096])
def test_rmsnorm_kernel(dim):
    x = torch.randn(37, 5, dim, device="cuda").bfloat16().requires_grad_()
    y = N.rms_norm(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = _ref_rms(xr)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim", [64, 128])
def test_rope_qknorm_kernel(head_dim):
    B, T, H = 2, 48, 3
    cos, sin = N.rotary_tables(T, head_dim, "cuda")
    q = torch.randn(B, T, H, head_dim, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, H, head_dim, device="cuda").bfloat16().requires_grad_()
    qo, ko = N.rope_qknorm(q, k, cos, sin)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    (qo * gq).sum().backward(retain_graph=True)
    (ko * gk).sum().backward()
    qr = q.detach().float().requires_grad_()
    kr = k.detach().float().requires_grad_()
    qro, kro = N._rope_qknorm_torch(qr, kr, cos, sin, N.RMS_EPS)
    ((qro * gq.float()).sum() + (kro * gk.float()).sum()).backward()
    torch.testing.assert_close(qo.float(), qro, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(ko.float(), kro, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q.grad.float(), qr.grad, rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(k.grad.float(), kr.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim", [64, 128])
def test_rope_qknorm_kernel_on_views_that_are_only_8_byte_aligned(head_dim):
    """Inputs that start 8 bytes into an allocation take the kernels with 8-byte accesses; same results."""
    B, T, H = 2, 40, 3
    n = B * T * H * head_dim
    cos, sin = N.rotary_tables(T, head_dim, "cuda")
    qbuf = torch.randn(n + 4, device="cuda").bfloat16()
    kbuf = torch.randn(n + 4, device="cuda").bfloat16()
    q = qbuf[4:].view(B, T, H, head_dim).requires_grad_()
    k = kbuf[4:].view(B, T, H, head_dim).requires_grad_()
    assert q.data_ptr() % 16 == 8 and q.is_contiguous()
    qo, ko = N.rope_qknorm(q, k, cos, sin)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    ((qo * gq).sum() + (ko * gk).sum()).backward()
    qr = q.detach().float().requires_grad_()
    kr = k.detach().float().requires_grad_()
    qro, kro = N._rope_qknorm_torch(qr, kr, cos, sin, N.RMS_EPS)
    ((qro * gq.float()).sum() + (kro * gk.float()).sum()).backward()
    torch.testing.assert_close(qo.float(), qro, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(ko.float(), kro, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q.grad.float(), qr.grad, rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(k.grad.float(), kr.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim", [64, 128])
def test_rope_alone_kernel(head_dim):
    """Rotary embedding of one tensor without the norm (the Llama-shaped model's use)."""
    B, T, H = 2, 33, 5
    cos, sin = N.rotary_tables(T, head_dim, "cuda")
    x = torch.randn(B, T, H, head_dim, device="cuda").bfloat16().requires_grad_()
    y = N.rope(x, cos, sin)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    d = head_dim // 2
    c, s_ = cos[None, :T, None, :].float(), sin[None, :T, None, :].float()
    yr = torch.cat([xr[..., :d] * c + xr[..., d:] * s_, xr[..., d:] * c - xr[..., :d] * s_], dim=-1)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_relu2_kernel():
    x = torch.randn(64, 3072, device="cuda").bfloat16().requires_grad_()
    h = N.relu2(x)
    g = torch.randn_like(h)
    h.backward(g)
    xr = x.detach().float().requires_grad_()
    hr = torch.relu(xr).square()
    hr.backward(g.float())
    torch.testing.assert_close(h.float(), hr, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
def test_embedding_kernel():
    table = torch.randn(1000, 768, device="cuda", requires_grad=True)
    idx = torch.randint(0, 1000, (4, 33), device="cuda")
    idx[0, :5] = 7  # repeated ids accumulate
    out = N.embedding(idx, table)
    g = torch.randn_like(out)
    out.backward(g)
    assert torch.equal(out, table.detach()[idx].bfloat16())
    ref = torch.zeros_like(table)
    ref.index_put_((idx.reshape(-1),), g.float().view(-1, 768), accumulate=True)
    torch.testing.assert_close(table.grad, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("residual", [False, True])
def test_linear_fn(residual):
    T, K, Nn = 300, 256, 520
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(Nn, K, device="cuda") / K ** 0.5).requires_grad_()
    r = torch.randn(T, Nn, device="cuda").bfloat16().requires_grad_() if residual else None
    y = N.linear(x, w, residual=r)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    yr = xr @ wr.t() + (r.detach().float() if residual else 0)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad, wr.grad, rtol=2e-2, atol=2e-2)
    assert w.grad.dtype == torch.float32
    if residual:
        assert torch.equal(r.grad, g)


@pytest.mark.gpu
def test_linear_relu2_and_split_k_weight_grad():
    T, K, Nn = 4096, 128, 256
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(Nn, K, device="cuda") / K ** 0.5).requires_grad_()
    y = N.linear(x, w, act="relu2")
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    pre = (xr @ wr.t()).bfloat16().float()
    # reference through the same bf16 rounding of the pre-activation
    yr = torch.relu(xr @ wr.t()).square()
    yr.backward(g.float())
    _close(y, torch.relu(pre).square(), 1e-2)
    _close(x.grad, xr.grad, 2e-2)
    _close(w.grad, wr.grad, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [50304, 1024])
def test_linear_cross_entropy(vocab):
    T, K = 700, 256
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(vocab, K, device="cuda") / K ** 0.5).requires_grad_()
    t = torch.randint(0, vocab, (T,), device="cuda")
    t[:9] = -1
    loss = N.linear_cross_entropy(x, w, t, ignore_index=-1, chunk_tokens=256)
    (loss * 0.5).backward()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    logits = (xr @ wr.t())
    lr = F.cross_entropy(logits, t, ignore_index=-1)
    (lr * 0.5).backward()
    torch.testing.assert_close(loss, lr, rtol=5e-3, atol=5e-3)
    _close(x.grad, xr.grad, 2e-2)
    _close(w.grad, wr.grad, 2e-2)
    with torch.no_grad():
        l2 = N.linear_cross_entropy(x, w, t, ignore_index=-1)
    torch.testing.assert_close(l2, lr, rtol=5e-3, atol=5e-3)


@pytest.mark.gpu
def test_fused_mlp_matches_unfused_reference():
    T, D = 520, 256
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_()
    res = torch.randn(T, D, device="cuda").bfloat16().requires_grad_()
    w_fc = (torch.randn(4 * D, D, device="cuda") / D ** 0.5).requires_grad_()
    w_pj = (torch.randn(D, 4 * D, device="cuda") / (4 * D) ** 0.5).requires_grad_()
    out = N.mlp(x, w_fc, w_pj, res)
    g = torch.randn_like(out)
    out.backward(g)
    xr = x.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_()
    fr = w_fc.detach().bfloat16().float().requires_grad_()
    pr = w_pj.detach().bfloat16().float().requires_grad_()
    ref = rr + torch.relu(xr @ fr.t()).square() @ pr.t()
    ref.backward(g.float())
    _close(out, ref, 2e-2)
    _close(x.grad, xr.grad, 3e-2)
    _close(w_fc.grad, fr.grad, 3e-2)
    _close(w_pj.grad, pr.grad, 3e-2)
    assert torch.equal(res.grad, g)


@pytest.mark.gpu
def test_norm_branch_adds_both_gradients():
    x = torch.randn(33, 768, device="cuda").bfloat16().requires_grad_()
    xp, h = N.norm_branch(x)
    g1, g2 = torch.randn_like(xp), torch.randn_like(h)
    (xp * g1).sum().backward(retain_graph=True)
    gx_pass = x.grad.clone()
    x.grad = None
    ((xp * g1).sum() + (h * g2).sum()).backward()
    xr = x.detach().float().requires_grad_()
    (_ref_rms(xr) * g2.float()).sum().backward()
    _close(x.grad, xr.grad + g1.float(), 2e-2)
    assert torch.equal(xp, x)
    _close(gx_pass, g1.float(), 1e-2)  # the pass-through output alone hands its gradient on unchanged


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 256, 3, 3, 128), (1, 1024, 4, 2, 128), (3, 384, 2, 2, 64), (2, 128, 2, 1, 64)])
def test_flash_attention_forward_matches_fp32_reference(shape):
    from dion_b200 import ops
    from dion_b200.ops.nn import flash_attention_forward

    B, T, H, Hkv, D = shape
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, T, H, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    out, lse = flash_attention_forward(q, k, v)
    ops.check_status()
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    kf = kf.repeat_interleave(H // Hkv, dim=1)
    vf = vf.repeat_interleave(H // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) / D ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, device="cuda", dtype=torch.bool), 1), float("-inf"))
    ref = torch.softmax(s, dim=-1) @ vf
    err = (out.float().transpose(1, 2) - ref).abs().max().item()
    assert err < 2e-2, err
    torch.testing.assert_close(lse, torch.logsumexp(s, dim=-1), rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 256, 3, 3, 128), (1, 1024, 4, 2, 128), (3, 384, 2, 2, 64), (2, 128, 4, 1, 64)])
def test_flash_attention_backward_matches_fp32_reference(shape):
    from dion_b200 import ops
    from dion_b200.ops.nn import flash_attention_backward, flash_attention_forward

    B, T, H, Hkv, D = shape
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(B, T, H, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    d_out = torch.randn(B, T, H, D, device="cuda", generator=g).to(torch.bfloat16)
    out, lse = flash_attention_forward(q, k, v)
    dq, dk, dv = flash_attention_backward(q, k, v, out, lse, d_out)
    ops.check_status()
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    kr = kf.transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    vr = vf.transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    s = (qf.transpose(1, 2) @ kr.transpose(-1, -2)) / D ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, device="cuda", dtype=torch.bool), 1), float("-inf"))
    ref = (torch.softmax(s, dim=-1) @ vr).transpose(1, 2)
    ref.backward(d_out.float())
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (got.float() - want).abs().max().item() / want.abs().max().item()
        assert err < 2e-2, (name, err)


@pytest.mark.gpu
def test_linear_fanout_matches_separate_linears():
    x = torch.randn(640, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    ws = [torch.nn.Parameter(torch.randn(n, 256, device="cuda") * 0.05) for n in (256, 128, 384)]
    outs = N.linear_fanout(x, *ws)
    gs = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, gs)
    got = [x.grad.clone()] + [w.grad.clone() for w in ws]
    x.grad = None
    for w in ws:
        w.grad = None
    ref = [N.linear(x, w) for w in ws]
    torch.autograd.backward(ref, gs)
    for o, r in zip(outs, ref):
        assert torch.equal(o, r)
    want = [x.grad] + [w.grad for w in ws]
    for g, w in zip(got, want):
        err = (g.float() - w.float()).abs().max().item() / w.float().abs().max().item()
        assert err < 1e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("rows,dim", [(300, 768), (64, 4096), (1000, 1024), (5, 256)])
@pytest.mark.parametrize("gain_dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_with_gain_kernels(rows, dim, gain_dtype):
    """RMSNorm with a learnable gain: forward, input gradient and the gain's gradient (per-block partial
    sums in a fixed order) against fp32 PyTorch; two backward passes give the same bits."""
    from dion_b200.ops import nn as N

    x = torch.randn(rows, dim, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(gain_dtype).requires_grad_()
    g = torch.randn(rows, dim, device="cuda").bfloat16()
    y = N.rms_norm_gain(x, w, 1e-5)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.square().mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    _close(y, yr, 2e-2)
    _close(x.grad, xr.grad, 3e-2)
    _close(w.grad, wr.grad, 2e-2)
    first = w.grad.clone()
    w.grad = None
    x.grad = None
    N.rms_norm_gain(x, w, 1e-5).backward(g)
    assert torch.equal(w.grad, first)


@pytest.mark.gpu
def test_swiglu_kernels():
    from dion_b200.ops import nn as N

    g = torch.randn(257, 1024, device="cuda").bfloat16().requires_grad_()
    u = torch.randn(257, 1024, device="cuda").bfloat16().requires_grad_()
    d = torch.randn(257, 1024, device="cuda").bfloat16()
    h = N.swiglu(g, u)
    h.backward(d)
    gr, ur = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    hr = torch.nn.functional.silu(gr) * ur
    hr.backward(d.float())
    _close(h, hr, 2e-2)
    _close(g.grad, gr.grad, 2e-2)
    _close(u.grad, ur.grad, 2e-2)
