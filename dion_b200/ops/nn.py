"""Differentiable model ops backed by the sm_100a kernels.

Every public function has two paths with the same semantics:
  * CUDA bf16 tensors -> ``torch.autograd.Function`` wrappers around the in-tree kernels
    (tcgen05 GEMM for the Linear layers, fused elementwise kernels for the rest);
  * anything else (CPU tests, fp32 debugging) -> plain differentiable PyTorch.

The math mirrors the reference model (models/gpt_model.py:54-61 rotary, 86-89 QK norm,
106-112 ReLU^2 MLP, 115-124 weight-less RMSNorm, 171-179 fp32 cross-entropy).
"""

from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import runtime
from .gemm import gemm
from .multi_tensor import cast_copy

RMS_EPS = 1.1920929e-07  # torch.finfo(torch.float32).eps, what F.rms_norm(eps=None) uses


def _fast(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and runtime.use_cuda_kernels(x)


# --------------------------------------------------------------------------- weights in bf16

def bf16_weight(w: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a (usually fp32) parameter, cached on the parameter and refreshed when
    the parameter changed.  Optimizers of this package write the copy in their update
    kernels and call :func:`mark_shadow_fresh`; any other in-place update is detected
    through the tensor version counter."""
    if w.dtype == torch.bfloat16:
        return w.detach()
    sh = getattr(w, "_bf16_shadow", None)
    if sh is None or sh.shape != w.shape or sh.device != w.device:
        sh = torch.empty_like(w, dtype=torch.bfloat16)
        w._bf16_shadow = sh
        w._bf16_shadow_version = None
    if w._bf16_shadow_version != w._version:
        cast_copy([w.detach()], [sh])
        w._bf16_shadow_version = w._version
    return sh


def refresh_bf16_weights(params) -> None:
    """Refresh all stale bf16 copies with a single multi-tensor launch."""
    src, dst, todo = [], [], []
    for w in params:
        if w.dtype == torch.bfloat16 or not w.is_cuda:
            continue
        sh = getattr(w, "_bf16_shadow", None)
        if sh is None or sh.shape != w.shape or sh.device != w.device:
            sh = torch.empty_like(w, dtype=torch.bfloat16)
            w._bf16_shadow = sh
            w._bf16_shadow_version = None
        if w._bf16_shadow_version != w._version:
            src.append(w.detach())
            dst.append(sh)
            todo.append(w)
    if src:
        cast_copy(src, dst)
        for w in todo:
            w._bf16_shadow_version = w._version


def shadow_for_update(w: torch.Tensor) -> Optional[torch.Tensor]:
    """The bf16 copy an optimizer kernel should write together with the fp32 update."""
    return getattr(w, "_bf16_shadow", None)


def mark_shadow_fresh(w: torch.Tensor) -> None:
    if getattr(w, "_bf16_shadow", None) is not None:
        w._bf16_shadow_version = w._version


def mark_shadow_stale(w: torch.Tensor) -> None:
    if getattr(w, "_bf16_shadow", None) is not None:
        w._bf16_shadow_version = None


# --------------------------------------------------------------------------- Linear

def _split_k_for(M: int, N: int, K: int) -> int:
    """Split the contraction so that a skinny weight-gradient GEMM fills the GPU."""
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    if tiles >= 148 or K < 2048:
        return 1
    want = max(1, (4 * 148 + tiles - 1) // tiles)
    return int(max(1, min(want, K // 512, 32)))


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T (+ residual); x: [T, K] bf16, W: [N, K] fp32 master or bf16."""

    @staticmethod
    def forward(ctx, x, weight, residual, act):
        wb = bf16_weight(weight)
        pre = None
        if act is not None:
            pre = torch.empty(x.shape[0], wb.shape[0], device=x.device, dtype=torch.bfloat16)
            gemm(x, wb.t(), out=pre)
            y = torch.empty_like(pre)
            torch.ops.dion_b200.relu2_fwd(pre, y)
        else:
            y = torch.empty(x.shape[0], wb.shape[0], device=x.device, dtype=torch.bfloat16)
            if residual is not None:
                gemm(x, wb.t(), c=residual, beta=1.0, out=y)
            else:
                gemm(x, wb.t(), out=y)
        ctx.save_for_backward(x, weight, pre)
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, pre = ctx.saved_tensors
        wb = bf16_weight(weight)
        dy = dy.contiguous()
        if pre is not None:
            dpre = torch.empty_like(pre)
            torch.ops.dion_b200.relu2_bwd(dy, pre, dpre)
            dy_lin = dpre
        else:
            dy_lin = dy
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            gemm(dy_lin, wb, out=dx)  # [T, N] @ [N, K]
        if ctx.needs_input_grad[1]:
            N, K = wb.shape
            T = x.shape[0]
            sk = _split_k_for(N, K, T)
            if sk > 1:
                dw32 = torch.zeros(N, K, device=x.device, dtype=torch.float32)
                gemm(dy_lin.t(), x, out=dw32, accumulate=True, split_k=sk)
            else:
                dw32 = torch.empty(N, K, device=x.device, dtype=torch.float32)
                gemm(dy_lin.t(), x, out=dw32)
            dw = dw32 if weight.dtype == torch.float32 else dw32.to(weight.dtype)
        dres = dy if ctx.has_residual else None
        return dx, dw, dres, None


def linear(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None,
           act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ weight.T) (+ residual)`` over the last dim of x.  ``act`` in {None, "relu2"}."""
    if _fast(x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        r2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        if act is not None and residual is not None:
            raise ValueError("activation and residual cannot be combined")
        y = _LinearFn.apply(x2, weight, r2, act)
        return y.view(*shp[:-1], weight.shape[0])
    y = F.linear(x, weight.to(x.dtype))
    if act == "relu2":
        y = torch.relu(y).square()
    if residual is not None:
        y = y + residual
    return y


class _LinearFanoutFn(torch.autograd.Function):
    """(x W_0^T, x W_1^T, ...) for several weights applied to the same input (the q / k / v
    projections): the backward pass accumulates the input gradient through the GEMM epilogue
    (``dx += dy_i W_i``) instead of leaving autograd to add three full-size tensors."""

    @staticmethod
    def forward(ctx, x, *weights):
        ctx.save_for_backward(x, *weights)
        outs = []
        for w in weights:
            wb = bf16_weight(w)
            y = torch.empty(x.shape[0], wb.shape[0], device=x.device, dtype=torch.bfloat16)
            gemm(x, wb.t(), out=y)
            outs.append(y)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *dys):
        x, *weights = ctx.saved_tensors
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            first = True
            for w, dy in zip(weights, dys):
                if dy is None:
                    continue
                wb = bf16_weight(w)
                if first:
                    gemm(dy.contiguous(), wb, out=dx)
                    first = False
                else:
                    gemm(dy.contiguous(), wb, c=dx, beta=1.0, out=dx)
            if first:
                dx.zero_()
        dws = []
        for i, (w, dy) in enumerate(zip(weights, dys)):
            if ctx.needs_input_grad[1 + i] and dy is not None:
                dws.append(_weight_grad(dy.contiguous(), x, w))
            else:
                dws.append(None)
        return (dx, *dws)


def linear_fanout(x: torch.Tensor, *weights: torch.Tensor):
    """``tuple(x @ w.T for w in weights)`` with a single accumulated input gradient."""
    if _fast(x):
        shp = x.shape
        outs = _LinearFanoutFn.apply(x.reshape(-1, shp[-1]), *weights)
        return tuple(o.view(*shp[:-1], w.shape[0]) for o, w in zip(outs, weights))
    return tuple(linear(x, w) for w in weights)


class _MLPFn(torch.autograd.Function):
    """out = residual + relu(x W_fc^T)^2 W_proj^T with the activation fused into the GEMM
    epilogues: the forward c_fc product writes h = relu^2 of its result, the backward c_proj product
    multiplies its result by 2 relu(pre) = 2 sqrt(h) on the way out - the pre-activation itself is
    never stored (one [T, 4d] tensor less to write and to keep per layer)."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, residual):
        fc, pj = bf16_weight(w_fc), bf16_weight(w_proj)
        T = x.shape[0]
        h = torch.empty(T, fc.shape[0], device=x.device, dtype=torch.bfloat16)
        gemm(x, fc.t(), out=h, act="relu2")
        out = torch.empty(T, pj.shape[0], device=x.device, dtype=torch.bfloat16)
        gemm(h, pj.t(), c=residual, beta=1.0, out=out)
        ctx.save_for_backward(x, w_fc, w_proj, h)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w_fc, w_proj, h = ctx.saved_tensors
        fc, pj = bf16_weight(w_fc), bf16_weight(w_proj)
        dy = dy.contiguous()
        dpre = torch.empty_like(h)
        gemm(dy, pj, c=h, out=dpre, act="mul_relu2_grad_sq")         # (dy W_proj) * 2 sqrt(h)
        dw_proj = _weight_grad(dy, h, w_proj) if ctx.needs_input_grad[2] else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            gemm(dpre, fc, out=dx)
        dw_fc = _weight_grad(dpre, x, w_fc) if ctx.needs_input_grad[1] else None
        return dx, dw_fc, dw_proj, dy


def _weight_grad(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """dW = dy^T x in fp32 (split over the token dimension when the tile grid is small)."""
    N, K, T = dy.shape[1], x.shape[1], x.shape[0]
    sk = _split_k_for(N, K, T)
    if sk > 1:
        dw = torch.zeros(N, K, device=x.device, dtype=torch.float32)
        gemm(dy.t(), x, out=dw, accumulate=True, split_k=sk)
    else:
        dw = torch.empty(N, K, device=x.device, dtype=torch.float32)
        gemm(dy.t(), x, out=dw)
    return dw if weight.dtype == torch.float32 else dw.to(weight.dtype)


def mlp(x: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """``residual + relu(x @ w_fc.T)**2 @ w_proj.T``."""
    if _fast(x):
        shp = x.shape
        out = _MLPFn.apply(x.reshape(-1, shp[-1]), w_fc, w_proj, residual.reshape(-1, w_proj.shape[0]))
        return out.view(*shp[:-1], w_proj.shape[0])
    return linear(linear(x, w_fc, act="relu2"), w_proj, residual=residual)


# --------------------------------------------------------------------------- RMSNorm

class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        torch.ops.dion_b200.rmsnorm_fwd(x2, None, None, y, rstd, eps)
        ctx.save_for_backward(x2, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd = ctx.saved_tensors
        dy2 = dy.contiguous().view(x2.shape)
        dx = torch.empty_like(x2)
        torch.ops.dion_b200.rmsnorm_bwd(dy2, x2, rstd, None, dx)
        return dx.view(dy.shape), None


class _NormBranchFn(torch.autograd.Function):
    """(x, rmsnorm(x)): hands the residual stream through unchanged next to its normalised
    copy, so that the backward pass adds the two incoming gradients inside the norm kernel."""

    @staticmethod
    def forward(ctx, x, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        torch.ops.dion_b200.rmsnorm_fwd(x2, None, None, y, rstd, eps)
        ctx.save_for_backward(x2, rstd)
        return x.view_as(x), y.view(x.shape)

    @staticmethod
    def backward(ctx, dx_pass, dy):
        x2, rstd = ctx.saved_tensors
        dx = torch.empty_like(x2)
        torch.ops.dion_b200.rmsnorm_bwd(dy.contiguous().view(x2.shape), x2, rstd,
                                        dx_pass.contiguous().view(x2.shape), dx)
        return dx.view(dy.shape), None


def norm_branch(x: torch.Tensor, eps: float = RMS_EPS):
    """Returns ``(x, rms_norm(x))`` for a pre-norm residual block."""
    if _fast(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096 and x.is_contiguous():
        return _NormBranchFn.apply(x, eps)
    return x, rms_norm(x, eps)


def rms_norm(x: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """Weight-less RMSNorm over the last dim."""
    if _fast(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096 and x.is_contiguous():
        return _RMSNormFn.apply(x, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)).to(x.dtype)


class _RMSNormGainFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gain, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        torch.ops.dion_b200.rmsnorm_gain_fwd(x2, gain, y, rstd, eps)
        ctx.save_for_backward(x2, rstd, gain)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd, gain = ctx.saved_tensors
        dy2 = dy.contiguous().view(x2.shape)
        dx = torch.empty_like(x2)
        partial = torch.ops.dion_b200.rmsnorm_gain_bwd(dy2, x2, rstd, gain, dx)
        return dx.view(dy.shape), partial.sum(dim=0).to(gain.dtype), None


def rms_norm_gain(x: torch.Tensor, gain: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """RMSNorm over the last dim with a learnable gain: ``x * rsqrt(mean(x^2) + eps) * gain``.  One kernel
    each way; the backward kernel also reduces the gain's gradient (per-block partial sums in a fixed
    order, summed afterwards)."""
    if (_fast(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096 and x.is_contiguous() and gain.is_cuda
            and gain.is_contiguous() and gain.dtype in (torch.float32, torch.bfloat16) and gain.data_ptr() % 16 == 0):
        return _RMSNormGainFn.apply(x, gain, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * gain.float()).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        h = torch.empty_like(g)
        torch.ops.dion_b200.swiglu_fwd(g, u, h)
        ctx.save_for_backward(g, u)
        return h

    @staticmethod
    def backward(ctx, dh):
        g, u = ctx.saved_tensors
        dg, du = torch.empty_like(g), torch.empty_like(u)
        torch.ops.dion_b200.swiglu_bwd(dh.contiguous(), g, u, dg, du)
        return dg, du


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """``silu(g) * u``: one kernel forward, one backward (both gradients)."""
    if (_fast(g) and u.dtype == g.dtype and g.is_contiguous() and u.is_contiguous() and g.numel() % 8 == 0
            and g.data_ptr() % 16 == 0 and u.data_ptr() % 16 == 0):
        return _SwiGLUFn.apply(g, u)
    return torch.nn.functional.silu(g) * u


# --------------------------------------------------------------------------- rotary + QK norm

def rotary_tables(seq_len: int, head_dim: int, device, base: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [seq_len, head_dim/2] cached in bf16 (models/gpt_model.py:36-51)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    t = torch.arange(seq_len, device=device).float()
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().bfloat16().contiguous(), freqs.sin().bfloat16().contiguous()


def _rope_qknorm_torch(q, k, cos, sin, eps):
    # q, k: [B, T, H, Dh]
    def rot(x):
        d = x.shape[-1] // 2
        x1, x2 = x[..., :d].float(), x[..., d:].float()
        c = cos[None, : x.shape[1], None, :].float()
        s = sin[None, : x.shape[1], None, :].float()
        y = torch.cat([x1 * c + x2 * s, x2 * c - x1 * s], dim=-1)
        y = y * torch.rsqrt(y.square().mean(-1, keepdim=True) + eps)
        return y.to(x.dtype)

    return rot(q), rot(k)


class _RopeQKNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, seq_len, heads, head_dim, eps):
        # q, k: [tokens, heads*head_dim] (possibly column slices of one fused buffer)
        qo = torch.empty(q.shape[0], heads * head_dim, device=q.device, dtype=q.dtype)
        ko = torch.empty_like(qo)
        torch.ops.dion_b200.rope_qknorm_fwd(q, k, qo, ko, cos, sin, seq_len, heads, head_dim, eps)
        ctx.save_for_backward(q, k, cos, sin)
        ctx.cfg = (seq_len, heads, head_dim, eps)
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        q, k, cos, sin = ctx.saved_tensors
        seq_len, heads, head_dim, eps = ctx.cfg
        if q.stride(0) == q.shape[1] and k.stride(0) == k.shape[1]:
            dq = torch.empty_like(q)
            dk = torch.empty_like(k)
        else:
            dq = torch.empty(q.shape, device=q.device, dtype=q.dtype)
            dk = torch.empty(k.shape, device=k.device, dtype=k.dtype)
        if dq.stride(0) != q.stride(0):
            q = q.contiguous()
            k = k.contiguous()
        torch.ops.dion_b200.rope_qknorm_bwd(dqo.contiguous(), dko.contiguous(), q, k, dq, dk, cos, sin, seq_len,
                                            heads, head_dim, eps)
        return dq, dk, None, None, None, None, None, None


def rope_qknorm(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                eps: float = RMS_EPS) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotary embedding followed by RMS norm over head_dim.  q, k: [B, T, H, Dh]."""
    B, T, H, Dh = q.shape
    if _fast(q) and Dh in (64, 128) and q.is_contiguous() and k.is_contiguous():
        qo, ko = _RopeQKNormFn.apply(q.view(B * T, H * Dh), k.view(B * T, H * Dh), cos, sin, T, H, Dh, eps)
        return qo.view(B, T, H, Dh), ko.view(B, T, H, Dh)
    return _rope_qknorm_torch(q, k, cos, sin, eps)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, seq_len, heads, head_dim):
        out = torch.empty(x.shape[0], heads * head_dim, device=x.device, dtype=x.dtype)
        torch.ops.dion_b200.rope_fwd(x, out, cos, sin, seq_len, heads, head_dim)
        ctx.save_for_backward(x, cos, sin)
        ctx.cfg = (seq_len, heads, head_dim)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, cos, sin = ctx.saved_tensors
        seq_len, heads, head_dim = ctx.cfg
        xc = x.contiguous()
        dx = torch.empty_like(xc)
        torch.ops.dion_b200.rope_bwd(dout.contiguous(), xc, dx, cos, sin, seq_len, heads, head_dim)
        return dx, None, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding (half-split pairs) of ``x: [B, T, H, Dh]`` without normalisation."""
    B, T, H, Dh = x.shape
    if _fast(x) and Dh in (64, 128) and x.is_contiguous():
        return _RopeFn.apply(x.view(B * T, H * Dh), cos, sin, T, H, Dh).view(B, T, H, Dh)
    d = Dh // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c = cos[None, :T, None, :].float()
    s = sin[None, :T, None, :].float()
    return torch.cat([x1 * c + x2 * s, x2 * c - x1 * s], dim=-1).to(x.dtype)


# --------------------------------------------------------------------------- ReLU^2

class _Relu2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        h = torch.empty_like(x)
        torch.ops.dion_b200.relu2_fwd(x, h)
        ctx.save_for_backward(x)
        return h

    @staticmethod
    def backward(ctx, dh):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        torch.ops.dion_b200.relu2_bwd(dh.contiguous(), x, dx)
        return dx


def relu2(x: torch.Tensor) -> torch.Tensor:
    if _fast(x) and x.is_contiguous() and x.numel() % 8 == 0:
        return _Relu2Fn.apply(x)
    return torch.relu(x).square()


# --------------------------------------------------------------------------- embedding

class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, table):
        out = torch.empty(idx.numel(), table.shape[1], device=table.device, dtype=torch.bfloat16)
        torch.ops.dion_b200.embedding_fwd(table.detach(), idx.reshape(-1).contiguous(), out)
        ctx.save_for_backward(idx)
        ctx.table_shape = table.shape
        ctx.table_dtype = table.dtype
        return out.view(*idx.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dt = torch.zeros(ctx.table_shape, device=dout.device, dtype=torch.float32)
        torch.ops.dion_b200.embedding_bwd(dout.contiguous().view(-1, dout.shape[-1]), idx.reshape(-1).contiguous(), dt)
        return None, dt if ctx.table_dtype == torch.float32 else dt.to(ctx.table_dtype)


def embedding(idx: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Token embedding gather producing bf16 activations from an fp32 (or bf16) table."""
    if table.is_cuda and out_dtype == torch.bfloat16 and runtime.use_cuda_kernels(table) and \
            table.dtype in (torch.float32, torch.bfloat16) and table.shape[1] % 8 == 0 and table.is_contiguous():
        return _EmbeddingFn.apply(idx, table)
    return F.embedding(idx, table).to(out_dtype)


# --------------------------------------------------------------------------- lm_head + cross entropy

class _LinearCrossEntropyFn(torch.autograd.Function):
    """loss = mean CE(x @ W^T, targets) without keeping the logits: the token dimension is
    processed in chunks; each chunk's logits are turned into their gradient in place by the
    cross-entropy kernel and immediately contracted into dX and dW."""

    @staticmethod
    def forward(ctx, x, weight, targets, ignore_index, chunk_tokens):
        wb = bf16_weight(weight)
        T, K = x.shape
        V = wb.shape[0]
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        valid = (targets != ignore_index).sum().clamp_min(1).to(torch.float32)
        inv_valid = valid.reciprocal()
        row_loss = torch.empty(T, device=x.device, dtype=torch.float32)
        dx = torch.empty_like(x) if need_grad else None
        dw = torch.zeros(V, K, device=x.device, dtype=torch.float32) if need_grad else None
        chunk = min(chunk_tokens, T)
        logits = torch.empty(chunk, V, device=x.device, dtype=torch.bfloat16)
        for t0 in range(0, T, chunk):
            t1 = min(t0 + chunk, T)
            n = t1 - t0
            lg = logits[:n]
            gemm(x[t0:t1], wb.t(), out=lg)
            torch.ops.dion_b200.cross_entropy_fwd_bwd(lg, targets[t0:t1], row_loss[t0:t1], inv_valid, 1.0,
                                                      ignore_index, need_grad)
            if need_grad:
                gemm(lg, wb, out=dx[t0:t1])  # [n, V] @ [V, K]
                gemm(lg.t(), x[t0:t1], out=dw, accumulate=True, split_k=1)  # [V, n] @ [n, K]
        loss = row_loss.sum() * inv_valid
        if need_grad:
            ctx.save_for_backward(dx, dw)
            ctx.w_dtype = weight.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        dxo = dx * dloss.to(dx.dtype) if ctx.needs_input_grad[0] else None
        dwo = None
        if ctx.needs_input_grad[1]:
            dwo = dw * dloss
            if ctx.w_dtype != torch.float32:
                dwo = dwo.to(ctx.w_dtype)
        return dxo, dwo, None, None, None


def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, ignore_index: int = -1,
                         chunk_tokens: int = 8192) -> torch.Tensor:
    """Mean cross-entropy of ``x @ weight.T`` against ``targets`` (fp32 softmax math)."""
    x2 = x.reshape(-1, x.shape[-1])
    t1 = targets.reshape(-1)
    V = weight.shape[0]
    if _fast(x2) and V % 8 == 0 and V <= 131072 and t1.dtype == torch.long:
        return _LinearCrossEntropyFn.apply(x2.contiguous(), weight, t1.contiguous(), ignore_index, chunk_tokens)
    logits = F.linear(x2, weight.to(x2.dtype)).float()
    return F.cross_entropy(logits, t1, ignore_index=ignore_index)


# --------------------------------------------------------------------------- attention

def flash_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None):
    """Causal attention forward by the tcgen05 kernel.  q: [B, T, H, D], k / v: [B, T, Hkv, D], bf16,
    contiguous, D in {64, 128}, T a multiple of 128.  Returns (out [B, T, H, D], lse [B, H, T])."""
    B, T, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    runtime.use_cuda_kernels(q)
    out = torch.empty_like(q)
    lse = torch.empty(B, H, T, dtype=torch.float32, device=q.device)
    torch.ops.dion_b200.attn_fwd(q, k, v, out, lse, float(scale), runtime.status_tensor(q.device))
    return out, lse


def flash_attention_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    B, T, H, D = q.shape
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and D in (64, 128) and T % 128 == 0 and H % k.shape[2] == 0 and B * H <= 65535
            and q.is_contiguous() and k.is_contiguous() and v.is_contiguous())


def flash_attention_backward(q, k, v, out, lse, d_out, scale: Optional[float] = None):
    """Gradients of :func:`flash_attention_forward` by the tcgen05 kernels: (dq, dk, dv)."""
    B, T, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty_like(lse)
    torch.ops.dion_b200.attn_bwd(q, k, v, out, d_out.contiguous(), lse, delta, dq, dk, dv, float(scale),
                                 runtime.status_tensor(q.device))
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        out, lse = flash_attention_forward(q, k, v)
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        return flash_attention_backward(q, k, v, out, lse, d_out)


# "kernel": the in-tree tcgen05 kernels wherever they apply; "library": always
# F.scaled_dot_product_attention (cuDNN / flash kernels of the framework)
ATTENTION_IMPL = os.environ.get("DION_B200_ATTENTION", "kernel")


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal self-attention; q, k, v: [B, T, H, Dh] -> [B, T, H*Dh].  Supports grouped
    KV heads (H_kv dividing H)."""
    B, T, H, Dh = q.shape
    Hkv = k.shape[2]
    if ATTENTION_IMPL == "kernel" and q.is_cuda:
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        if flash_attention_supported(q, k, v):
            return _FlashAttnFn.apply(q, k, v).view(B, T, H * Dh)
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    y = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=(Hkv != H))
    return y.transpose(1, 2).reshape(B, T, H * Dh)
