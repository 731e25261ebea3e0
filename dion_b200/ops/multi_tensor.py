"""Multi-tensor optimizer updates.  On CUDA tensors each call is one (or a few) kernel
launches over the whole list; on CPU tensors the same math runs as plain PyTorch, which
is also the reference the GPU tests compare against.

Math follows the reference's scalar optimizers and Muon helpers
(dion/scalar_opts.py:89-187, dion/muon.py:525-573, dion/dion.py:794).
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import runtime

Tensors = Sequence[torch.Tensor]


def _cuda_path(ts: Tensors) -> bool:
    return len(ts) > 0 and runtime.use_cuda_kernels(ts[0])


def _kernel_dtypes_ok(*lists: Tensors) -> bool:
    for l in lists:
        for t in l:
            if t.dtype not in (torch.float32, torch.bfloat16) or not t.is_contiguous():
                return False
    return True


def adamw_update(X: Tensors, G: Tensors, M: Tensors, V: Tensors, *, lr: float, beta1: float, beta2: float,
                 weight_decay: float, step: int, epsilon: float, shadow: Optional[Tensors] = None) -> None:
    """AdamW with bias correction folded into the step size (scalar_opts.py:89-149)."""
    if len(X) == 0:
        return
    if _cuda_path(X) and X[0].dtype == torch.float32 and _kernel_dtypes_ok(X, G, M, V):
        torch.ops.dion_b200.adamw_multi(list(X), list(G), list(M), list(V), list(shadow or []), lr, beta1, beta2,
                                        weight_decay, epsilon, step)
        return
    adamw_update_reference(X, G, M, V, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, step=step,
                           epsilon=epsilon, shadow=shadow)


def adamw_update_reference(X, G, M, V, *, lr, beta1, beta2, weight_decay, step, epsilon, shadow=None):
    bc1 = 1 - beta1 ** step
    bc2_sqrt = (1 - beta2 ** step) ** 0.5
    for i, (x, g, m, v) in enumerate(zip(X, G, M, V)):
        g = g.to(m.dtype)
        m.lerp_(g, 1 - beta1)
        v.lerp_((g * g).to(v.dtype), 1 - beta2)
        denom = v.float().sqrt().div_(bc2_sqrt).add_(epsilon)
        x.mul_(1 - lr * weight_decay)
        x.sub_((m.float() / denom * (lr / bc1)).to(x.dtype))
        if shadow:
            shadow[i].copy_(x)


def lion_update(X: Tensors, G: Tensors, M: Tensors, *, lr: float, beta1: float, beta2: float, weight_decay: float,
                shadow: Optional[Tensors] = None) -> None:
    """Lion (scalar_opts.py:152-187)."""
    if len(X) == 0:
        return
    if _cuda_path(X) and X[0].dtype == torch.float32 and _kernel_dtypes_ok(X, G, M):
        torch.ops.dion_b200.lion_multi(list(X), list(G), list(M), list(shadow or []), lr, beta1, beta2, weight_decay)
        return
    lion_update_reference(X, G, M, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, shadow=shadow)


def lion_update_reference(X, G, M, *, lr, beta1, beta2, weight_decay, shadow=None):
    for i, (x, g, m) in enumerate(zip(X, G, M)):
        g = g.to(m.dtype)
        u = m.lerp(g, 1 - beta1).sign_()
        m.lerp_(g, 1 - beta2)
        x.mul_(1 - lr * weight_decay)
        x.sub_((u.float() * lr).to(x.dtype))
        if shadow:
            shadow[i].copy_(x)


def muon_momentum(G: Tensors, M: Tensors, *, mu: float, nesterov: bool, U: Optional[List[torch.Tensor]] = None,
                  sumsq: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """``M = mu*M + G``; returns bf16 ``U = mu*M + G`` (Nesterov) or ``M`` (muon.py:525-552).
    ``sumsq[i]`` (fp32, zeroed by the caller) receives ``sum(U_i**2)`` of the bf16 values."""
    if U is None:
        U = [torch.empty_like(m, dtype=torch.bfloat16) for m in M]
    if len(G) == 0:
        return U
    if _cuda_path(M) and M[0].dtype == torch.float32 and _kernel_dtypes_ok(G, M):
        torch.ops.dion_b200.muon_pre_multi(list(G), list(M), list(U), mu, nesterov, sumsq)
        return U
    for i, (g, m, u) in enumerate(zip(G, M, U)):
        g = g.to(m.dtype)
        m.mul_(mu).add_(g)
        u.copy_((m * mu + g) if nesterov else m)
        if sumsq is not None:
            sumsq[i] += u.float().square().sum()
    return U


def muon_apply(X: Tensors, U: Tensors, *, decay: float, step: float, shadow: Optional[Tensors] = None) -> None:
    """``X = decay * X - step * U`` (muon.py:556-573)."""
    if len(X) == 0:
        return
    if _cuda_path(X) and X[0].dtype == torch.float32 and U[0].dtype == torch.bfloat16 and _kernel_dtypes_ok(X, U):
        torch.ops.dion_b200.muon_post_multi(list(X), list(U), list(shadow or []), decay, step)
        return
    for i, (x, u) in enumerate(zip(X, U)):
        x.mul_(decay).sub_((u.float() * step).to(x.dtype))
        if shadow:
            shadow[i].copy_(x)


def dion_accumulate(G: Tensors, M: Tensors, nonzero: Optional[torch.Tensor] = None) -> None:
    """``M += G`` (dion.py:794); ``nonzero[i]`` (int32, zeroed by the caller) is set when M_i has a non-zero entry."""
    if len(G) == 0:
        return
    if _cuda_path(M) and _kernel_dtypes_ok(G, M):
        torch.ops.dion_b200.dion_accum_multi(list(G), list(M), nonzero)
        return
    for i, (g, m) in enumerate(zip(G, M)):
        m.add_(g.to(m.dtype))
        if nonzero is not None:
            nonzero[i] |= int(bool((m != 0).any()))


def cast_copy(src: Tensors, dst: Tensors) -> None:
    """``dst[i] = src[i]`` with dtype conversion (fp32 <-> bf16), one launch for the list."""
    if len(src) == 0:
        return
    if _cuda_path(src) and _kernel_dtypes_ok(src, dst):
        torch.ops.dion_b200.cast_multi(list(src), list(dst))
        return
    for s, d in zip(src, dst):
        d.copy_(s)
