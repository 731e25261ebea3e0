"""tcgen05 GEMM front end: ``gemm(a, b)`` computes ``alpha * a @ b (+ beta * c)`` for
bf16 or fp32 (TF32) operands given as arbitrary row/column-major 2-D or 3-D views.

It carries every matrix product the reference issues through cuBLAS: the power-iteration products
``M @ Q`` / ``M^T @ P`` (dion/dion.py:801, 839, 921, 951, 1073, 1098), ``foreach_baddbmm_``
(dion/dion.py:1494-1530), the Newton-Schulz products (dion/newton_schulz_triton.py:336-374) and the
model's linear layers.

On CPU tensors (tests, host-side logic) the same call runs a plain PyTorch
implementation of identical semantics, which is also the numerical reference of the
GPU tests.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import runtime

_ACT = {None: 0, "none": 0, "relu2": 1, "relu2_save_pre": 2, "mul_relu2_grad": 3, "mul_relu2_grad_sq": 4}


def _apply_act(x: torch.Tensor, act) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act == "relu2":
        return torch.relu(x).square()
    raise ValueError(f"unknown activation {act!r}")


def gemm_reference(a, b, *, c=None, out=None, alpha=1.0, beta=0.0, act=None, out_dtype=None, accumulate=False,
                   shadow=None, compute_dtype=torch.float32):
    """PyTorch implementation with the semantics of :func:`gemm` (fp32 accumulate)."""
    acc = torch.matmul(a.to(compute_dtype), b.to(compute_dtype)).float() * alpha
    pre = acc
    if act == "mul_relu2_grad":
        res = acc * 2.0 * torch.relu(c.float())
    elif act == "mul_relu2_grad_sq":
        res = acc * 2.0 * torch.relu(c.float()).sqrt()
    else:
        res = _apply_act(acc, "relu2" if act == "relu2_save_pre" else act)
        if c is not None and beta != 0.0:
            res = res + beta * c.float()
    if out is None:
        out = torch.empty(acc.shape, dtype=out_dtype or a.dtype, device=a.device)
        accumulate = False
    if accumulate:
        out.add_(res.to(out.dtype))
    else:
        out.copy_(res.to(out.dtype))
    if shadow is not None:
        shadow.copy_((pre if act == "relu2_save_pre" else out).to(shadow.dtype))
    return out


def _tma_ok(t: torch.Tensor) -> bool:
    es = t.element_size()
    if t.data_ptr() % 16:
        return False
    s_row, s_col = t.stride(-2), t.stride(-1)
    rows, cols = t.shape[-2], t.shape[-1]
    if s_col == 1 and (s_row >= cols or rows == 1):
        ld = s_row if rows > 1 else max(s_row, cols)
    elif s_row == 1 and (s_col >= rows or cols == 1):
        ld = s_col if cols > 1 else max(s_col, rows)
    else:
        return False
    if (ld * es) % 16:
        return False
    if t.dim() == 3 and t.shape[0] > 1 and (t.stride(0) * es) % 16:
        return False
    return True


def gemm(a: torch.Tensor, b: torch.Tensor, *, c: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         alpha: float = 1.0, beta: float = 0.0, act: Optional[str] = None, out_dtype: Optional[torch.dtype] = None,
         accumulate: bool = False, split_k: int = 1, symmetric: bool = False, shadow: Optional[torch.Tensor] = None,
         block_n: int = 0, pair: int = 0, out_ptrs: Optional[torch.Tensor] = None, c_ptrs: Optional[torch.Tensor] = None,
         shadow_ptrs: Optional[torch.Tensor] = None, out_dup: int = 1, a_lo: Optional[torch.Tensor] = None,
         b_lo: Optional[torch.Tensor] = None, c_col_scale: Optional[torch.Tensor] = None,
         split3: bool = False) -> torch.Tensor:
    """``out = act(alpha * a @ b + beta * c)``.

    a: ``[B,] M, K``; b: ``[B,] K, N``; each may be a transposed view (one unit stride in
    the last two dims).  ``accumulate=True`` adds ``alpha * a @ b`` into an fp32 ``out``
    with atomics (needed for ``split_k > 1``).  ``symmetric=True`` promises that the
    result is symmetric (e.g. ``x @ x.T``) and computes only half of the tiles.
    ``shadow`` receives a bf16 copy of ``out``.  ``*_ptrs`` are int64 CUDA tensors with
    one device address per batch element, for outputs that are separate allocations.
    With ``out_dup = k > 1`` every batch element is stored to k destinations, ``out_ptrs[b * k + j]``
    (for instance one slot of a symmetric buffer on each rank of a group).
    ``a_lo`` / ``b_lo`` (fp32, laid out like ``a`` / ``b``): ``a`` and ``b`` are then the tf32-exact high
    halves of split operands and the product is ``a @ b + a_lo @ b + a @ b_lo`` accumulated in one pass
    over three K-segments - a 3xTF32 product in a single launch.
    ``c_col_scale`` (fp32 ``[B, N]``) scales the columns of the addend: ``beta * c * diag(c_col_scale)``.
    ``split3=True`` (fp32 operands): the same 3xTF32 product without any hi / lo tensors - the kernel splits
    every operand tile in shared memory, so the operands are read once.  On CPU tensors, and for operands
    the kernel cannot address, the product is taken in plain fp32.
    """
    if a.dim() not in (2, 3) or a.dim() != b.dim():
        raise ValueError("gemm expects two 2-D or two 3-D operands")
    if a.dtype != b.dtype:
        raise ValueError(f"operand dtypes differ: {a.dtype} vs {b.dtype}")
    M, N = a.shape[-2], b.shape[-1]
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an existing output")
        shape = (*a.shape[:-2], M, N)
        out = torch.empty(shape, dtype=out_dtype or a.dtype, device=a.device)

    if (a_lo is None) != (b_lo is None):
        raise ValueError("hi / lo operands need both low halves")
    if split3 and (a_lo is not None or (a.is_cuda and a.dtype != torch.float32)):
        raise ValueError("split3 takes fp32 operands without separate low halves")
    if c_col_scale is not None and (c is None or not a.is_cuda):
        if c is None:
            raise ValueError("c_col_scale needs the addend c")
        return gemm(a, b, c=c.float() * c_col_scale.view(*c.shape[:-2], 1, c.shape[-1]), out=out, alpha=alpha,
                    beta=beta, act=act, out_dtype=out_dtype, a_lo=a_lo, b_lo=b_lo, split3=split3)
    if a_lo is not None and (not a.is_cuda or a.dtype != torch.float32 or not (_tma_ok(a_lo) and _tma_ok(b_lo))):
        # no kernel for this case: the same sum from three products
        out = gemm(a, b, c=c, out=out, alpha=alpha, beta=beta, act=act, out_dtype=out_dtype)
        gemm(a_lo, b, c=out, out=out, alpha=alpha, beta=1.0)
        return gemm(a, b_lo, c=out, out=out, alpha=alpha, beta=1.0)
    if not runtime.use_cuda_kernels(a):
        if out_ptrs is not None or c_ptrs is not None or shadow_ptrs is not None:
            raise ValueError("pointer-array outputs need CUDA tensors")
        return gemm_reference(a, b, c=c, out=out, alpha=alpha, beta=beta, act=act, accumulate=accumulate,
                              shadow=shadow)

    if a.dtype not in (torch.bfloat16, torch.float32) or not (_tma_ok(a) and _tma_ok(b)) or out.stride(-1) != 1:
        # shapes TMA cannot address (pitch not a multiple of 16 bytes): library GEMM
        if out_ptrs is not None or c_ptrs is not None or shadow_ptrs is not None:
            raise ValueError("unaligned operands cannot be combined with pointer-array outputs")
        cd = torch.float32 if a.dtype == torch.float32 else a.dtype
        return gemm_reference(a, b, c=c, out=out, alpha=alpha, beta=beta, act=act, accumulate=accumulate,
                              shadow=shadow, compute_dtype=cd)

    if split_k > 1 and not accumulate:
        raise ValueError("split_k > 1 needs accumulate=True")
    torch.ops.dion_b200.gemm(a, b, c, out, shadow, c_ptrs, out_ptrs, shadow_ptrs, float(alpha), float(beta),
                             _ACT[act], 1 if accumulate else 0, int(split_k), bool(symmetric), int(block_n), int(pair),
                             runtime.status_tensor(a.device), int(out_dup), a_lo, b_lo, c_col_scale, bool(split3))
    return out
