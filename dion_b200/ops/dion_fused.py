"""Front ends of the kernels that fuse Dion's reductions over ranks with the arithmetic that follows
(csrc/dion_fused.cu), each with a PyTorch statement of the same semantics for CPU tensors and tests.

A "slot buffer" is an fp32 tensor ``[nslots, ...]``: slot s holds what rank s contributed to a sum.
``wait`` is ``None`` (the slots are complete when the kernel starts) or the tuple returned by
``SymmetricArena.wait_args()``: the kernel then first tells the ranks of the group that this rank's
contribution has been stored and waits, with a bound, for theirs.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import runtime

_NO_WAIT = ([], 0, 0, 0, 0, 0)


def slot_reduce(slots: torch.Tensor, out: Optional[torch.Tensor], hi: Optional[torch.Tensor],
                lo: Optional[torch.Tensor], dests: Sequence[int], scale: float, wait: Optional[tuple] = None) -> None:
    """``out = scale * sum_s slots[s]`` (slot order), optionally with its tf32 halves ``hi`` / ``lo``
    (``hi`` = low 13 mantissa bits cleared, ``lo = out - hi``) and copies stored to the raw device
    addresses ``dests`` (e.g. slots of another group's buffers)."""
    if runtime.use_cuda_kernels(slots):
        peers, flag_off, channel, rank, epoch, budget = wait if wait is not None else _NO_WAIT
        torch.ops.dion_b200.slot_reduce(slots, out, hi, lo, list(dests), float(scale), list(peers), flag_off, channel,
                                        rank, epoch, budget, runtime.status_tensor(slots.device))
        return
    if dests:
        raise ValueError("raw destination addresses need CUDA tensors")
    acc = slots[0].clone()
    for s in range(1, slots.shape[0]):
        acc += slots[s]
    acc *= scale
    if out is not None:
        out.copy_(acc)
    if hi is not None:
        h = (acc.contiguous().view(torch.int32) & -8192).view(torch.float32)
        hi.copy_(h)
        lo.copy_(acc - h)


def dion_r_post_reference(slots, scale, nonzero, Qm, P, eps, finish=True):
    """PyTorch statement of :func:`dion_r_post`: returns (R fp32, P, ss, Qn or None)."""
    R = slots[0].clone()
    for s in range(1, slots.shape[0]):
        R = R + slots[s]
    R = R * scale
    B = R.shape[0]
    nz = (nonzero != 0).view(B, 1, 1) if nonzero is not None else torch.ones(B, 1, 1, dtype=torch.bool, device=R.device)
    R = torch.where(nz, R.nan_to_num(), Qm.float())
    if P is not None:
        P = torch.where(nz, P.nan_to_num(), torch.zeros_like(P))
    ss = R.square().sum(dim=-2)
    Qn = None
    if finish:
        Qn = torch.where((ss > 0).unsqueeze(1), R / (ss.sqrt().unsqueeze(1) + eps), Qm.float())
    return R, P, ss, Qn


def dion_r_post(slots: torch.Tensor, scale: float, nonzero: Optional[torch.Tensor], Qm: torch.Tensor,
                P: Optional[torch.Tensor], R32: Optional[torch.Tensor], Rm: Optional[torch.Tensor],
                ss: Optional[torch.Tensor], finish: bool, eps: float, Qn: Optional[torch.Tensor],
                Qs: Optional[torch.Tensor], qs_col0: int, wait: Optional[tuple] = None) -> None:
    """After ``R = A^T P`` (``slots: [nslots, B, n, r]``): R = scale * sum of the slots; matrices whose
    momentum is all zero (``nonzero[b] == 0``) get R = previous Q (``Qm``) and P = 0, all others have
    NaN / inf replaced in R and in ``P`` (in place) (fix_all_zero_or_nan, dion/dion.py:1416-1444).
    ``R32`` / ``Rm`` receive R in fp32 / in their own dtype, ``ss`` its column sums of squares.  With
    ``finish`` the new Q = R / (sqrt(ss) + eps), keeping the previous Q in columns whose sum is zero, goes
    to ``Qn`` (all columns) and columns ``[qs_col0, qs_col0 + Qs.shape[2])`` of it to ``Qs``
    (column_normalize and update_Q_matrix_, dion/dion.py:1460-1491, 1533-1561)."""
    if runtime.use_cuda_kernels(slots):
        peers, flag_off, channel, rank, epoch, budget = wait if wait is not None else _NO_WAIT
        torch.ops.dion_b200.dion_r_post(slots, float(scale), nonzero, Qm, P, R32, Rm, ss, bool(finish), float(eps), Qn,
                                        Qs, int(qs_col0), list(peers), flag_off, channel, rank, epoch, budget,
                                        runtime.status_tensor(slots.device))
        return
    R, Pn, s2, Q = dion_r_post_reference(slots, scale, nonzero, Qm, P, eps, finish)
    if P is not None:
        P.copy_(Pn)
    if R32 is not None:
        R32.copy_(R)
    if Rm is not None:
        Rm.copy_(R.to(Rm.dtype))
    if ss is not None:
        ss.copy_(s2)
    if finish:
        if Qn is not None:
            Qn.copy_(Q.to(Qn.dtype))
        if Qs is not None:
            Qs.copy_(Q[:, :, qs_col0:qs_col0 + Qs.shape[2]].to(Qs.dtype))


def dion_q_norm(R32: torch.Tensor, ss: torch.Tensor, Qm: torch.Tensor, eps: float, Qn: Optional[torch.Tensor],
                Qs: Optional[torch.Tensor], qs_col0: int) -> None:
    """The column normalisation of :func:`dion_r_post` on its own, for sums of squares that were
    completed over the ranks sharding R's rows."""
    if runtime.use_cuda_kernels(R32):
        torch.ops.dion_b200.dion_q_norm(R32, ss, Qm, float(eps), Qn, Qs, int(qs_col0))
        return
    Q = torch.where((ss > 0).unsqueeze(1), R32 / (ss.sqrt().unsqueeze(1) + eps), Qm.float())
    if Qn is not None:
        Qn.copy_(Q.to(Qn.dtype))
    if Qs is not None:
        Qs.copy_(Q[:, :, qs_col0:qs_col0 + Qs.shape[2]].to(Qs.dtype))
