"""Tensor-parallel region functions on local shards (explicit collectives with the matching
backward), vocabulary-parallel embedding and cross-entropy.

The reference expresses the same data flow through DTensor ``parallelize_module`` plans
(models/gpt_model.py:291-333): column-parallel inputs are replicated, row-parallel outputs
are all-reduced, the embedding is sharded by vocabulary rows and the lm_head logits are
gathered.  Here the collectives are written out, and the lm_head never materialises the
gathered logits: the cross-entropy exchanges only per-token max / sum-exp / target logit.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import nn as K


class _CopyToRegion(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRegion(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromRegion(torch.autograd.Function):
    """All-gather along the last dim forward, slice backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        world, rank = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = g.shape[-1] // world
        return g[..., rank * n:(rank + 1) * n].contiguous(), None


def copy_to_tp_region(x, group):
    return _CopyToRegion.apply(x, group)


def reduce_from_tp_region(x, group):
    return _ReduceFromRegion.apply(x, group)


def gather_from_tp_region(x, group):
    return _GatherFromRegion.apply(x, group)


def vocab_parallel_embedding(idx: torch.Tensor, table_local: torch.Tensor, group, out_dtype) -> torch.Tensor:
    """Embedding whose rows are sharded over `group`: look up the locally owned ids, zero the
    others, all-reduce."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rows = table_local.shape[0]
    lo = rank * rows
    mask = (idx >= lo) & (idx < lo + rows)
    local_idx = torch.where(mask, idx - lo, torch.zeros_like(idx))
    out = K.embedding(local_idx, table_local, out_dtype)
    out = out * mask.unsqueeze(-1).to(out.dtype)
    return reduce_from_tp_region(out, group)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy over logits whose vocabulary dim is sharded: three small
    all-reduces (max, sum-exp, target logit) instead of gathering the logits."""

    @staticmethod
    def forward(ctx, logits_local, targets, group, ignore_index):
        rank = dist.get_rank(group)
        v_loc = logits_local.shape[-1]
        lo = rank * v_loc
        lf = logits_local.float()
        mx = lf.max(dim=-1).values
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lf - mx.unsqueeze(-1))
        se = ex.sum(dim=-1)
        dist.all_reduce(se, group=group)
        valid = targets != ignore_index
        mine = valid & (targets >= lo) & (targets < lo + v_loc)
        t_loc = torch.where(mine, targets - lo, torch.zeros_like(targets))
        tl = torch.where(mine, lf.gather(-1, t_loc.unsqueeze(-1)).squeeze(-1), torch.zeros_like(mx))
        dist.all_reduce(tl, group=group)
        n_valid = valid.sum().clamp_min(1).float()
        loss = torch.where(valid, mx + se.log() - tl, torch.zeros_like(mx)).sum() / n_valid
        probs = ex / se.unsqueeze(-1)
        probs.scatter_add_(-1, t_loc.unsqueeze(-1), -mine.float().unsqueeze(-1))
        probs = probs * (valid.float() / n_valid).unsqueeze(-1)
        ctx.save_for_backward(probs.to(logits_local.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return grad * g.to(grad.dtype), None, None, None


def vocab_parallel_cross_entropy(x: torch.Tensor, weight_local: torch.Tensor, targets: torch.Tensor, group,
                                 ignore_index: int = -1) -> torch.Tensor:
    x2 = copy_to_tp_region(x.reshape(-1, x.shape[-1]), group)
    logits = K.linear(x2, weight_local)
    return _VocabParallelCE.apply(logits, targets.reshape(-1), group, ignore_index)
