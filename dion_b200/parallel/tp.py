"""Tensor-parallel region functions on local shards (explicit collectives with the matching
backward), vocabulary-parallel embedding and cross-entropy.

The reference expresses the same data flow through DTensor ``parallelize_module`` plans
(models/gpt_model.py:291-333): column-parallel inputs are replicated, row-parallel outputs
are all-reduced, the embedding is sharded by vocabulary rows and the lm_head logits are
gathered.  Here the collectives are written out, and the lm_head never materialises the
gathered logits: the cross-entropy exchanges only per-token max / sum-exp / target logit.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import nn as K
from ..ops import runtime
from ..ops.gemm import gemm
from . import fsdp_comm, symm


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


# ------------------------------------------------------------------ fused GEMM -> all-reduce
class _TPComm:
    """Per-group state of the fused row-parallel product: a symmetric receive buffer with two slots
    (each holds one [world, T / world, N] bf16 block, written by the peers' GEMM epilogues) and the
    all-gather kernel that redistributes the reduced row blocks."""

    def __init__(self, group, device):
        self.group, self.device = group, torch.device(device)
        self.recv = fsdp_comm._Arena(group, self.device)
        self.gather = fsdp_comm.SymmAllGather(group, self.device)
        self.calls = 0
        self.fused_gathers = 0
        self.pushed = 0  # all-reduced products that went through the push into every rank's slots
        self._ptr_cache = {}

    def ptrs(self, slot_off: int, block_bytes: int) -> torch.Tensor:
        """Destination of this rank's partial row block k: slot `rank` of rank k's receive buffer."""
        ar = self.recv.arena
        key = (ar.peers[0], slot_off, block_bytes)
        t = self._ptr_cache.get(key)
        if t is None:
            addr = [ar.peers[k] + slot_off + ar.rank * block_bytes for k in range(ar.world)]
            t = self._ptr_cache[key] = torch.tensor(addr, dtype=torch.int64, device=self.device)
        return t


# All-reduce of a row-parallel product by pushing the partial result to every rank costs (world - 1) times the
# data on NVLink; beyond this group size the product is reduce-scattered and all-gathered instead.
_MAX_PUSH_WORLD = 4
_PUSH_ALL_REDUCE = os.environ.get("DION_B200_TP_PUSH", "1") != "0"
_tp_comms = {}


def _tp_comm(group, device):
    if not symm._usable(group, torch.device(device)):
        return None
    key = symm._key(group)
    c = _tp_comms.get(key)
    if c is None:
        c = _tp_comms[key] = _TPComm(group, device)
    return c


def _matmul_reduce_scatter(pairs, group, residual=None) -> torch.Tensor:
    """Row block `rank` of ``sum over ranks r and over i of x_i_r @ w_t_i_r`` (+ `residual`), for
    ``pairs = [(x_i: [T, K_i], w_t_i: [K_i, N]), ...]``; returns [T / world, N].

    All products but the last accumulate in a local buffer; the last one is a GEMM whose epilogue
    stores row block k of the partial result straight into rank k's receive buffer (peer stores over
    NVLink, tile by tile while the remaining tiles are still being multiplied).  After a flag barrier
    every rank adds up the `world` partial blocks it received (fp32, rank order, so the result does
    not depend on timing).  Falls back to GEMMs + the process group's reduce-scatter when the shapes
    or the group do not fit."""
    x, w_t = pairs[-1]
    T, N = x.shape[0], w_t.shape[1]
    comm = _tp_comm(group, x.device) if x.is_cuda else None
    world = dist.get_world_size(group)
    ok = (comm is not None and x.dtype == torch.bfloat16 and T % world == 0 and (T // world) % 8 == 0 and N % 8 == 0
          and comm.recv.ensure(T * N * 2))
    acc = None
    for xi, wi in pairs[:-1]:
        if xi.is_cuda:
            acc = gemm(xi, wi) if acc is None else gemm(xi, wi, c=acc, out=acc, beta=1.0)
        else:
            acc = xi @ wi if acc is None else acc + xi @ wi
    if not ok:
        if x.is_cuda:
            y = gemm(x, w_t) if acc is None else gemm(x, w_t, c=acc, out=acc, beta=1.0)
        else:
            y = x @ w_t if acc is None else acc + x @ w_t
        out = torch.empty(T // world, N, dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y.contiguous(), group=group)
        return out if residual is None else out + residual
    ar = comm.recv.arena
    comm.calls += 1
    slot = comm.calls & 1
    slot_off = comm.recv.slot_offset(slot)
    rows = T // world
    block_bytes = rows * N * 2
    recv = ar.buf[slot_off:slot_off + T * N * 2].view(torch.bfloat16).view(world, rows, N)
    torch.ops.dion_b200.gemm_scatter(x, w_t, acc, recv[0], comm.ptrs(slot_off, block_bytes), 1, rows, world, 1.0,
                                     0.0 if acc is None else 1.0, runtime.status_tensor(x.device))
    ar.barrier()
    mine = torch.sum(recv, dim=0, dtype=torch.float32)  # fp32 accumulation, fixed order
    if residual is not None:
        mine += residual
    return mine.to(torch.bfloat16)


def _gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    """All-gather of row blocks: [R, ...] on every rank -> [world * R, ...] in rank order (the in-tree
    all-gather kernel over symmetric memory where it applies, the process group's otherwise)."""
    world = dist.get_world_size(group)
    x = x.contiguous()
    out = x.new_empty((world * x.shape[0],) + tuple(x.shape[1:]))
    comm = _tp_comm(group, x.device) if x.is_cuda else None
    if comm is not None:
        comm.gather(out.view(-1), x.view(-1), group)
    else:
        dist.all_gather_into_tensor(out, x, group=group)
    return out


# The all-gather inside the GEMM kernel (copier warps pull the peers' rows while the tensor cores work on
# the rows that are already there) is opt-in until it has been measured against all-gather + GEMM.
_FUSED_GATHER = os.environ.get("DION_B200_TP_FUSED_GATHER", "0") == "1"


def _gather_matmul(x: torch.Tensor, w_t: torch.Tensor, group):
    """``(xg, xg @ w_t)`` with xg the all-gather of the row block x: [R, K] over `group` and w_t: [K, N]
    a transposed view of a weight.  With ``DION_B200_TP_FUSED_GATHER=1`` one kernel does both: two extra
    warps per CTA stage this rank's rows in symmetric memory, announce them, and pull the peers' rows
    into xg chunk by chunk, while the TMA producer of each tile waits for the chunk counter of its rows
    (tiles start with this rank's own rows)."""
    comm = _tp_comm(group, x.device) if x.is_cuda else None
    R, Kd = x.shape
    slots = comm.gather._slots if comm is not None else None
    ok = (_FUSED_GATHER and slots is not None and x.dtype == torch.bfloat16 and w_t.dtype == torch.bfloat16
          and x.is_contiguous() and R % 256 == 0 and Kd % 8 == 0 and w_t.stride(0) == 1 and w_t.stride(1) == Kd
          and w_t.data_ptr() % 16 == 0 and slots.ensure(R * Kd * 2))
    if not ok:
        xg = _gather_rows(x, group)
        return xg, (gemm(xg, w_t) if x.is_cuda else xg @ w_t)
    ar = slots.arena
    world = ar.world
    ar.epoch += 1
    xg = torch.empty(world * R, Kd, dtype=torch.bfloat16, device=x.device)
    y = torch.empty(world * R, w_t.shape[1], dtype=torch.bfloat16, device=x.device)
    counters = torch.empty(2 + world * R // 128, dtype=torch.int32, device=x.device)  # cleared by the launch
    torch.ops.dion_b200.gemm_gather(x, xg, w_t, y, ar.peers, 0, slots.slot_offset(ar.epoch & 1), ar.rank, ar.epoch,
                                    fsdp_comm._CH_AG, counters, runtime.status_tensor(x.device), fsdp_comm._WAIT_NS)
    comm.gather.kernel_calls += 1
    comm.fused_gathers += 1
    return xg, y


def _matmul_all_reduce(x: torch.Tensor, w_t: torch.Tensor, group) -> torch.Tensor:
    """``sum over ranks of x_r @ w_t_r`` for x: [T, K] bf16 and w_t: [K, N] (a transposed view of the
    local weight), identical on every rank: the GEMM -> reduce-scatter above followed by the
    all-gather kernel.  Falls back to GEMM + the process group's all-reduce when the shapes or the
    group do not fit."""
    T, N = x.shape[0], w_t.shape[1]
    comm = _tp_comm(group, x.device) if x.is_cuda else None
    world = dist.get_world_size(group)
    if (comm is not None and _PUSH_ALL_REDUCE and world <= _MAX_PUSH_WORLD and x.dtype == torch.bfloat16
            and w_t.dtype == torch.bfloat16 and (T * N) % 8 == 0 and N % 8 == 0 and comm.recv.ensure(world * T * N * 2)):
        # Small groups: the GEMM epilogue stores every tile of the partial product into slot `rank` of a
        # receive buffer on every rank of the group (the local copy included) while the other tiles are still
        # being multiplied; one kernel then waits for the peers' announcements and adds the slots in rank
        # order.  Two launches, and the NVLink transfer hides behind the product.
        ar = comm.recv.arena
        comm.calls += 1
        slot_off = comm.recv.slot_offset(comm.calls & 1)
        slots = ar.buf[slot_off:slot_off + world * T * N * 2].view(torch.bfloat16).view(world, T, N)
        key = ("all", ar.peers[0], slot_off, T, N)
        table = comm._ptr_cache.get(key)
        if table is None:
            table = comm._ptr_cache[key] = torch.tensor([ar.peers[k] + slot_off + ar.rank * T * N * 2 for k in range(world)],
                                                        dtype=torch.int64, device=x.device)
        gemm(x, w_t, out=slots[0], out_ptrs=table, out_dup=world)
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        torch.ops.dion_b200.slot_reduce_bf16(slots, out, None, *ar.wait_args(), runtime.status_tensor(x.device))
        comm.pushed += 1
        return out
    ok = (comm is not None and x.dtype == torch.bfloat16 and T % world == 0 and (T // world) % 8 == 0 and N % 8 == 0
          and comm.recv.ensure(T * N * 2))
    if not ok:
        y = gemm(x, w_t) if x.is_cuda else x @ w_t
        dist.all_reduce(y, group=group)
        return y
    mine = _matmul_reduce_scatter([(x, w_t)], group)
    out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    comm.gather(out.view(-1), mine.view(-1), group)
    return out


class _RowParallelLinearFn(torch.autograd.Function):
    """y = all-reduce(x_local @ W_local^T) for a row-parallel weight W_local: [N, K_local]."""

    @staticmethod
    def forward(ctx, x, weight, group):
        wb = K.bf16_weight(weight)
        ctx.save_for_backward(x, weight)
        return _matmul_all_reduce(x, wb.t(), group)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        wb = K.bf16_weight(weight)
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, wb)
        if ctx.needs_input_grad[1]:
            dw = K._weight_grad(dy, x, weight)
        return dx, dw, None


class _ColumnParallelInputGradFn(torch.autograd.Function):
    """y = x @ W_local^T for a column-parallel weight W_local: [N_local, K] with a replicated input;
    the input gradient sum over ranks of dy_r @ W_r runs through the same fused product."""

    @staticmethod
    def forward(ctx, x, weight, group):
        wb = K.bf16_weight(weight)
        ctx.save_for_backward(x, weight)
        ctx.group = group
        return gemm(x, wb.t())

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        wb = K.bf16_weight(weight)
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _matmul_all_reduce(dy, wb, ctx.group)
        if ctx.needs_input_grad[1]:
            dw = K._weight_grad(dy, x, weight)
        return dx, dw, None


def row_parallel_linear(x: torch.Tensor, weight_local: torch.Tensor, group) -> torch.Tensor:
    """All-reduced output of a row-parallel linear layer (attn.c_proj / mlp.c_proj under the
    reference's RowwiseParallel plan, models/gpt_model.py:318-327)."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        shp = x.shape
        y = _RowParallelLinearFn.apply(x.reshape(-1, shp[-1]), weight_local, group)
        return y.view(*shp[:-1], weight_local.shape[0])
    return reduce_from_tp_region(K.linear(x, weight_local), group)


def column_parallel_linear(x: torch.Tensor, weight_local: torch.Tensor, group) -> torch.Tensor:
    """Local output columns of a column-parallel linear layer on a replicated input; the backward
    all-reduces the input gradient."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        shp = x.shape
        y = _ColumnParallelInputGradFn.apply(x.reshape(-1, shp[-1]), weight_local, group)
        return y.view(*shp[:-1], weight_local.shape[0])
    return K.linear(copy_to_tp_region(x, group), weight_local)


# ------------------------------------------------------------------ sequence-parallel variants
# The residual stream is kept as row blocks of the flattened token dimension ([B * T / world, C] on
# every rank, rank order): norms and residual additions touch 1 / world of the tokens, the row-parallel
# products end in a reduce-scatter instead of an all-reduce, and the column-parallel products start
# with the all-gather that the all-reduce would have ended with.  The reference's plan keeps the
# activations replicated (models/gpt_model.py:291-333); the communicated volume is the same.

class _GatherRowsFn(torch.autograd.Function):
    """All-gather of row blocks forward, reduce-scatter (sum) of the gradient backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = g.new_empty((g.shape[0] // world,) + tuple(g.shape[1:]))
        dist.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None


class _ScatterSumRowsFn(torch.autograd.Function):
    """Reduce-scatter (sum) of row blocks forward, all-gather of the gradient backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        x = x.contiguous()
        out = x.new_empty((x.shape[0] // world,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _gather_rows(g, ctx.group), None


def gather_rows(x, group):
    return _GatherRowsFn.apply(x, group)


def scatter_sum_rows(x, group):
    return _ScatterSumRowsFn.apply(x, group)


class _GatherLinearFn(torch.autograd.Function):
    """(xg W_0^T, xg W_1^T, ...) with xg the all-gather of the row block x: [R, K] and column-parallel
    W_i: [N_i_local, K].  Backward: the input gradient ``sum_i dy_i W_i`` summed over the ranks comes
    back as this rank's row block through the fused GEMM -> reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group, *weights):
        xg, y0 = _gather_matmul(x, K.bf16_weight(weights[0]).t(), group)
        ctx.save_for_backward(xg, *weights)
        ctx.group = group
        return (y0, *(gemm(xg, K.bf16_weight(w).t()) for w in weights[1:]))

    @staticmethod
    def backward(ctx, *dys):
        xg, *weights = ctx.saved_tensors
        dys = [torch.zeros(xg.shape[0], w.shape[0], dtype=xg.dtype, device=xg.device) if dy is None else dy.contiguous()
               for dy, w in zip(dys, weights)]
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _matmul_reduce_scatter([(dy, K.bf16_weight(w)) for dy, w in zip(dys, weights)], ctx.group)
        dws = [K._weight_grad(dy, xg, w) if ctx.needs_input_grad[2 + i] else None
               for i, (dy, w) in enumerate(zip(dys, weights))]
        return (dx, None, *dws)


class _LinearScatterFn(torch.autograd.Function):
    """Row block `rank` of ``sum over ranks of u_r W_r^T`` (+ residual) for a row-parallel
    W_r: [N, K_local] (fused GEMM -> reduce-scatter); the backward all-gathers the gradient rows."""

    @staticmethod
    def forward(ctx, u, weight, residual, group):
        ctx.save_for_backward(u, weight)
        ctx.group = group
        ctx.has_residual = residual is not None
        return _matmul_reduce_scatter([(u, K.bf16_weight(weight).t())], group, residual)

    @staticmethod
    def backward(ctx, dy):
        u, weight = ctx.saved_tensors
        dyg = _gather_rows(dy, ctx.group)
        du = gemm(dyg, K.bf16_weight(weight)) if ctx.needs_input_grad[0] else None
        dw = K._weight_grad(dyg, u, weight) if ctx.needs_input_grad[1] else None
        return du, dw, (dy if ctx.has_residual else None), None


def gather_linear(x: torch.Tensor, group, *weights_local: torch.Tensor):
    """``tuple(all_gather_rows(x) @ w.T for w in weights_local)`` for column-parallel weights and a
    row-block input x: [R, K]; outputs are [R * world, N_local]."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _GatherLinearFn.apply(x, group, *weights_local)
    xg = gather_rows(x, group)
    return tuple(K.linear(xg, w) for w in weights_local)


def linear_scatter(u: torch.Tensor, weight_local: torch.Tensor, group, residual=None) -> torch.Tensor:
    """Row block of the reduced output of a row-parallel layer: u: [T, K_local] -> [T / world, N]
    (+ `residual`, a row block)."""
    if u.is_cuda and u.dtype == torch.bfloat16:
        return _LinearScatterFn.apply(u, weight_local, residual, group)
    y = scatter_sum_rows(K.linear(u, weight_local), group)
    return y if residual is None else y + residual


def copy_to_tp_region(x, group):
    return _CopyToRegion.apply(x, group)


def reduce_from_tp_region(x, group):
    return _ReduceFromRegion.apply(x, group)


def gather_from_tp_region(x, group):
    return _GatherFromRegion.apply(x, group)


def vocab_parallel_embedding(idx: torch.Tensor, table_local: torch.Tensor, group, out_dtype,
                             scatter_rows: bool = False) -> torch.Tensor:
    """Embedding whose rows are sharded over `group`: look up the locally owned ids, zero the
    others, all-reduce - or, with `scatter_rows`, reduce-scatter into row blocks of the flattened
    tokens ([idx.numel() / world, C])."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rows = table_local.shape[0]
    lo = rank * rows
    mask = (idx >= lo) & (idx < lo + rows)
    local_idx = torch.where(mask, idx - lo, torch.zeros_like(idx))
    out = K.embedding(local_idx, table_local, out_dtype)
    out = out * mask.unsqueeze(-1).to(out.dtype)
    if scatter_rows:
        return scatter_sum_rows(out.reshape(-1, out.shape[-1]), group)
    return reduce_from_tp_region(out, group)


class _VocabParallelLinearCEFn(torch.autograd.Function):
    """Mean cross-entropy of ``x @ W_local^T`` with the vocabulary rows of W sharded over `group`,
    without keeping the logits: the tokens are processed in chunks; per chunk the ranks exchange only
    the per-token max and (sum-exp, target logit), and the chunk's logits are turned into their
    gradient and contracted into dX (this rank's partial sum over its vocabulary rows) and dW_local
    right away.  The reference gathers the full logits instead (models/gpt_model.py:296-300)."""

    @staticmethod
    def forward(ctx, x, weight_local, targets, group, ignore_index, chunk_tokens):
        fast = x.is_cuda and x.dtype == torch.bfloat16
        wb = K.bf16_weight(weight_local) if fast else weight_local.detach().to(x.dtype)
        T, Kd = x.shape
        v_loc = wb.shape[0]
        lo = dist.get_rank(group) * v_loc
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        valid = targets != ignore_index
        n_valid = valid.sum().clamp_min(1).float()
        dx = torch.empty_like(x) if need_grad else None
        dw = torch.zeros(v_loc, Kd, device=x.device, dtype=torch.float32) if need_grad else None
        loss_sum = torch.zeros((), device=x.device, dtype=torch.float32)
        chunk = min(chunk_tokens, T)
        for t0 in range(0, T, chunk):
            t1 = min(t0 + chunk, T)
            xc, tc, vc = x[t0:t1], targets[t0:t1], valid[t0:t1]
            lf = (gemm(xc, wb.t()) if fast else xc @ wb.t()).float()
            mx = lf.max(dim=-1).values
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
            ex = lf.sub_(mx.unsqueeze(-1)).exp_()
            mine = vc & (tc >= lo) & (tc < lo + v_loc)
            t_loc = torch.where(mine, tc - lo, torch.zeros_like(tc))
            # exp(target logit - max) of the locally owned targets; its log is the shifted target logit
            et = torch.where(mine, ex.gather(-1, t_loc.unsqueeze(-1)).squeeze(-1), torch.zeros_like(mx))
            stats = torch.stack([ex.sum(dim=-1), et])
            dist.all_reduce(stats, group=group)
            se, et = stats[0], stats[1]
            loss_sum += torch.where(vc, se.log() - et.clamp_min(1e-38).log(), torch.zeros_like(se)).sum()
            if need_grad:
                probs = ex.div_(se.unsqueeze(-1))
                probs.scatter_add_(-1, t_loc.unsqueeze(-1), -mine.to(probs.dtype).unsqueeze(-1))
                probs.mul_((vc.float() / n_valid).unsqueeze(-1))
                g = probs.to(x.dtype)
                if fast:
                    gemm(g, wb, out=dx[t0:t1])
                    gemm(g.t(), xc, out=dw, accumulate=True, split_k=1)
                else:
                    dx[t0:t1] = g @ wb
                    dw += (g.t() @ xc).float()
        if need_grad:
            ctx.save_for_backward(dx, dw)
            ctx.w_dtype = weight_local.dtype
        return loss_sum / n_valid

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        dxo = dx * dloss.to(dx.dtype) if ctx.needs_input_grad[0] else None
        dwo = (dw * dloss).to(ctx.w_dtype) if ctx.needs_input_grad[1] else None
        return dxo, dwo, None, None, None, None


def vocab_parallel_cross_entropy(x: torch.Tensor, weight_local: torch.Tensor, targets: torch.Tensor, group,
                                 ignore_index: int = -1, rows_sharded: bool = False,
                                 chunk_tokens: int = 8192) -> torch.Tensor:
    """Mean cross-entropy of ``x @ weight_local.T`` with the vocabulary sharded over `group`.  `x` is
    replicated, or (`rows_sharded`) this rank's row block of the flattened tokens."""
    x2 = x.reshape(-1, x.shape[-1])
    # every rank contributes the part of dX that comes from its vocabulary rows: summed by the
    # backward of the region function in front (all-reduce, or reduce-scatter into row blocks)
    x2 = gather_rows(x2, group) if rows_sharded else copy_to_tp_region(x2, group)
    return _VocabParallelLinearCEFn.apply(x2.contiguous(), weight_local, targets.reshape(-1).contiguous(), group,
                                          ignore_index, chunk_tokens)
