"""GPT (modded-nanoGPT style) with rotary attention, QK-norm, ReLU^2 MLP, weight-less
RMSNorm and untied embeddings.  Module and parameter names, initialisation, loss and the
parallelisation plan follow the reference (models/gpt_model.py:17-376), so checkpoints and
parameter groups interchange; the forward pass runs on the sm_100a kernels of
:mod:`dion_b200.ops.nn` (bf16 activations) when the model lives on a GPU and on plain
PyTorch otherwise.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, Replicate, Shard

from ..ops import nn as K
from ..parallel import tp as TP


@dataclass
class GPTConfig:
    sequence_len: int = 1024
    vocab_size: int = 50304
    n_layer: int = 2
    n_head: int = 6
    n_embd: int = 768


def _local(w: torch.Tensor) -> torch.Tensor:
    """Local shard of a (possibly tensor-parallel DTensor) parameter, differentiable."""
    return w.to_local() if isinstance(w, DTensor) else w


def _tp_group(w: torch.Tensor):
    """(process group, shard dim) when `w` is sharded over a tensor-parallel mesh dim."""
    if not isinstance(w, DTensor):
        return None, None
    for i, pl in enumerate(w.placements):
        if pl.is_shard() and w.device_mesh.size(i) > 1:
            return w.device_mesh.get_group(i), pl.dim
    return None, None


class Rotary(nn.Module):
    """cos/sin tables cached in bf16 per sequence length (models/gpt_model.py:26-51)."""

    def __init__(self, dim: int, base: float = 10000.0):
        super().__init__()
        self.dim = dim
        self.base = base
        self.inv_freq = None
        self.seq_len_cached = None
        self.cos_cached = None
        self.sin_cached = None

    def init_inv_freq(self):
        self.inv_freq = 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.dim))

    def tables(self, seq_len: int, device):
        if seq_len != self.seq_len_cached or self.cos_cached is None or self.cos_cached.device != torch.device(device):
            self.seq_len_cached = seq_len
            self.cos_cached, self.sin_cached = K.rotary_tables(seq_len, self.dim, device, self.base)
        return self.cos_cached, self.sin_cached

    def forward(self, x):
        cos, sin = self.tables(x.shape[1], x.device)
        return cos[None, :, None, :], sin[None, :, None, :]


class CausalSelfAttention(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.n_head = config.n_head
        self.n_embd = config.n_embd
        assert self.n_embd % self.n_head == 0
        self.head_dim = self.n_embd // self.n_head
        self.c_q = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_k = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_v = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.c_proj = nn.Linear(self.n_embd, self.n_embd, bias=False)
        self.rotary = Rotary(self.head_dim)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, bt=None) -> torch.Tensor:
        """h: normalised input [B, T, C]; returns residual + attention output.  With `bt` = (B, T) the
        model runs sequence-parallel: h and residual are this rank's row block [B * T / tp, C] of the
        flattened tokens, gathered in front of the q / k / v products and scattered after c_proj."""
        group, _ = _tp_group(self.c_q.weight)
        if bt is not None:
            B, T = bt
            q, k, v = TP.gather_linear(h, group, _local(self.c_q.weight), _local(self.c_k.weight),
                                       _local(self.c_v.weight))
        else:
            B, T, _ = h.shape
            if group is not None:
                h = TP.copy_to_tp_region(h, group)
            q, k, v = K.linear_fanout(h, _local(self.c_q.weight), _local(self.c_k.weight), _local(self.c_v.weight))
        q, k, v = (t.view(B, T, -1, self.head_dim) for t in (q, k, v))
        cos, sin = self.rotary.tables(T, h.device)
        q, k = K.rope_qknorm(q, k, cos, sin)
        y = K.causal_attention(q, k, v)
        if bt is not None:
            return TP.linear_scatter(y.reshape(B * T, -1), _local(self.c_proj.weight), group, residual)
        if group is not None:
            return residual + TP.row_parallel_linear(y, _local(self.c_proj.weight), group)
        return K.linear(y, _local(self.c_proj.weight), residual=residual)


class MLP(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, bias=False)
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=False)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, bt=None) -> torch.Tensor:
        group, _ = _tp_group(self.c_fc.weight)
        if bt is not None:
            # sequence-parallel: all-gather -> c_fc, c_proj -> reduce-scatter (+ residual) on row blocks
            (pre,) = TP.gather_linear(h, group, _local(self.c_fc.weight))
            return TP.linear_scatter(K.relu2(pre), _local(self.c_proj.weight), group, residual)
        if group is not None:
            # column-parallel c_fc (its input gradient is summed over the group by a fused
            # GEMM -> all-reduce), row-parallel c_proj (its output likewise)
            u = K.relu2(TP.column_parallel_linear(h, _local(self.c_fc.weight), group))
            return residual + TP.row_parallel_linear(u, _local(self.c_proj.weight), group)
        return K.mlp(h, _local(self.c_fc.weight), _local(self.c_proj.weight), residual)


class Block(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.attn = CausalSelfAttention(config)
        self.mlp = MLP(config)

    def forward(self, x: torch.Tensor, bt=None) -> torch.Tensor:
        x, h = K.norm_branch(x)
        x = self.attn(h, x, bt)
        x, h = K.norm_branch(x)
        x = self.mlp(h, x, bt)
        return x


class GPT(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.config = config
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            h=nn.ModuleList([Block(config) for _ in range(config.n_layer)]),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        # activations: bf16 on GPUs (the kernels' dtype), parameter dtype elsewhere
        self.activation_dtype: Optional[torch.dtype] = None
        # tensor parallelism with the residual stream sharded over the tokens (set by the TP plan)
        self.sequence_parallel = False

    # -- initialisation (models/gpt_model.py:140-157)
    def init_weights(self):
        self.apply(self._init_weights)

    def _init_weights(self, module):
        if isinstance(module, nn.Linear):
            fan_out, fan_in = module.weight.size(0), module.weight.size(1)
            std = 1.0 / math.sqrt(fan_in) * min(1.0, math.sqrt(fan_out / fan_in))
            torch.nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                torch.nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=1.0)
        elif isinstance(module, Rotary):
            module.init_inv_freq()

    def _act_dtype(self, device) -> torch.dtype:
        if self.activation_dtype is not None:
            return self.activation_dtype
        return torch.bfloat16 if torch.device(device).type == "cuda" else self.lm_head.weight.dtype

    # -- forward
    def forward(self, idx, targets=None, return_logits=False):
        bt = self._sequence_parallel_shape(idx)
        x = self._forward_emb(idx, bt)
        return self._forward(x, targets, return_logits, bt)

    def _sequence_parallel_shape(self, idx):
        """(B, T) when this call runs sequence-parallel: the TP plan asked for it and the flattened
        tokens split into row blocks of a multiple of 8 rows."""
        if not self.sequence_parallel:
            return None
        group, _ = _tp_group(self.transformer.wte.weight)
        if group is None:
            return None
        world = group.size()
        n = idx.numel()
        return tuple(idx.shape) if n % world == 0 and (n // world) % 8 == 0 else None

    def _forward_emb(self, idx, bt=None):
        w = self.transformer.wte.weight
        group, _ = _tp_group(w)
        dtype = self._act_dtype(idx.device)
        if group is not None:
            return TP.vocab_parallel_embedding(idx, _local(w), group, dtype, scatter_rows=bt is not None)
        return K.embedding(idx, _local(w), dtype)

    def _forward(self, x, targets, return_logits, bt=None):
        for block in self.transformer.h:
            x = block(x, bt) if bt is not None else block(x)
        x = K.rms_norm(x)
        w = self.lm_head.weight
        group, _ = _tp_group(w)
        if targets is not None and not return_logits:
            if bt is not None:
                return TP.vocab_parallel_cross_entropy(x, _local(w), targets, group, ignore_index=-1, rows_sharded=True)
            if group is not None:
                return TP.vocab_parallel_cross_entropy(x, _local(w), targets, group, ignore_index=-1)
            return K.linear_cross_entropy(x, _local(w), targets, ignore_index=-1)
        if bt is not None:
            if targets is None and not return_logits:
                return None
            # the logits path works on all tokens: gather the row blocks (the backward scatters the sum)
            x = TP.gather_rows(x, group).view(bt[0], bt[1], -1)
            if targets is None:
                x = x[:, [-1], :]
            return TP.gather_from_tp_region(K.linear(x, _local(w)), group).float()
        if targets is None:
            if not return_logits:
                return None  # no targets, no logits requested: there is no loss to report
            x = x[:, [-1], :]  # only the last position is needed for sampling
        if group is not None:
            logits = TP.gather_from_tp_region(K.linear(TP.copy_to_tp_region(x, group), _local(w)), group)
        else:
            logits = K.linear(x, _local(w))
        return logits.float()

    def compile(self):  # noqa: A003 - API parity with the reference (models/gpt_model.py:195-200)
        """The reference compiles the forward with torch.compile; here the forward already runs
        on hand-written kernels, so this is a no-op kept for API compatibility."""
        return self

    def refresh_weights(self) -> None:
        """Refresh the bf16 copies of all fp32 parameters with one multi-tensor launch."""
        K.refresh_bf16_weights([_local(p) for p in self.parameters() if not isinstance(p, DTensor)])

    @torch.no_grad()
    def generate(self, input_ids: torch.LongTensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None) -> torch.LongTensor:
        """Sample `max_new_tokens` tokens, feeding at most `sequence_len` tokens of context."""
        idx = input_ids
        for _ in range(max_new_tokens):
            ctx = idx if idx.size(1) <= self.config.sequence_len else idx[:, -self.config.sequence_len:]
            logits = self(ctx, targets=None, return_logits=True)
            nxt = logits[:, -1, :] / temperature
            if top_k is not None:
                v, _ = torch.topk(nxt, min(top_k, nxt.size(-1)))
                nxt[nxt < v[:, [-1]]] = -float("Inf")
            probs = F.softmax(nxt, dim=-1)
            idx = torch.cat([idx, torch.multinomial(probs, num_samples=1)], dim=1)
        return idx


# --------------------------------------------------------------------------- parallelisation plan

def parallelize_gpt_model(model: GPT, device_mesh: DeviceMesh, dp_name: Optional[str] = "dp",
                          fs_name: Optional[str] = "fs", tp_name: Optional[str] = "tp",
                          fsdp_reshard_after_forward: bool = True, sequence_parallel: bool = False):
    """Shard `model` in place over the named mesh dimensions: tensor parallel first, then
    FSDP2 over ``fs`` (or over ``(dp, fs)`` as hybrid sharding when ``dp_name`` is given)
    (models/gpt_model.py:236-288).  `sequence_parallel` keeps the residual stream sharded over the
    tokens between the tensor-parallel products (all-gather -> GEMM, GEMM -> reduce-scatter) instead of
    all-reducing every row-parallel output."""
    names = [n for n in (dp_name, fs_name, tp_name) if n]
    if not names:
        raise ValueError("At least one of dp_name, fs_name, or tp_name must be provided")
    if dp_name and not fs_name:
        raise ValueError("Data parallelism with fully_shard() requires 2D FSDP mesh")
    if device_mesh.ndim < len(names):
        raise ValueError(f"Expected {len(names)}-D device mesh {names}, but got mesh with {device_mesh.ndim} dimensions")
    actual = list(device_mesh.mesh_dim_names)
    if not all(n in actual for n in names):
        raise ValueError(f"Expected device mesh to have names {names}, but got {actual}")
    if tp_name:
        tp_mesh = device_mesh[tp_name]
        if tp_mesh.size() > 1:
            _apply_tp(model, tp_mesh)
            model.sequence_parallel = bool(sequence_parallel)
    if fs_name:
        fsdp_mesh = device_mesh[fs_name] if not dp_name else device_mesh[dp_name, fs_name]
        _apply_fsdp(model, fsdp_mesh, fsdp_reshard_after_forward)


def _apply_tp(model: GPT, tp_mesh: DeviceMesh):
    """Column-parallel c_q/c_k/c_v/c_fc and lm_head (weights Shard(0)), row-parallel
    attn.c_proj/mlp.c_proj (Shard(1)), vocabulary-sharded embedding (Shard(0))
    (models/gpt_model.py:291-333).  The forward pass issues its own collectives on the local
    shards; `parallelize_module` is only used to distribute the parameters."""
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    parallelize_module(model, tp_mesh, parallelize_plan={
        "transformer.wte": RowwiseParallel(input_layouts=Replicate(), output_layouts=Replicate()),
        "lm_head": ColwiseParallel(input_layouts=Replicate(), output_layouts=Replicate()),
    })
    for block in model.transformer.h:
        parallelize_module(block, tp_mesh, parallelize_plan={
            "attn.c_q": ColwiseParallel(),
            "attn.c_k": ColwiseParallel(),
            "attn.c_v": ColwiseParallel(),
            "attn.c_proj": RowwiseParallel(),
            "mlp.c_fc": ColwiseParallel(),
            "mlp.c_proj": RowwiseParallel(),
        })
        assert block.attn.n_head % tp_mesh.size() == 0, \
            f"attn.n_head {block.attn.n_head} must be divisible by TP size {tp_mesh.size()}"
        block.attn.n_head = block.attn.n_head // tp_mesh.size()


def _apply_fsdp(model: GPT, fsdp_mesh: DeviceMesh, reshard_after_forward: bool = True):
    """FSDP2 per block and at the root, bf16 parameters / fp32 gradient reduction, sharding
    the dimension TP does not shard: Shard(1) for column-parallel weights, Shard(0) for
    row-parallel ones, Shard(1) for the embedding and lm_head (models/gpt_model.py:336-376)."""
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    mp_policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for block in model.transformer.h:
        shard_map = {
            block.attn.c_q.weight: Shard(1),
            block.attn.c_k.weight: Shard(1),
            block.attn.c_v.weight: Shard(1),
            block.attn.c_proj.weight: Shard(0),
            block.mlp.c_fc.weight: Shard(1),
            block.mlp.c_proj.weight: Shard(0),
        }
        fully_shard(block, mesh=fsdp_mesh, shard_placement_fn=lambda p, m=shard_map: m.get(p), mp_policy=mp_policy,
                    reshard_after_forward=reshard_after_forward)
    shard_map = {model.transformer.wte.weight: Shard(1), model.lm_head.weight: Shard(1)}
    fully_shard(model, mesh=fsdp_mesh, mp_policy=mp_policy, shard_placement_fn=lambda p, m=shard_map: m.get(p),
                reshard_after_forward=False)
    # all-gather / reduce-scatter as in-tree kernels over symmetric memory where the group allows it
    from ..parallel import fsdp_comm

    fsdp_comm.install(model)
