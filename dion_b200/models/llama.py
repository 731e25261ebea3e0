"""Llama-3-shaped decoder (grouped-query attention, SwiGLU feed-forward, RMSNorm with
learnable gains, rotary embedding, untied embedding / lm_head) on the kernels of
:mod:`dion_b200.ops.nn`.  The reference ships no Llama model; this one exists so that the
optimizers can be exercised and benchmarked at the 8B shape (4096 x 4096, 1024 x 4096,
14336 x 4096 and 4096 x 14336 matrices) under FSDP2.

All 2-D block weights go to Dion / Muon; the 1-D norm gains, the embedding and the lm_head
go to the scalar optimizer, as `make_llama_param_groups` arranges.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import Shard

from ..ops import nn as K


@dataclass
class LlamaConfig:
    sequence_len: int = 4096
    vocab_size: int = 128256
    n_layer: int = 32
    n_head: int = 32
    n_kv_head: int = 8
    n_embd: int = 4096
    ffn_dim: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5

    @staticmethod
    def llama3_8b(**overrides) -> "LlamaConfig":
        return LlamaConfig(**overrides)


class RMSNormGain(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rms_norm_gain(x, self.weight, self.eps)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_head, self.n_kv_head = cfg.n_head, cfg.n_kv_head
        self.head_dim = cfg.n_embd // cfg.n_head
        self.wq = nn.Linear(cfg.n_embd, cfg.n_head * self.head_dim, bias=False)
        self.wk = nn.Linear(cfg.n_embd, cfg.n_kv_head * self.head_dim, bias=False)
        self.wv = nn.Linear(cfg.n_embd, cfg.n_kv_head * self.head_dim, bias=False)
        self.wo = nn.Linear(cfg.n_head * self.head_dim, cfg.n_embd, bias=False)
        self.rope_theta = cfg.rope_theta
        self._tables = None

    def _rope(self, T: int, device):
        if self._tables is None or self._tables[0].shape[0] != T or self._tables[0].device != torch.device(device):
            self._tables = K.rotary_tables(T, self.head_dim, device, self.rope_theta)
        return self._tables

    def forward(self, h: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        B, T, _ = h.shape
        q = K.linear(h, self.wq.weight).view(B, T, self.n_head, self.head_dim)
        k = K.linear(h, self.wk.weight).view(B, T, self.n_kv_head, self.head_dim)
        v = K.linear(h, self.wv.weight).view(B, T, self.n_kv_head, self.head_dim)
        cos, sin = self._rope(T, h.device)
        q = K.rope(q, cos, sin)
        k = K.rope(k, cos, sin)
        y = K.causal_attention(q, k, v)
        return K.linear(y, self.wo.weight, residual=residual)


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w_gate = nn.Linear(cfg.n_embd, cfg.ffn_dim, bias=False)
        self.w_up = nn.Linear(cfg.n_embd, cfg.ffn_dim, bias=False)
        self.w_down = nn.Linear(cfg.ffn_dim, cfg.n_embd, bias=False)

    def forward(self, h: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        g = K.linear(h, self.w_gate.weight)
        u = K.linear(h, self.w_up.weight)
        return K.linear(K.swiglu(g, u), self.w_down.weight, residual=residual)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attention_norm = RMSNormGain(cfg.n_embd, cfg.norm_eps)
        self.attention = LlamaAttention(cfg)
        self.ffn_norm = RMSNormGain(cfg.n_embd, cfg.norm_eps)
        self.feed_forward = LlamaMLP(cfg)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.attention(self.attention_norm(x), x)
        x = self.feed_forward(self.ffn_norm(x), x)
        return x


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.n_embd)
        self.layers = nn.ModuleList([LlamaBlock(cfg) for _ in range(cfg.n_layer)])
        self.norm = RMSNormGain(cfg.n_embd, cfg.norm_eps)
        self.output = nn.Linear(cfg.n_embd, cfg.vocab_size, bias=False)

    def init_weights(self, std: float = 0.02) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=std)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, mean=0.0, std=1.0)
            elif isinstance(m, RMSNormGain):
                nn.init.ones_(m.weight)

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None, return_logits: bool = False):
        dtype = torch.bfloat16 if idx.is_cuda else self.output.weight.dtype
        x = K.embedding(idx, self.tok_embeddings.weight, dtype)
        for layer in self.layers:
            x = layer(x)
        x = self.norm(x)
        if targets is not None and not return_logits:
            return K.linear_cross_entropy(x, self.output.weight, targets, ignore_index=-1)
        if targets is None:
            if not return_logits:
                return None
            x = x[:, [-1], :]
        return K.linear(x, self.output.weight).float()


def make_llama_param_groups(model: Llama, scalar_opt: str = "adamw", lr: float = 0.01) -> List[dict]:
    """Matrices of the blocks -> default (Dion / Muon) group; gains, embedding, lm_head ->
    the scalar optimizer, no weight decay."""
    matrices = [p for layer in model.layers for p in layer.parameters() if p.ndim == 2]
    gains = [p for p in model.parameters() if p.ndim == 1]
    return [
        dict(params=matrices),
        dict(params=gains, algorithm=scalar_opt, lr=lr, weight_decay=0),
        dict(params=list(model.tok_embeddings.parameters()), algorithm=scalar_opt, lr=lr, weight_decay=0),
        dict(params=list(model.output.parameters()), algorithm=scalar_opt,
             lr=lr / math.sqrt(model.config.n_embd), weight_decay=0),
    ]


def parallelize_llama_model(model: Llama, fsdp_mesh: DeviceMesh, reshard_after_forward: bool = True) -> None:
    """FSDP2 per block with bf16 parameters / fp32 reduction.  Every matrix is sharded along
    its *long* dimension (rows of gate/up, columns of down), so that Dion's P factor - the
    thing that is reduced, orthonormalised and gathered - spans the short dimension."""
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        ff, at = layer.feed_forward, layer.attention
        shard = {ff.w_gate.weight: Shard(0), ff.w_up.weight: Shard(0), ff.w_down.weight: Shard(1),
                 at.wq.weight: Shard(1), at.wk.weight: Shard(1), at.wv.weight: Shard(1), at.wo.weight: Shard(0)}
        fully_shard(layer, mesh=fsdp_mesh, mp_policy=mp, reshard_after_forward=reshard_after_forward,
                    shard_placement_fn=lambda p, m=shard: m.get(p))
    top = {model.tok_embeddings.weight: Shard(1), model.output.weight: Shard(1)}
    fully_shard(model, mesh=fsdp_mesh, mp_policy=mp, reshard_after_forward=False,
                shard_placement_fn=lambda p, m=top: m.get(p))
    from ..parallel import fsdp_comm

    fsdp_comm.install(model)
