"""The reference's ``models.gpt_model`` import path (models/gpt_model.py:18-376): the GPT model, its building
blocks and its parallelisation plan under the reference's names."""

from __future__ import annotations

import torch

from ..ops import nn as _nn
from .gpt import (  # noqa: F401
    GPT,
    MLP,
    Block,
    CausalSelfAttention,
    GPTConfig,
    Rotary,
    _apply_fsdp,
    _apply_tp,
    parallelize_gpt_model,
)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x: [B, T, H, D]`` with half-split pairs, ``cos`` / ``sin`` holding one row of
    ``D / 2`` values per position, given as ``[T, D/2]`` or broadcastable ``[1, T, 1, D/2]``
    (models/gpt_model.py:54-61).  CUDA bf16 inputs with head sizes 64 and 128 run the rotary kernel."""
    if x.ndim != 4:
        raise ValueError("expected [batch, tokens, heads, head_dim]")
    T, half = x.shape[1], x.shape[3] // 2
    cos2, sin2 = cos.reshape(-1, half), sin.reshape(-1, half)
    if cos2.shape[0] < T or sin2.shape[0] < T:
        raise ValueError("cos / sin hold fewer positions than x has tokens")
    return _nn.rope(x, cos2.to(x.dtype).contiguous(), sin2.to(x.dtype).contiguous())
