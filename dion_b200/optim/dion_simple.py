"""DionSimple: the single-device, educational form of Dion with Householder QR
(behaviour of dion/dion_simple.py:11-206)."""

from __future__ import annotations

from typing import Any, Dict, Tuple

import torch
from torch import Tensor
from torch.distributed.tensor import DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from ..ops import nn as nn_ops
from .scalar import adamw_update, lion_update


def dion_simple_update(X: Tensor, G: Tensor, M: Tensor, Q: Tensor, lr: float, mu: float, weight_decay: float,
                       epsilon: float = 1e-8) -> None:
    """One Dion step: M += G; P = qr(M Q); R = M^T P; M -= (1 - mu) P R^T;
    Q = colnorm(R); X = (1 - wd lr) X - lr sqrt(fan_out / fan_in) P Q^T."""
    M.add_(G)
    P, _ = torch.linalg.qr(M @ Q)
    R = M.T @ P
    M.addmm_(P, R.T, alpha=-(1 - mu))
    Q.copy_(R / (R.norm(dim=0, keepdim=True) + epsilon))
    fan_out, fan_in = X.shape
    X.mul_(1 - weight_decay * lr)
    X.addmm_(P, Q.T, alpha=-lr * (fan_out / fan_in) ** 0.5)


class DionSimple(Optimizer):
    """Fixed integer ``rank``; Q is always (fan_in, rank); DTensors are rejected."""

    def __init__(self, params: ParamsT, lr: float, mu: float = 0.95, betas: Tuple[float, float] = (0.9, 0.95),
                 weight_decay: float = 0.01, rank: int = 768, epsilon: float = 1e-8):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if mu < 0.0:
            raise ValueError(f"Invalid momentum factor (mu): {mu}")
        if len(betas) != 2 or betas[0] < 0.0 or betas[1] < 0.0:
            raise ValueError(f"Invalid betas: {betas}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        if rank < 1:
            raise ValueError(f"Invalid rank value: {rank}")
        defaults = dict(lr=lr, mu=mu, beta1=betas[0], beta2=betas[1], weight_decay=weight_decay, algorithm="dion",
                        step=0)
        super().__init__(params, defaults)
        self.rank = rank
        self.epsilon = epsilon
        for group in self.param_groups:
            if group["algorithm"] == "dion":
                for p in group["params"]:
                    if p.dim() != 2:
                        raise ValueError(f"Expected Dion parameters to be 2D tensor, but got {p.dim()}D.")
                    if isinstance(p, DTensor):
                        raise NotImplementedError(
                            "This version of Dion optimizer does not support distributed tensors.")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            algo = group["algorithm"]
            group["step"] += 1
            if algo not in ("dion", "adamw", "lion"):
                raise ValueError(f"Unknown algorithm: {algo}")
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    self._init_state(p, state, algo)
                if algo == "dion":
                    dion_simple_update(p, p.grad, state["momentum"], state["Q"], group["lr"], group["mu"],
                                       group["weight_decay"], self.epsilon)
                elif algo == "adamw":
                    adamw_update(p, p.grad, state["momentum"], state["variance"], group["lr"], group["beta1"],
                                 group["beta2"], group["weight_decay"], group["step"], self.epsilon)
                else:
                    lion_update(p, p.grad, state["momentum"], group["lr"], group["beta1"], group["beta2"],
                                group["weight_decay"])
                nn_ops.mark_shadow_stale(p)
        return loss

    def _init_state(self, p: Tensor, state: Dict[str, Any], algo: str) -> None:
        state["momentum"] = torch.zeros_like(p)
        if algo == "dion":
            r = min(self.rank, min(p.shape))
            state["Q"] = torch.randn((p.size(1), r), device=p.device, dtype=p.dtype)
        elif algo == "adamw":
            state["variance"] = torch.zeros_like(p)
