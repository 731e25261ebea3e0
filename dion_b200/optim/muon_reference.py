"""MuonReference (Moonlight-style per-parameter Muon with in-class AdamW / Lion) and
MuonKellerJordan (round-robin ownership + flat all-reduce).  Behaviour and state layout of
dion/muon_reference.py:10-337; these are the readable oracles for the batched Muon."""

from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch.distributed.tensor import DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from ..ops import nn as nn_ops
from .newton_schulz import newton_schulz_torch

_FIXED = (3.4445, -4.7750, 2.0315)


def zeropower_fixed_coeffs(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Newton-Schulz with one coefficient triple repeated `steps` times (2-D input)."""
    assert G.dim() == 2, "Expected 2D tensor"
    return newton_schulz_torch(G, eps, coeffs=(_FIXED,) * steps)


class MuonReference(Optimizer):
    def __init__(self, params: ParamsT, lr: float = 1e-3, mu: float = 0.95, betas: Tuple[float, float] = (0.95, 0.95),
                 weight_decay: float = 0.1, epsilon: float = 1e-8, nesterov: bool = True,
                 adjust_lr: Optional[str] = "spectral_norm", ns_steps: int = 5):
        if adjust_lr not in ("spectral_norm", "rms_norm", None):
            raise ValueError(f"Invalid adjust_lr value: {adjust_lr}. Must be 'spectral_norm', 'rms_norm', or None.")
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=mu, nesterov=nesterov, ns_steps=ns_steps,
                        adjust_lr=adjust_lr, betas=betas, epsilon=epsilon)
        if isinstance(params, dict):
            params = [params]
        params = list(params)
        super().__init__(params, defaults)
        # remember which algorithm every parameter uses (kept in the state, like the reference)
        for entry in params:
            if isinstance(entry, dict):
                algo = entry.get("algorithm", "muon")
                if algo not in ("muon", "adamw", "lion"):
                    raise ValueError(f"Unknown algorithm: {algo}")
                members = entry["params"]
                members = [members] if isinstance(members, torch.Tensor) else list(members)
            else:
                algo = "muon"
                if isinstance(entry, torch.Tensor):
                    members = [entry]
                elif isinstance(entry, tuple) and len(entry) == 2:
                    members = [entry[1]]
                else:
                    raise ValueError(f"Invalid parameter type: {type(entry)}")
            for p in members:
                self.state[p]["algorithm"] = algo
                if algo == "muon" and p.ndim != 2:
                    raise ValueError(f"Muon requires 2D parameters, but got {p.ndim}D")

    @staticmethod
    def _scaled_lr(mode, lr, shape):
        if mode is None:
            return lr
        if mode == "spectral_norm":
            return lr * math.sqrt(shape[0] / shape[1])
        if mode == "rms_norm":
            return lr * 0.2 * math.sqrt(max(shape[0], shape[1]))
        raise ValueError(f"Unknown adjust_lr value: {mode}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd, eps = group["lr"], group["weight_decay"], group["epsilon"]
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                state = self.state[p]
                algo = state["algorithm"]
                if algo == "muon":
                    if g.ndim > 2:
                        g = g.view(g.size(0), -1)
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(g)
                    buf = state["momentum_buffer"]
                    buf.mul_(group["momentum"]).add_(g)
                    g = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    if isinstance(g, DTensor):
                        u_full = zeropower_fixed_coeffs(g.full_tensor(), steps=group["ns_steps"], eps=eps)
                        u = DTensor.from_local(u_full, device_mesh=g.device_mesh, placements=None,
                                               run_check=False).redistribute(placements=g.placements)
                    else:
                        u = zeropower_fixed_coeffs(g, steps=group["ns_steps"], eps=eps)
                    p.mul_(1 - lr * wd)
                    p.add_(u.to(p.dtype), alpha=-self._scaled_lr(group["adjust_lr"], lr, p.shape))
                elif algo == "adamw":
                    if "step" not in state:
                        state["step"] = 0
                        state["moment1"] = torch.zeros_like(g)
                        state["moment2"] = torch.zeros_like(g)
                    state["step"] += 1
                    t = state["step"]
                    m1, m2 = state["moment1"], state["moment2"]
                    m1.lerp_(g, 1 - beta1)
                    m2.lerp_(g.square(), 1 - beta2)
                    upd = m1 / (eps + m2.sqrt())
                    scale = (1 - beta1 ** t) / (1 - beta2 ** t) ** 0.5
                    p.mul_(1 - lr * wd)
                    p.add_(upd, alpha=-lr / scale)
                elif algo == "lion":
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(p)
                    buf = state["momentum_buffer"]
                    upd = buf.lerp(g, 1 - beta1).sign_()
                    buf.lerp_(g, 1 - beta2)
                    p.mul_(1 - lr * wd)
                    p.add_(upd, alpha=-lr)
                else:
                    raise ValueError(f"Unknown algorithm: {algo}")
                nn_ops.mark_shadow_stale(p)
        return loss


class MuonKellerJordan(Optimizer):
    """Every rank orthogonalises the parameters ``i % world == rank`` and the updates are
    combined with one flat bf16 all-reduce (modded-nanogpt scheme)."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps))
        for group in self.param_groups:
            for p in group["params"]:
                if isinstance(p, DTensor):
                    raise NotImplementedError("DTensor parameters not supported.")

    @torch.no_grad()
    def step(self):
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        for group in self.param_groups:
            params = group["params"]
            total = sum(p.numel() for p in params)
            flat = torch.zeros(total, device=params[0].device, dtype=torch.bfloat16)
            off = 0
            for i, p in enumerate(params):
                if i % world == rank:
                    g = p.grad
                    assert g is not None, "Gradient is None"
                    state = self.state[p]
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(g)
                    buf = state["momentum_buffer"]
                    buf.mul_(group["momentum"]).add_(g)
                    g = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    u = zeropower_fixed_coeffs(g, steps=group["ns_steps"])
                    u = u * (g.size(0) / g.size(1)) ** 0.5
                    flat[off:off + p.numel()] = u.flatten()
                off += p.numel()
            if world > 1 and dist.is_initialized():
                dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            off = 0
            for p in params:
                p.add_(flat[off:off + p.numel()].view_as(p).type_as(p), alpha=-group["lr"])
                off += p.numel()
                nn_ops.mark_shadow_stale(p)
