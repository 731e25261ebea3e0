"""Llama-shaped decoder on CPU: forward against a plain PyTorch statement of the same block,
parameter grouping, and a few optimizer steps."""
import math

import torch
import torch.nn.functional as F

from dion_b200 import Dion, Muon
from dion_b200.models.llama import Llama, LlamaConfig, make_llama_param_groups
from dion_b200.ops import nn as K


def _cfg():
    return LlamaConfig(sequence_len=32, vocab_size=128, n_layer=2, n_head=4, n_kv_head=2, n_embd=32, ffn_dim=80)


def _plain_forward(model: Llama, idx: torch.Tensor) -> torch.Tensor:
    cfg = model.config
    hd = cfg.n_embd // cfg.n_head
    x = model.tok_embeddings.weight[idx]
    T = idx.shape[1]
    cos, sin = K.rotary_tables(T, hd, idx.device, cfg.rope_theta)
    cos, sin = cos.float()[None, :, None, :], sin.float()[None, :, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w

    def rope(v):
        a, b = v[..., : hd // 2], v[..., hd // 2:]
        return torch.cat([a * cos + b * sin, b * cos - a * sin], dim=-1)

    for layer in model.layers:
        at, ff = layer.attention, layer.feed_forward
        h = norm(x, layer.attention_norm.weight)
        B = h.shape[0]
        q = (h @ at.wq.weight.T).view(B, T, cfg.n_head, hd)
        k = (h @ at.wk.weight.T).view(B, T, cfg.n_kv_head, hd)
        v = (h @ at.wv.weight.T).view(B, T, cfg.n_kv_head, hd)
        q, k = rope(q), rope(k)
        rep = cfg.n_head // cfg.n_kv_head
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(hd)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        y = torch.einsum("bhts,bshd->bthd", s.softmax(-1), v).reshape(B, T, -1)
        x = x + y @ at.wo.weight.T
        h = norm(x, layer.ffn_norm.weight)
        x = x + (F.silu(h @ ff.w_gate.weight.T) * (h @ ff.w_up.weight.T)) @ ff.w_down.weight.T
    return norm(x, model.norm.weight) @ model.output.weight.T


def test_forward_matches_plain_pytorch():
    torch.manual_seed(0)
    model = Llama(_cfg())
    model.init_weights()
    with torch.no_grad():
        for m in model.modules():
            if hasattr(m, "eps"):
                m.weight.normal_(1.0, 0.1)  # gains away from one so that they matter
    idx = torch.randint(0, 128, (3, 32))
    logits = model(idx, torch.zeros_like(idx), return_logits=True)
    ref = _plain_forward(model, idx)
    torch.testing.assert_close(logits, ref, rtol=1e-4, atol=1e-4)
    loss = model(idx, idx)
    torch.testing.assert_close(loss, F.cross_entropy(ref.view(-1, 128), idx.view(-1)), rtol=1e-4, atol=1e-4)


def test_param_groups_route_matrices_and_scalars():
    model = Llama(_cfg())
    groups = make_llama_param_groups(model)
    assert "algorithm" not in groups[0] and all(p.ndim == 2 for p in groups[0]["params"])
    assert len(groups[0]["params"]) == 7 * 2
    rest = [p for g in groups[1:] for p in g["params"]]
    assert all(g["algorithm"] == "adamw" for g in groups[1:])
    assert len(groups[0]["params"]) + len(rest) == len(list(model.parameters()))


def test_dion_and_muon_reduce_the_loss():
    for make in (lambda g: Dion(g, lr=0.02, rank_fraction=0.5), lambda g: Muon(g, lr=0.02, nesterov=True)):
        torch.manual_seed(0)
        model = Llama(_cfg())
        model.init_weights()
        opt = make(make_llama_param_groups(model, lr=0.01))
        idx = torch.randint(0, 128, (4, 32))
        losses = []
        for _ in range(6):
            loss = model(idx, idx)
            loss.backward()
            opt.step()
            model.zero_grad(set_to_none=True)
            losses.append(loss.item())
        assert losses[-1] < losses[0] - 0.2, losses
