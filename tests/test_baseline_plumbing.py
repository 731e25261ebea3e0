"""Single-process plumbing on the small GPT of the benchmark plan: 4 layers, d_model 256, 4 heads,
MLP 4x, vocabulary 50304, sequence 256, batch 8, fp32, random-init weights, uniform-random token ids
from a seed.  One step of the reference's `DionReference` (rank_fraction 0.25, error feedback) and of
its `MuonReference` (5 quintic Newton-Schulz steps) on the gradients of that model, compared with
this library's optimizers on the same gradients: on the CPU (PyTorch paths) and, on a GPU, with the
CUDA kernels doing the work."""
import pytest
import torch

from dion_b200 import Dion, Muon, MuonReference
from dion_b200.models import GPT, GPTConfig

from _reference import load_reference

ref = load_reference()
needs_ref = pytest.mark.skipif(ref is None, reason="reference package not importable")


def _model_and_grads():
    torch.manual_seed(0)
    model = GPT(GPTConfig(sequence_len=256, vocab_size=50304, n_layer=4, n_head=4, n_embd=256))
    model.init_weights()
    g = torch.Generator().manual_seed(1234)
    idx = torch.randint(0, 50304, (8, 256), generator=g)
    tgt = torch.randint(0, 50304, (8, 256), generator=g)
    loss = model(idx, tgt)
    loss.backward()
    assert torch.isfinite(loss) and abs(loss.item() - 10.8) < 1.0   # about ln(50304) at initialisation
    mats = [p for p in model.transformer.h.parameters()]
    return model, mats


def _copies(mats, device):
    out = []
    for p in mats:
        q = torch.nn.Parameter(p.detach().clone().to(device))
        q.grad = p.grad.detach().clone().to(device)
        out.append(q)
    return out


def _check(ours, theirs, tol):
    for a, b in zip(ours, theirs):
        err = (a.detach().cpu().float() - b.detach().cpu().float()).abs().max().item()
        scale = b.detach().abs().max().item()
        assert err <= tol * scale, (tuple(a.shape), err, scale)


@needs_ref
@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_dion_step_matches_reference_dion_on_model_gradients(device):
    _, mats = _model_and_grads()
    P, Pr = _copies(mats, device), _copies(mats, "cpu")
    opt = Dion(P, lr=0.02, rank_fraction=0.25, weight_decay=0.01)
    opt_ref = ref.DionReference(Pr, lr=0.02, rank_fraction=0.25, weight_decay=0.01, qr_method="qr")
    for g in opt.param_groups:
        for p in g["params"]:
            opt._get_or_initialize_state(p, g)
    for p, pr in zip(P, Pr):
        opt_ref.state[pr] = {"momentum": torch.zeros_like(pr), "Q": opt.state[p]["Q"].detach().cpu().clone()}
    before = [p.detach().clone() for p in Pr]
    opt.step()
    opt_ref.step()
    assert any((a - b).abs().max() > 0 for a, b in zip(before, Pr))
    # fp32 states run as TF32 / 3xTF32 products on the GPU
    _check(P, Pr, 1e-5 if device == "cpu" else 2e-4)
    _check([opt.state[p]["momentum"] for p in P], [opt_ref.state[p]["momentum"] for p in Pr],
           1e-4 if device == "cpu" else 5e-3)


@needs_ref
@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_muon_step_matches_reference_muon_on_model_gradients(device):
    _, mats = _model_and_grads()
    # the reference's MuonReference (fixed quintic coefficients, 5 steps) against ours
    P, Pr = _copies(mats, "cpu"), _copies(mats, "cpu")
    MuonReference(P, lr=0.02, mu=0.95, ns_steps=5).step()
    ref.MuonReference(Pr, lr=0.02, mu=0.95, ns_steps=5).step()
    _check(P, Pr, 1e-5)
    # the batched Muon (Newton-Schulz in bf16; on the GPU the tcgen05 kernels) against the reference's
    P2, Pr2 = _copies(mats, device), _copies(mats, "cpu")
    Muon(P2, lr=0.02, mu=0.95, nesterov=True, adjust_lr="spectral_norm").step()
    ref.Muon(Pr2, lr=0.02, mu=0.95, nesterov=True, adjust_lr="spectral_norm", use_triton=False).step()
    _check(P2, Pr2, 2e-3 if device == "cpu" else 1e-2)
