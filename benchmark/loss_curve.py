"""Loss curves of this package and of the unmodified reference on the same learnable synthetic data, from the
same initial weights: a check that the differences in numerics (bf16 residual stream and norms here, fp32
under the reference's autocast; Cholesky-QR orthonormalisation here, sketch + Householder QR there; tensor-core
TF32 products for fp32 states) do not change how training progresses.

    python benchmark/loss_curve.py --impl ours      --steps 300 --json ours.json
    python benchmark/loss_curve.py --impl reference --steps 300 --json ref.json
    python benchmark/loss_curve.py --compare ours.json ref.json

Data: a fixed random first-order Markov chain over `--states` tokens (every token has `--fanout` equally likely
successors), embedded in the 50304-token vocabulary; the best achievable loss is log(fanout).  Batches are
drawn on the host from a seeded generator, so both arms see the same tokens.  Model: GPT-160M (12 layers,
d_model 768, 12 heads), Dion rank_fraction 1.0 + Lion as in the headline benchmark, bf16 optimizer states, one
GPU.  Initial weights: drawn once by this package's `GPT.init_weights` under a fixed seed and loaded into both
models (parameter names are the same).  `--tiny` shrinks everything for a CPU smoke run.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch


def markov_batches(steps: int, batch: int, seq: int, states: int, fanout: int, vocab: int, seed: int):
    """`steps` pairs (x, y) of int64 [batch, seq] host tensors from one fixed chain."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randperm(vocab, generator=g)[:states]                    # which vocabulary entries the chain uses
    succ = torch.randint(0, states, (states, fanout), generator=g)       # successors of every state
    out = []
    for _ in range(steps):
        s = torch.randint(0, states, (batch,), generator=g)
        choice = torch.randint(0, fanout, (batch, seq + 1), generator=g)
        toks = torch.empty(batch, seq + 1, dtype=torch.int64)
        for t in range(seq + 1):
            toks[:, t] = s
            s = succ[s, choice[:, t]]
        toks = ids[toks]
        out.append((toks[:, :-1].contiguous(), toks[:, 1:].contiguous()))
    return out


def compare(paths):
    runs = [json.load(open(p)) for p in paths]
    print("| step | " + " | ".join(r["impl"] for r in runs) + " |")
    print("|---|" + "---|" * len(runs))
    n = min(len(r["losses"]) for r in runs)
    for i in list(range(0, n, max(n // 15, 1))) + [n - 1]:
        print(f"| {i + 1} | " + " | ".join(f"{r['losses'][i]:.4f}" for r in runs) + " |")
    tail = [sum(r["losses"][n - 20:n]) / 20 for r in runs]
    print("mean of the last 20 steps: " + ", ".join(f"{r['impl']} {t:.4f}" for r, t in zip(runs, tail))
          + f"; floor log(fanout) = {math.log(runs[0]['fanout']):.4f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--states", type=int, default=2048)
    ap.add_argument("--fanout", type=int, default=4)
    ap.add_argument("--lr", type=float, default=0.02)
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--compare", nargs="+", default=None, metavar="RUN.json")
    a = ap.parse_args()
    if a.compare:
        compare(a.compare)
        return
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    dims = dict(n_layer=2, n_head=4, n_embd=64, seq=64, vocab=512) if a.tiny else \
        dict(n_layer=12, n_head=12, n_embd=768, seq=1024, vocab=50304)
    states = min(a.states, dims["vocab"])
    data = markov_batches(a.steps, a.batch, dims["seq"], states, a.fanout, dims["vocab"], seed=99)

    # initial weights: this package's initialisation, on the host, shared by both arms
    from dion_b200.models import GPT, GPTConfig

    torch.manual_seed(4321)
    init_model = GPT(GPTConfig(sequence_len=dims["seq"], vocab_size=dims["vocab"], n_layer=dims["n_layer"],
                               n_head=dims["n_head"], n_embd=dims["n_embd"]))
    init_model.init_weights()
    init = {k: v.detach().clone() for k, v in init_model.state_dict().items()}
    del init_model

    def groups_of(model):
        return [dict(params=list(model.transformer.h.parameters())),
                dict(params=list(model.transformer.wte.parameters()), algorithm="lion", lr=a.lr, betas=(0.95, 0.98),
                     weight_decay=0),
                dict(params=list(model.lm_head.parameters()), algorithm="lion", lr=a.lr / math.sqrt(dims["n_embd"]),
                     betas=(0.95, 0.98), weight_decay=0)]

    bf = torch.bfloat16
    if a.impl == "ours":
        from dion_b200 import Dion, DionMixedPrecisionConfig

        model = GPT(GPTConfig(sequence_len=dims["seq"], vocab_size=dims["vocab"], n_layer=dims["n_layer"],
                              n_head=dims["n_head"], n_embd=dims["n_embd"])).to(dev)
        model.load_state_dict(init)
        opt = Dion(groups_of(model), lr=a.lr, mu=0.95, weight_decay=0.01, rank_fraction=1.0,
                   mixed_precision_config=DionMixedPrecisionConfig(momentum_dtype=bf, variance_dtype=bf, Q_dtype=bf))

        def step(x, y):
            loss = model(x, y)
            loss.backward()
            opt.step()
            model.zero_grad(set_to_none=True)
            return loss.detach()
    else:
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "dion")) or not os.path.isdir(os.path.join(ref_dir, "models")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
            return
        from dion_b200.utils.compilers import ensure_openmp_cxx

        ensure_openmp_cxx()
        sys.path.insert(0, ref_dir)
        for name in [m for m in sys.modules if m == "dion" or m.startswith("dion.")]:
            del sys.modules[name]
        from dion import Dion as RefDion, DionMixedPrecisionConfig as RefMP
        from models.gpt_model import GPT as RefGPT, GPTConfig as RefCfg

        torch._dynamo.config.cache_size_limit = 100
        if hasattr(torch._dynamo.config, "recompile_limit"):
            torch._dynamo.config.recompile_limit = 100
        model = RefGPT(RefCfg(sequence_len=dims["seq"], vocab_size=dims["vocab"], n_layer=dims["n_layer"],
                              n_head=dims["n_head"], n_embd=dims["n_embd"])).to(dev)
        model.init_weights()                 # also fills the rotary frequencies, which are no parameters
        model.load_state_dict(init)
        if cuda:
            model.compile()
        opt = RefDion(groups_of(model), lr=a.lr, mu=0.95, weight_decay=0.01, rank_fraction=1.0,
                      mixed_precision_config=RefMP(momentum_dtype=bf, variance_dtype=bf, Q_dtype=bf))
        autocast = torch.amp.autocast(device_type=dev.type, dtype=bf)

        def step(x, y):
            with autocast:
                loss = model(x, y)
            loss.backward()
            opt.step()
            model.zero_grad(set_to_none=True)
            return loss.detach()

    losses = []
    for x, y in data:
        losses.append(step(x.to(dev), y.to(dev)))
    losses = [float(l) for l in torch.stack(losses).float().cpu()]
    rec = {"impl": a.impl, "steps": a.steps, "batch": a.batch, "seq_len": dims["seq"], "states": states,
           "fanout": a.fanout, "lr": a.lr, "losses": losses}
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rec, f)
    print(json.dumps({k: v for k, v in rec.items() if k != "losses"} | {"first": losses[0], "last": losses[-1],
                                                                      "mean_last_20": sum(losses[-20:]) / min(20, len(losses))}))


if __name__ == "__main__":
    main()
