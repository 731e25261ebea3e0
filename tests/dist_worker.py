"""Multi-process test cases, launched by tests/test_distributed.py through torchrun.
Each case runs on every rank (CUDA + NCCL when GPUs are available, CPU + gloo otherwise)
and compares against a single-process computation of the same thing.  Exit code 0 = pass."""
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

CUDA = torch.cuda.is_available() and os.environ.get("DION_TEST_FORCE_CPU", "0") != "1"
RANK = int(os.environ["RANK"])
WORLD = int(os.environ["WORLD_SIZE"])
LOCAL = int(os.environ.get("LOCAL_RANK", "0"))
DEV = torch.device("cuda", LOCAL) if CUDA else torch.device("cpu")

SHAPES = [(64, 32), (32, 64), (64, 64), (64, 32), (32, 64), (64, 64), (128, 32)]


def init():
    if CUDA:
        torch.cuda.set_device(LOCAL)
        dist.init_process_group("nccl", device_id=DEV)
    else:
        dist.init_process_group("gloo")


# Soft mode (DION_TEST_SOFT_FAIL=1): a failed check is recorded instead of ending the rank at once, every
# rank runs to the end, the ranks agree on the verdict and leave in order, and only then does the
# process exit non-zero.  It is used where a rank must not die while its memory is bound to an
# NVSwitch multicast object.
SOFT = os.environ.get("DION_TEST_SOFT_FAIL", "0") == "1"
FAILURES = []


def fail(msg):
    print(f"[rank {RANK}] FAIL: {msg}", flush=True)
    if SOFT:
        FAILURES.append(msg)
    else:
        raise SystemExit(1)


def check(name, a, b, tol):
    err = ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-12)).item()
    ok = err < tol
    if RANK == 0 or not ok:
        print(f"[rank {RANK}] {name}: scaled max err {err:.3e} (tol {tol}) {'ok' if ok else 'FAIL'}", flush=True)
    if not ok:
        fail(name)


def make_params(seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, generator=g).to(DEV)) for s in SHAPES]


def rank_grads(step, shapes=SHAPES):
    """Per-rank gradients (deterministic) and their mean over ranks."""
    out = []
    for r in range(WORLD):
        g = torch.Generator().manual_seed(1000 * step + r)
        out.append([torch.randn(s, generator=g) for s in shapes])
    mean = [sum(out[r][i] for r in range(WORLD)) / WORLD for i in range(len(shapes))]
    return [t.to(DEV) for t in out[RANK]], [t.to(DEV) for t in mean]


# ------------------------------------------------------------------------------------------ cases

def case_symm():
    """Symmetric-memory barrier / all-reduce / reduce-scatter / reduce-into kernels against torch sums,
    and the group-wide agreement on the arena's size.  Runs with plain peer loads and stores or, with
    DION_B200_MULTICAST=1, with the multimem instructions (see case_symm_multicast)."""
    if not CUDA:
        print("symm kernels need GPUs; skipped")
        return
    from dion_b200 import ops
    from dion_b200.parallel import symm

    group = dist.group.WORLD
    # no arena yet: the request is served from ordinary memory and remembered ...
    first = symm.empty(group, (1 << 20,), torch.float32, DEV)
    assert symm.arena_for(group) is None and first.numel() == 1 << 20
    symm.begin_step([group], DEV)   # ... and the next step boundary agrees on a size and creates the arena
    arena = symm.arena_for(group)
    assert arena is not None, "arena was not created"
    if RANK == 0:
        print(f"arena of {arena.capacity} bytes, multicast {'on' if arena.mc_base else 'off'}", flush=True)
    if os.environ.get("DION_B200_MULTICAST", "1") == "1" and os.environ.get("DION_TEST_NEED_MULTICAST") == "1":
        if not arena.mc_base:
            fail("the symmetric allocation has no multicast address on this machine")
    for dtype, n in ((torch.float32, 1 << 20), (torch.float32, 1003), (torch.bfloat16, 1 << 18), (torch.bfloat16, 777)):
        symm.begin_step([group], DEV)
        t = symm.empty(group, (n,), dtype, DEV)
        assert arena.offset_of(t) is not None
        gen = torch.Generator().manual_seed(5)
        full = [torch.randn(n, generator=gen) for _ in range(WORLD)]
        t.copy_(full[RANK].to(dtype))
        ref = (sum(f.to(dtype).float() for f in full) / WORLD).to(DEV)
        symm.all_reduce(t, group, average=True)
        check(f"symm all_reduce {dtype} n={n}", t, ref, 1e-5 if dtype == torch.float32 else 1e-2)
        # every rank must hold bit-identical results
        gathered = [torch.empty_like(t) for _ in range(WORLD)]
        dist.all_gather(gathered, t)
        if not all(torch.equal(gathered[0], g) for g in gathered):
            fail("all-reduce results differ between ranks")
        # one-shot reduce into a local buffer
        src = symm.empty(group, (n,), dtype, DEV)
        src.copy_(full[RANK].to(dtype))
        dst = torch.ones(n, device=DEV, dtype=torch.float32)
        arena.reduce_into(src, arena.offset_of(src), dst, scale=0.5, beta=2.0)
        check(f"symm reduce_into {dtype} n={n}", dst, (2.0 + 0.5 * sum(f.to(dtype).float() for f in full)).to(DEV), 1e-2)
    # reduce-scatter: rank r keeps slice r of the mean
    for dtype, per in ((torch.float32, 4096 + 8), (torch.bfloat16, 1 << 16)):
        symm.begin_step([group], DEV)
        n = per * WORLD
        t = symm.empty(group, (n,), dtype, DEV)
        gen = torch.Generator().manual_seed(11)
        full = [torch.randn(n, generator=gen) for _ in range(WORLD)]
        t.copy_(full[RANK].to(dtype))
        out = symm.reduce_scatter(t, group, average=True)
        ref = (sum(f.to(dtype).float() for f in full) / WORLD)[RANK * per:(RANK + 1) * per].to(DEV)
        check(f"symm reduce_scatter {dtype} n={n}", out, ref, 1e-5 if dtype == torch.float32 else 1e-2)
    # a step that needs more than the arena holds overflows to ordinary memory on every rank alike; the
    # ranks learn each other's needs through the arena and replace it at a later step boundary
    cap0 = arena.capacity
    big = cap0 // 4 + (1 << 20)  # fp32 elements: more bytes than the arena holds
    for step in range(3):
        symm.begin_step([group], DEV)
        t = symm.empty(group, (big,), torch.float32, DEV)
        t.fill_(float(RANK + 1))
        symm.all_reduce(t, group, average=False)   # library collective while it does not fit
        check(f"all_reduce around arena growth, step {step}", t[:1000], torch.full((1000,), WORLD * (WORLD + 1) / 2.0, device=DEV), 1e-6)
    arena2 = symm.arena_for(group)
    if arena2 is None or arena2.capacity <= cap0 or arena2.offset_of(t) is None:
        fail(f"arena did not grow: {cap0} -> {None if arena2 is None else arena2.capacity}")
    caps = [None] * WORLD
    dist.all_gather_object(caps, arena2.capacity if arena2 is not None else -1)
    if len(set(caps)) != 1:
        fail(f"ranks hold arenas of different sizes: {caps}")
    symm.arena_for(group).barrier()
    torch.cuda.synchronize()
    ops.check_status(DEV)


def case_symm_multicast():
    """case_symm with the kernels on multimem.ld_reduce / multimem.st (the default outside the tests)."""
    os.environ["DION_TEST_NEED_MULTICAST"] = "1"
    case_symm()


def _expect_pushed(*kinds):
    """On GPUs with symmetric memory on: the partial products of Dion's power iteration went through the
    GEMM-epilogue push into the consumers' slots (not through a collective kernel or the library)."""
    if not CUDA or os.environ.get("DION_B200_SYMM", "1") == "0" or os.environ.get("DION_B200_FUSED_REDUCE", "1") == "0":
        return
    from dion_b200.parallel import symm

    for kind in kinds:
        if symm.stats.get(f"{kind}.kernel", 0) <= 0:
            fail(f"{kind}: never took the pushed path ({dict(symm.stats)})")
    if RANK == 0:
        print(f"collective paths so far: {dict(sorted(symm.stats.items()))}", flush=True)


def _single_process_dion(rank_fraction, steps):
    from dion_b200 import Dion

    P = make_params()
    opt = Dion(P, lr=0.02, rank_fraction=rank_fraction, weight_decay=0.1)
    for s in range(steps):
        _, mean = rank_grads(s)
        for p, g in zip(P, mean):
            p.grad = g.clone()
        opt.step()
    return P, opt


def _check_sharded_orthonormalisation():
    """Batches split over the ranks (including one that does not divide evenly and one smaller than
    the group) give the same result as the redundant computation, identically on every rank."""
    from dion_b200.optim.orthogonalize import orthonormalize_many

    g = dist.group.WORLD
    gen = torch.Generator().manual_seed(3)
    Ps = [torch.randn(b, a, r, generator=gen).to(DEV) for b, a, r in ((2 * WORLD + 1, 96, 32), (1, 64, 32), (WORLD - 1 or 1, 128, 64))]
    whole = orthonormalize_many(Ps)
    split = orthonormalize_many(Ps, shard_groups=[g] * len(Ps))
    for i, (a, b) in enumerate(zip(split, whole)):
        check(f"sharded orthonormalisation batch {i}", a, b, 1e-5)
        ref = a.clone()
        dist.broadcast(ref, src=0)
        if Ps[i].shape[0] > 1:  # gathered: every rank received the same bytes
            assert torch.equal(a, ref), "ranks hold different orthonormal factors"
    # first-use check of an all-gather kernel: one that works is kept, one that returns something else
    # than the process group (here: on one rank only) is dropped by every rank, and the result is right
    from dion_b200.optim import orthogonalize as O

    def good(out, inp, group):
        dist.all_gather_into_tensor(out, inp, group=group)

    def bad(out, inp, group):
        dist.all_gather_into_tensor(out, inp, group=group)
        if RANK == WORLD - 1:
            out[:1] += 1.0

    part = torch.full((4, 3, 2), float(RANK), device=DEV)
    want = torch.cat([torch.full((4, 3, 2), float(r), device=DEV) for r in range(WORLD)])
    for fn, kept in ((good, True), (bad, False)):
        state = O._Gatherer(fn)
        for _ in range(2):
            out = torch.empty(4 * WORLD, 3, 2, device=DEV)
            O._exchange(out, part, g, state)
            assert torch.equal(out, want)
        assert state.checked and (state.fn is not None) == kept


def case_dion_ddp():
    _check_sharded_orthonormalisation()
    """Dion with a ProcessGroup replicate mesh, gradient sync owned by the optimizer:
    full-gradient path (rank_fraction 1) and compressed P/R path (rank_fraction 0.25)."""
    from dion_b200 import Dion

    for rf in (1.0, 0.25):
        P = make_params()
        opt = Dion(P, replicate_mesh=dist.group.WORLD, replicate_mesh_grad_sync=True, lr=0.02, rank_fraction=rf,
                   weight_decay=0.1)
        steps = 3
        for s in range(steps):
            mine, _ = rank_grads(s)
            for p, g in zip(P, mine):
                p.grad = g.clone()
            opt.step()
        Pref, optref = _single_process_dion(rf, steps)
        tol = 2e-3 if CUDA else 1e-4
        for i, (p, q) in enumerate(zip(P, Pref)):
            check(f"dion ddp rf={rf} X[{i}]", p, q, tol)
        # momentum is decoupled per rank when compressed; its mean follows the single-process run
        opt.synchronize_for_checkpoint()
        for i, (p, q) in enumerate(zip(P, Pref)):
            check(f"dion ddp rf={rf} M[{i}] after synchronize_for_checkpoint", opt.state[p]["momentum"],
                  optref.state[q]["momentum"], 5e-3 if CUDA else 1e-4)
    _expect_pushed("dion_p_exchange", "dion_r_exchange")  # the compressed run synchronises P and R over the replicas


def case_muon_ddp():
    """Muon with a ProcessGroup: matrices are split over ranks and all-gathered."""
    from dion_b200 import Muon

    P = make_params()
    Pref = make_params()
    opt = Muon(P, distributed_mesh=dist.group.WORLD, lr=0.02, nesterov=True)
    optref = Muon(Pref, lr=0.02, nesterov=True)
    for s in range(3):
        _, mean = rank_grads(s)
        for p, q, g in zip(P, Pref, mean):
            p.grad = g.clone()
            q.grad = g.clone()
        opt.step()
        optref.step()
    for i, (p, q) in enumerate(zip(P, Pref)):
        check(f"muon ddp X[{i}]", p, q, 2e-2)


def _tiny_gpt():
    from dion_b200.models import GPT, GPTConfig

    torch.manual_seed(0)
    m = GPT(GPTConfig(sequence_len=64, vocab_size=512, n_layer=2, n_head=4, n_embd=64))
    m.init_weights()
    return m


def _full(t):
    from torch.distributed.tensor import DTensor

    return t.full_tensor() if isinstance(t, DTensor) else t


def _train(model, opt, steps, data_rank=None, data_world=None):
    losses = []
    for s in range(steps):
        g = torch.Generator().manual_seed(77 + s)
        idx = torch.randint(0, 512, (4 * WORLD, 64), generator=g)
        tgt = torch.randint(0, 512, (4 * WORLD, 64), generator=g)
        if data_rank is not None:
            idx, tgt = idx[data_rank::data_world], tgt[data_rank::data_world]
        loss = model(idx.to(DEV), tgt.to(DEV))
        loss.backward()
        opt.step()
        model.zero_grad(set_to_none=True)
        losses.append(loss.detach().float())
    return torch.stack(losses)


def case_fsdp():
    """GPT under FSDP2 (fs = world) with Dion (outer mesh) and with Muon, against a
    single-process run on the full batch."""
    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion, Muon
    from dion_b200.models.gpt import parallelize_gpt_model

    for name in ("dion", "muon"):
        mesh = init_device_mesh("cuda" if CUDA else "cpu", (1, WORLD, 1), mesh_dim_names=("dp", "fs", "tp"))
        ref = _tiny_gpt().to(DEV)
        model = _tiny_gpt().to(DEV)
        parallelize_gpt_model(model, mesh, dp_name=None, fs_name="fs", tp_name="tp")
        mk = lambda m: [dict(params=list(m.transformer.h.parameters())),
                        dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()),
                             algorithm="adamw", lr=0.002)]
        if name == "dion":
            opt = Dion(mk(model), replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"], lr=0.02, rank_fraction=0.5)
            optref = Dion(mk(ref), lr=0.02, rank_fraction=0.5)
            # same Q on both sides
            for g in opt.param_groups[:1]:
                for p in g["params"]:
                    opt._get_or_initialize_state(p, g)
            for (n1, p1), (n2, p2) in zip(model.transformer.h.named_parameters(), ref.transformer.h.named_parameters()):
                optref.state[p2] = {"momentum": torch.zeros_like(p2), "Q": _full(opt.state[p1]["Q"]).clone()}
                # the sharding decides the orientation of the power iteration; mirror it
                optref._get_dion_param_config(p2).is_transposed = opt._param_config[p1].is_transposed
        else:
            opt = Muon(mk(model), distributed_mesh=mesh["fs"], lr=0.02, nesterov=True)
            optref = Muon(mk(ref), lr=0.02, nesterov=True)
        l1 = _train(model, opt, 3, data_rank=RANK, data_world=WORLD)
        l2 = _train(ref, optref, 3)
        dist.all_reduce(l1, op=dist.ReduceOp.SUM)
        l1 /= WORLD
        check(f"fsdp {name} losses", l1, l2, 3e-2 if CUDA else 2e-3)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), ref.named_parameters()):
            # embedding / lm_head use a sign-like update in the first steps, where tiny
            # gradient differences flip whole entries by 2 * lr
            loose = "wte" in n1 or "lm_head" in n1
            check(f"fsdp {name} {n1}", _full(p1.detach()), p2.detach(), 6e-2 if (CUDA or loose) else 5e-3)
        if name == "dion":
            # every class of the 2-layer model has an even number of matrices: P leaves its reduction
            # over the shard group as this rank's share (reduce-scatter), not as the whole batch
            if WORLD == 2:  # with more ranks the classes of this small model (2, 2 and 8 matrices) do not all split evenly
                assert opt.p_reduce_scatters > 0, "P was all-reduced although the batches split evenly"
            _expect_pushed("dion_p_exchange")
        if name == "muon":
            # the momentum is linear in the gradients, so it pins down that every path (library
            # all-to-all or peer stores from the momentum kernel) applies it exactly once per step
            for (n1, p1), (n2, p2) in zip(model.transformer.h.named_parameters(), ref.transformer.h.named_parameters()):
                # (a second application per step would be off by about 0.9 of the scale)
                check(f"fsdp muon momentum {n1}", _full(opt.state[p1]["momentum"]), optref.state[p2]["momentum"],
                      0.3 if CUDA else 5e-2)
    if CUDA and os.environ.get("DION_B200_SYMM", "1") != "0":
        from dion_b200.parallel import fsdp_comm

        calls = [(a.kernel_calls, r.kernel_calls) for a, r in fsdp_comm._installed.values()]
        assert calls and all(a > 0 and r > 0 for a, r in calls), f"FSDP ran on library collectives: {calls}"


def case_fsdp_comm():
    """All-gather / reduce-scatter kernels behind the FSDP2 hooks against the library collectives:
    several sizes (the arenas regrow), fp32 and bf16, SUM and AVG, slot reuse back to back."""
    from dion_b200.parallel.fsdp_comm import SymmAllGather, SymmReduceScatter

    g = dist.group.WORLD
    ag, rs = SymmAllGather(g, DEV), SymmReduceScatter(g, DEV)
    gen = torch.Generator().manual_seed(7 + RANK)
    for it, (n, dtype) in enumerate([(4096, torch.bfloat16), (1 << 20, torch.bfloat16), (40, torch.float32),
                                     (3 << 19, torch.float32), (1 << 20, torch.bfloat16), (8, torch.bfloat16)]):
        # all-gather, the way FSDP calls it: the input is a view of the output
        out = ag.allocate((n * WORLD,), dtype=dtype, device=DEV)
        inp = out.narrow(0, RANK * n, n)
        inp.copy_(torch.randn(n, generator=gen).to(DEV))
        want = torch.empty_like(out)
        dist.all_gather_into_tensor(want, inp.clone(), group=g)
        ag(out, inp, g)
        assert torch.equal(out, want), f"all-gather mismatch (n={n}, {dtype})"
        # separate input buffer
        inp2 = torch.randn(n, generator=gen).to(DEV).to(dtype)
        out2 = torch.empty(n * WORLD, dtype=dtype, device=DEV)
        dist.all_gather_into_tensor(want, inp2, group=g)
        ag(out2, inp2, g)
        assert torch.equal(out2, want)
        # reduce-scatter, input from allocate() then output from allocate()
        for op in (dist.ReduceOp.AVG, dist.ReduceOp.SUM):
            rin = rs.allocate((n * WORLD,), dtype=dtype, device=DEV)
            rin.copy_(torch.randn(n * WORLD, generator=gen).to(DEV))
            rout = rs.allocate((n,), dtype=dtype, device=DEV)
            want_r = torch.empty(n, dtype=dtype, device=DEV)
            if CUDA:
                dist.reduce_scatter_tensor(want_r, rin.clone(), op=op, group=g)
            else:
                full = rin.clone().float()
                dist.all_reduce(full, group=g)
                want_r = (full / (WORLD if op == dist.ReduceOp.AVG else 1))[RANK * n:(RANK + 1) * n].to(dtype)
            if CUDA:
                rs(rout, rin, g, op)
            else:
                # gloo has no reduce-scatter; the object is only exercised for its bookkeeping here
                rout.copy_(want_r)
            check(f"reduce-scatter n={n} {dtype} {op}", rout, want_r, 2e-2 if dtype == torch.bfloat16 else 1e-5)
    if CUDA:
        from dion_b200 import ops

        ops.check_status()
        assert ag.kernel_calls > 0 and rs.kernel_calls > 0, (ag.kernel_calls, ag.fallback_calls, rs.kernel_calls,
                                                              rs.fallback_calls)
        if RANK == 0:
            print(f"fsdp_comm: all-gather kernel/fallback {ag.kernel_calls}/{ag.fallback_calls}, "
                  f"reduce-scatter {rs.kernel_calls}/{rs.fallback_calls}", flush=True)


def case_hybrid():
    """Meshes with two active dimensions (needs a multiple of four ranks).
    (a) dp2 x fs: FSDP2 over `fs`, Dion keeps the replicas in step by exchanging only the low-rank
        P / R factors over `dp` (compressed sync, rank_fraction 0.25, fp32 Q / bf16 momentum); every
        replica sees different data, yet the parameters must stay identical across `dp`.
    (b) fs2 x tp: FSDP2 + tensor parallelism, against a single-process run on the full batch."""
    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion, DionMixedPrecisionConfig
    from dion_b200.models.gpt import parallelize_gpt_model

    if WORLD % 4 != 0:
        print("hybrid meshes need 4 ranks; skipped")
        return
    kind = "cuda" if CUDA else "cpu"
    mk = lambda m: [dict(params=list(m.transformer.h.parameters())),
                    dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()),
                         algorithm="adamw", lr=0.002)]
    def stage(msg):
        if os.environ.get("DION_TEST_VERBOSE"):
            print(f"[rank {RANK}] hybrid: {msg}", file=sys.stderr, flush=True)

    # ---- (a)
    stage("dp x fs: building")
    mesh = init_device_mesh(kind, (2, WORLD // 2, 1), mesh_dim_names=("dp", "fs", "tp"))
    model = _tiny_gpt().to(DEV)
    parallelize_gpt_model(model, mesh, dp_name=None, fs_name="fs", tp_name="tp")
    opt = Dion(mk(model), replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"], replicate_mesh_grad_sync=True,
               lr=0.02, rank_fraction=0.25,
               mixed_precision_config=DionMixedPrecisionConfig(momentum_dtype=torch.bfloat16, Q_dtype=torch.float32))
    stage("dp x fs: training")
    losses = _train(model, opt, 4, data_rank=RANK, data_world=WORLD)
    stage("dp x fs: trained")
    assert torch.isfinite(losses).all(), losses
    opt.synchronize_for_checkpoint()
    stage("dp x fs: synchronised")
    dp_group = mesh["dp"].get_group()
    for n, p_ in model.named_parameters():
        loc = p_.detach().to_local() if hasattr(p_, "to_local") else p_.detach()
        ref = loc.clone()
        dist.broadcast(ref, src=dist.get_global_rank(dp_group, 0), group=dp_group)
        check(f"hybrid dp x fs replica consistency {n}", loc, ref, 1e-6)
    st = next(iter(opt.state.values()))
    assert st["momentum"].dtype == torch.bfloat16 and st["Q"].dtype == torch.float32
    _expect_pushed("dion_p_exchange", "dion_r_exchange")
    # ---- (b)
    stage("fs x tp: building")
    mesh = init_device_mesh(kind, (1, 2, WORLD // 2), mesh_dim_names=("dp", "fs", "tp"))
    ref = _tiny_gpt().to(DEV)
    model = _tiny_gpt().to(DEV)
    parallelize_gpt_model(model, mesh, dp_name=None, fs_name="fs", tp_name="tp")
    tp = WORLD // 2
    opt = Dion(mk(model), replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"], inner_shard_mesh=mesh["tp"],
               lr=0.02, rank_fraction=0.5, rank_multiple_of=tp)
    optref = Dion(mk(ref), lr=0.02, rank_fraction=0.5, rank_multiple_of=tp)
    for g in opt.param_groups[:1]:
        for p_ in g["params"]:
            opt._get_or_initialize_state(p_, g)
    for (n1, p1), (n2, p2) in zip(model.transformer.h.named_parameters(), ref.transformer.h.named_parameters()):
        optref.state[p2] = {"momentum": torch.zeros_like(p2), "Q": _full(opt.state[p1]["Q"]).clone()}
        optref._get_dion_param_config(p2).is_transposed = opt._param_config[p1].is_transposed
    # sharding classification (dion/dion.py:498-607): column-parallel weights are Shard(0) over tp and
    # Shard(1) over fs -> orthogonalise over the tp-sharded dim, not transposed; row-parallel weights
    # the other way round -> transposed; Q is Shard(0) on the outer and Shard(1) on the inner mesh dim
    from torch.distributed.tensor import Shard

    blk = model.transformer.h[0]
    for w, inner_dim, outer_dim, transposed in ((blk.attn.c_q.weight, 0, 1, False), (blk.mlp.c_fc.weight, 0, 1, False),
                                                (blk.attn.c_proj.weight, 1, 0, True), (blk.mlp.c_proj.weight, 1, 0, True)):
        c = opt._param_config[w]
        assert (c.inner_shard_tensor_dim, c.outer_shard_tensor_dim, c.is_transposed) == (inner_dim, outer_dim, transposed), c
        q = opt.state[w]["Q"]
        names = q.device_mesh.mesh_dim_names
        assert q.placements[names.index("fs")] == Shard(0) and q.placements[names.index("tp")] == Shard(1), q.placements
        m, n = w.shape
        assert q.shape[0] == (m if transposed else n)
    fs_rank = mesh["fs"].get_local_rank()
    stage("fs x tp: training")
    l1 = _train(model, opt, 3, data_rank=fs_rank, data_world=2)
    stage("fs x tp: trained")
    l2 = _train(ref, optref, 3)
    dist.all_reduce(l1, op=dist.ReduceOp.SUM)
    l1 /= WORLD
    _expect_pushed("dion_p_exchange", "dion_r_exchange")
    check("hybrid fs x tp losses", l1, l2, 3e-2 if CUDA else 2e-3)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), ref.named_parameters()):
        loose = "wte" in n1 or "lm_head" in n1
        check(f"hybrid fs x tp {n1}", _full(p1.detach()), p2.detach(), 6e-2 if (CUDA or loose) else 5e-3)


def case_gemm_gather():
    """GPUs only: the GEMM that all-gathers the row blocks of its first operand inside the kernel,
    against the all-gather collective followed by an fp32 product."""
    if not CUDA:
        return
    from dion_b200 import ops
    from dion_b200.parallel import tp as TP

    g = dist.group.WORLD
    TP._FUSED_GATHER = True
    try:
        for rep, (R, Kd, N) in enumerate([(256, 64, 96), (1024, 768, 1536), (4096, 768, 2304), (2048, 1024, 4096), (1024, 768, 1536)]):
            # 128 x 128 tiles, 128 x 256 tiles, CTA pairs with 256 x 256 tiles (K >= 1024), and a repeat
            gen = torch.Generator(device="cpu").manual_seed(100 * rep + RANK)
            x = torch.randn(R, Kd, generator=gen).to(DEV).to(torch.bfloat16)
            w = torch.randn(N, Kd, generator=torch.Generator().manual_seed(7 + rep)).mul_(0.05).to(DEV).to(torch.bfloat16)
            xg, y = TP._gather_matmul(x, w.t(), g)
            ref_xg = torch.empty(WORLD * R, Kd, dtype=torch.bfloat16, device=DEV)
            dist.all_gather_into_tensor(ref_xg, x, group=g)
            ops.check_status()
            assert torch.equal(xg, ref_xg), f"gathered operand differs ({R}x{Kd})"
            check(f"gemm_gather {R}x{Kd}x{N}", y, ref_xg.float() @ w.float().t(), 2e-2)
            # the unfused all-gather shares the staging slots and epochs with the fused kernel
            check("gather_rows after gemm_gather", TP._gather_rows(x, g), ref_xg, 1e-6)
        calls = [c.fused_gathers for c in TP._tp_comms.values()]
        assert calls and all(c >= 5 for c in calls), f"the all-gather did not run inside the GEMM: {calls}"
    finally:
        TP._FUSED_GATHER = False


def _check_vocab_parallel_ce(group):
    """Chunked vocabulary-parallel lm_head + cross-entropy (several chunks, a ragged last one, ignored
    targets) against F.cross_entropy on the full logits: loss, dX and dW."""
    import torch.nn.functional as F

    from dion_b200.parallel import tp as TP

    T, Kd, V = (192 if CUDA else 104), 64, 64 * WORLD
    gen = torch.Generator().manual_seed(11)
    dt = torch.bfloat16 if CUDA else torch.float32
    x = torch.randn(T, Kd, generator=gen).to(DEV).to(dt).requires_grad_()
    w = (torch.randn(V, Kd, generator=gen) * 0.3).to(DEV).requires_grad_()
    tgt = torch.randint(0, V, (T,), generator=gen).to(DEV)
    tgt[::7] = -1
    v_loc = V // WORLD
    w_loc = w.detach()[RANK * v_loc:(RANK + 1) * v_loc].clone().requires_grad_()
    x1 = x.detach().clone().requires_grad_()
    loss = TP.vocab_parallel_cross_entropy(x1, w_loc, tgt, group, ignore_index=-1, chunk_tokens=64 if CUDA else 32)
    (loss * 2.0).backward()
    ref = F.cross_entropy(x.float() @ w.t().float(), tgt, ignore_index=-1)
    (ref * 2.0).backward()
    tol = 3e-2 if CUDA else 1e-5
    check("vocab-parallel CE loss", loss.detach().reshape(1), ref.detach().reshape(1), tol)
    check("vocab-parallel CE dX", x1.grad, x.grad, tol)
    check("vocab-parallel CE dW", w_loc.grad, w.grad[RANK * v_loc:(RANK + 1) * v_loc], tol)


def case_tp_sp():
    """Tensor parallelism with the residual stream sharded over the tokens (all-gather -> GEMM,
    GEMM -> reduce-scatter) against a single-process run, plus the logits / generation path."""
    case_tp(sequence_parallel=True)


def case_tp(sequence_parallel=False):
    """GPT with tensor parallelism (tp = world): loss and a Dion step (inner mesh) against a
    single-process run."""
    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion
    from dion_b200.models.gpt import parallelize_gpt_model

    mesh = init_device_mesh("cuda" if CUDA else "cpu", (1, 1, WORLD), mesh_dim_names=("dp", "fs", "tp"))
    if not sequence_parallel:
        _check_vocab_parallel_ce(mesh.get_group("tp"))
    ref = _tiny_gpt().to(DEV)
    model = _tiny_gpt().to(DEV)
    parallelize_gpt_model(model, mesh, dp_name=None, fs_name="fs", tp_name="tp", sequence_parallel=sequence_parallel)
    assert model.sequence_parallel == sequence_parallel
    if sequence_parallel:
        torch.manual_seed(5)
        idx = torch.randint(0, 512, (2, 64), device=DEV)
        tgt = torch.randint(0, 512, (2, 64), device=DEV)
        tol = 6e-2 if CUDA else 3e-2     # FSDP's mixed precision runs the forward on bf16 copies of the weights
        with torch.no_grad():
            check("tp_sp logits", model(idx, tgt, return_logits=True), ref(idx, tgt, return_logits=True), tol)
            check("tp_sp last-token logits", model(idx, None, return_logits=True), ref(idx, None, return_logits=True), tol)
            assert model(idx) is None
            odd = idx[:, :63]            # 126 tokens do not split into blocks of 8 rows: replicated path
            check("tp_sp ragged", model(odd, None, return_logits=True), ref(odd, None, return_logits=True), tol)
    mk = lambda m: [dict(params=list(m.transformer.h.parameters())),
                    dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()),
                         algorithm="adamw", lr=0.002)]
    opt = Dion(mk(model), replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"], inner_shard_mesh=mesh["tp"],
               lr=0.02, rank_fraction=0.5, rank_multiple_of=WORLD)
    optref = Dion(mk(ref), lr=0.02, rank_fraction=0.5, rank_multiple_of=WORLD)
    for g in opt.param_groups[:1]:
        for p in g["params"]:
            opt._get_or_initialize_state(p, g)
    for (n1, p1), (n2, p2) in zip(model.transformer.h.named_parameters(), ref.transformer.h.named_parameters()):
        optref.state[p2] = {"momentum": torch.zeros_like(p2), "Q": _full(opt.state[p1]["Q"]).clone()}
        optref._get_dion_param_config(p2).is_transposed = opt._param_config[p1].is_transposed
    l1 = _train(model, opt, 3)           # tensor-parallel ranks see the same data
    l2 = _train(ref, optref, 3)
    check("tp losses", l1, l2, 3e-2 if CUDA else 2e-3)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), ref.named_parameters()):
        loose = "wte" in n1 or "lm_head" in n1
        check(f"tp {n1}", _full(p1.detach()), p2.detach(), 6e-2 if (CUDA or loose) else 5e-3)
    if CUDA and os.environ.get("DION_B200_SYMM", "1") != "0":
        from dion_b200.parallel import tp as TP

        calls = [c.calls for c in TP._tp_comms.values()]
        assert calls and all(c > 0 for c in calls), f"row-parallel products ran on library collectives: {calls}"
        if RANK == 0:
            print(f"tp: fused GEMM -> reduce-scatter / all-gather products: {calls}", flush=True)


def case_structured():
    """Periodic token data (low-rank gradients, ill-conditioned P from the first step): Dion under tensor
    parallelism (row-sharded Gram matrices) and under FSDP2 (P reduce-scattered, work split over the ranks)
    follows the single-process oracle that orthonormalises with Householder QR."""
    from torch.distributed.device_mesh import init_device_mesh

    from dion_b200 import Dion, DionReference
    from dion_b200.models.gpt import parallelize_gpt_model

    def groups(m):
        return [dict(params=list(m.transformer.h.parameters())),
                dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()), algorithm="lion",
                     lr=0.002)]

    def batch(step, rank, world):
        base = (torch.arange(65) * 7) % 23
        x = torch.stack([(base + i + step) % 23 for i in range(8)])
        per = 8 // world
        x = x[rank * per:(rank + 1) * per].to(DEV)
        return x[:, :-1].contiguous(), x[:, 1:].contiguous()

    def train(m, opt, steps, rank, world):
        out = []
        for s in range(steps):
            x, y = batch(s, rank, world)
            loss = m(x, y)
            loss.backward()
            opt.step()
            m.zero_grad(set_to_none=True)
            out.append(loss.detach().float().clone())
        return torch.stack(out)

    steps = 21
    ref = _tiny_gpt().to(DEV)
    want = train(ref, DionReference(groups(ref), lr=0.02, rank_fraction=1.0, qr_method="qr"), steps, 0, 1)
    kind = "cuda" if CUDA else "cpu"
    for mode in ("tp", "fsdp"):
        shape = (1, 1, WORLD) if mode == "tp" else (1, WORLD, 1)
        mesh = init_device_mesh(kind, shape, mesh_dim_names=("dp", "fs", "tp"))
        model = _tiny_gpt().to(DEV)
        parallelize_gpt_model(model, mesh, dp_name=None, fs_name="fs", tp_name="tp")
        opt = Dion(groups(model), replicate_mesh=mesh["dp"], outer_shard_mesh=mesh["fs"],
                   inner_shard_mesh=mesh["tp"] if mode == "tp" else None, lr=0.02, rank_fraction=1.0,
                   rank_multiple_of=WORLD)
        got = train(model, opt, steps, *((0, 1) if mode == "tp" else (RANK, WORLD)))
        dist.all_reduce(got)
        got /= WORLD
        assert opt.robust_switches >= 1, "the ill-conditioned treatment never came on"
        assert got[-1] < 0.5 * got[0]
        check(f"structured {mode} losses", got[4:], want[4:], 0.1 if CUDA else 2e-2)


def case_functional():
    """The free functions that mirror the reference's helpers, on sharded inputs: orthonormalisation of
    row-sharded matrices (batched Cholesky-QR and the oracle's per-matrix methods), averaged all-reduce, scalar
    updates behind a gradient all-reduce, and the DTensor sketch."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Replicate, Shard

    from dion_b200 import dion as D
    from dion_b200 import dion_reference as DR

    mesh = init_device_mesh("cuda" if CUDA else "cpu", (WORLD,), mesh_dim_names=("shard",))
    g = torch.Generator().manual_seed(7)
    full = torch.randn(3, 16 * WORLD, 8, generator=g).to(DEV)
    rows = full.shape[1] // WORLD
    local = full[:, RANK * rows:(RANK + 1) * rows].contiguous()
    P = DTensor.from_local(local, device_mesh=mesh, placements=[Shard(1)], run_check=False)

    # batched Cholesky-QR on row shards against the single-process result on the whole matrices
    out = D.distributed_orthogonalize(P, shard_mesh_dim=0)
    assert isinstance(out, DTensor) and tuple(out.placements) == (Shard(1),)
    want = D.orthogonalize(full)
    check("distributed_orthogonalize (cholesky-qr)", out.to_local(), want[:, RANK * rows:(RANK + 1) * rows], 2e-3 if CUDA else 1e-4)
    rep = D.distributed_orthogonalize(DTensor.from_local(full, device_mesh=mesh, placements=[Replicate()], run_check=False))
    check("distributed_orthogonalize (replicated)", rep.to_local(), want, 2e-3 if CUDA else 1e-5)

    # the oracle's per-matrix methods on one row-sharded matrix: orthonormal columns spanning the same space
    P2 = DTensor.from_local(local[0].contiguous(), device_mesh=mesh, placements=[Shard(0)], run_check=False)
    for method in ("qr", "cqr", "rcqr"):
        q = DR.distributed_orthogonalize(P2, qr_method=method, shard_mesh_dim=0)
        parts = [torch.empty_like(q.to_local()) for _ in range(WORLD)]
        dist.all_gather(parts, q.to_local().contiguous())
        Q = torch.cat(parts, dim=0).float()
        check(f"oracle {method}: Q^T Q = I", Q.T @ Q, torch.eye(8, device=DEV), 1e-3)
        proj = Q @ (Q.T @ full[0])
        check(f"oracle {method}: span", proj, full[0], 1e-3)

    # averaged all-reduce of a list, in place and returned
    grads, mean = rank_grads(3, shapes=[(5, 4), (9,)])
    got = D.all_reduce_replicate_mesh([t.clone() for t in grads], mesh, return_dtensor=False)
    for a, b in zip(got, mean):
        check("all_reduce_replicate_mesh", a, b, 1e-5)
    assert D.all_reduce_replicate_mesh(grads[0], None) is grads[0]

    # Lion / AdamW behind the gradient all-reduce equal the same update with the mean gradient
    for algo in ("lion", "adamw"):
        X = [torch.ones(5, 4, device=DEV), torch.ones(9, device=DEV)]
        Xw = [x.clone() for x in X]
        M, Mw = [torch.zeros_like(x) for x in X], [torch.zeros_like(x) for x in X]
        V, Vw = [torch.zeros_like(x) for x in X], [torch.zeros_like(x) for x in X]
        G = [t.clone() for t in grads]
        if algo == "lion":
            task = D.lion_update_allreduce_grad(X, G, M, 0.01, 0.9, 0.99, 0.1, replicate_mesh=mesh)
            from dion_b200.scalar_opts import lion_update_foreach

            lion_update_foreach(Xw, mean, Mw, 0.01, 0.9, 0.99, 0.1)
        else:
            task = D.adamw_update_allreduce_grad(X, G, M, V, 0.01, 0.9, 0.99, 0.1, 1, 1e-8, replicate_mesh=mesh)
            from dion_b200.scalar_opts import adamw_update_foreach

            adamw_update_foreach(Xw, mean, Mw, Vw, 0.01, 0.9, 0.99, 0.1, 1, 1e-8)
        steps = sum(1 for _ in task)
        assert steps == 1, "one yield while the all-reduce is in flight"
        for a, b in zip(X, Xw):
            check(f"{algo}_update_allreduce_grad", a, b, 1e-5)

    # DTensor sketch, sharded along m over the mesh dimension (DTensor random numbers need a CUDA mesh)
    if CUDA:
        S = D.generate_random_sketch_matrix(P, 1.25, shard_mesh_dim=0)
        assert tuple(S.shape) == (3, 128, 16 * WORLD) and tuple(S.to_local().shape) == (3, 128, rows)
        assert tuple(S.placements) == (Shard(2),)


def case_checkpoint():
    """Distributed checkpoint round trip of model + Dion state through CheckpointManager."""
    import tempfile

    from dion_b200 import Dion
    from dion_b200.models.data import DistributedDataLoader, write_synthetic_shards
    from dion_b200.training import CheckpointManager

    box = [None]
    if RANK == 0:
        box[0] = tempfile.mkdtemp(prefix="dion_ckpt_")
        write_synthetic_shards(box[0], 512, train_tokens=200_000, val_tokens=50_000)
    dist.broadcast_object_list(box, src=0)
    root = box[0]

    def build():
        m = _tiny_gpt().to(DEV)
        o = Dion([dict(params=list(m.transformer.h.parameters())),
                  dict(params=list(m.transformer.wte.parameters()) + list(m.lm_head.parameters()),
                       algorithm="adamw", lr=0.002)], replicate_mesh=dist.group.WORLD, lr=0.02, rank_fraction=0.25)
        tl = DistributedDataLoader(os.path.join(root, "fineweb_train_*.bin"), 2, 64, RANK, WORLD, device=DEV)
        vl = DistributedDataLoader(os.path.join(root, "fineweb_val_*.bin"), 2, 64, RANK, WORLD, device=DEV)
        return m, o, tl, vl

    def steps(m, o, tl, n):
        out = []
        for _ in range(n):
            x, y = tl.next_batch()
            loss = m(x, y)
            loss.backward()
            o.step()
            m.zero_grad(set_to_none=True)
            out.append(loss.detach().float())
        return torch.stack(out)

    m, o, tl, vl = build()
    steps(m, o, tl, 2)
    o.synchronize_for_checkpoint()
    mgr = CheckpointManager(os.path.join(root, "ckpt"), m, o, tl, vl)
    mgr.save(step=2)
    after = steps(m, o, tl, 2)

    m2, o2, tl2, vl2 = build()
    mgr2 = CheckpointManager(os.path.join(root, "ckpt"), m2, o2, tl2, vl2)
    mgr2.load()
    assert mgr2.step == 2
    resumed = steps(m2, o2, tl2, 2)
    check("losses after resume", resumed, after, 2e-2 if CUDA else 1e-4)
    keys = set(o2.state_dict()["param_groups"][0].keys())
    assert {"algorithm", "beta1", "beta2", "epsilon", "lr", "mu", "oversample", "params", "rank_fraction",
            "rank_multiple_of", "step", "weight_decay"} <= keys, keys


CASES = {k[5:]: v for k, v in list(globals().items()) if k.startswith("case_")}

if __name__ == "__main__":
    init()
    try:
        for name in sys.argv[1:]:
            if RANK == 0:
                print(f"=== case {name}", flush=True)
            if SOFT:
                try:
                    CASES[name]()
                except BaseException as e:  # recorded; this rank still takes part in the verdict and the teardown
                    import traceback

                    traceback.print_exc()
                    FAILURES.append(f"{name}: {type(e).__name__}: {e}")
            else:
                CASES[name]()
            dist.barrier()
        if CUDA:
            from dion_b200 import ops

            if SOFT:
                try:
                    ops.check_status(DEV)
                except Exception as e:
                    FAILURES.append(f"status word: {e}")
            else:
                ops.check_status(DEV)
        if SOFT:
            verdict = torch.tensor([0 if FAILURES else 1], dtype=torch.int32, device=DEV)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
            if CUDA:
                torch.cuda.synchronize()
            dist.barrier()
            if int(verdict.item()) == 0:
                FAILURES.append("some rank failed")
    finally:
        dist.destroy_process_group()
    if FAILURES:
        print(f"[rank {RANK}] failures: {FAILURES}", flush=True)
        sys.exit(1)
    if RANK == 0:
        print("ALL OK", flush=True)
