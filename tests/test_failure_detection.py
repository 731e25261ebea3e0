"""Failure detection without faulting anything: bounded device-side waits that report through the
status word, a rank that leaves between steps, and the atomicity of checkpoint writes."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_peer_wait_runs_out_and_reports_through_the_status_word():
    """A barrier whose second participant never signals: the kernel gives up after its time budget,
    records `peer timeout`, the host raises, and the context stays usable."""
    from dion_b200 import ops
    from dion_b200.ops import _ext, runtime

    _ext.load(required=True)
    dev = torch.device("cuda", 0)
    buf = torch.zeros(8192, dtype=torch.uint8, device=dev)       # a private flag block, nothing else writes it
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    base = buf.data_ptr()
    ops.check_status(dev)
    # world of two, both "peers" are this buffer; rank 0 signals its own flag, the flag of rank 1 stays 0
    torch.ops.dion_b200.symm_barrier(counter, [base, base], 0, 0, 0, 1, runtime.status_tensor(dev))
    with pytest.raises(ops.DionKernelError, match="peer"):
        ops.check_status(dev)
    ops.check_status(dev)                                          # the word was cleared
    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    b = torch.randn(128, 256, device=dev).to(torch.bfloat16)
    out = ops.gemm(a, b, out_dtype=torch.float32)
    torch.testing.assert_close(out, a.float() @ b.float(), rtol=1e-3, atol=1e-3)


def test_rank_leaving_between_steps_is_detected_not_waited_for():
    """Two gloo ranks; rank 1 stops after the first step.  Rank 0's next collective must fail within
    the process-group timeout (an exception on the host), not hang."""
    code = r'''
import os, sys, datetime, torch, torch.distributed as dist
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
rank = dist.get_rank()
t = torch.ones(4)
dist.all_reduce(t)                      # step 1: everybody is there
assert t[0].item() == 2
if rank == 1:
    dist.destroy_process_group()        # leaves between steps, nothing in flight
    sys.exit(0)
try:
    dist.all_reduce(t)                  # step 2: the peer is gone
    print("NOT DETECTED", flush=True)
except Exception as e:                  # connection closed / timed out
    print("DETECTED", type(e).__name__, flush=True)
'''
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), "-c", code]
    # torchrun has no -c; run the snippet from a temporary file instead
    import tempfile

    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(code)
        path = f.name
    try:
        cmd = cmd[:-2] + [path]
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=120)
    finally:
        os.unlink(path)
    assert "DETECTED" in res.stdout and "NOT DETECTED" not in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_checkpoint_write_is_atomic(tmp_path, monkeypatch):
    """A save that dies half way leaves neither a partial checkpoint nor a damaged previous one."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp

    from dion_b200 import training

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29990 - os.getpid() % 50))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        model = torch.nn.Linear(8, 8, bias=False)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)

        class Loader:
            def state_dict(self):
                return {"pos": 3}

            def load_state_dict(self, sd):
                self.loaded = sd

        mgr = training.CheckpointManager(str(tmp_path), model, opt, Loader(), Loader())
        mgr.save(step=1)
        good = sorted(os.listdir(tmp_path))
        assert len(good) == 1
        before = model.weight.detach().clone()

        real_save = dcp.save

        def dying_save(state, checkpoint_id=None, **kw):
            os.makedirs(checkpoint_id, exist_ok=True)
            with open(os.path.join(checkpoint_id, "partial.distcp"), "w") as f:
                f.write("half a shard")
            raise RuntimeError("injected: writer died")

        monkeypatch.setattr(dcp, "save", dying_save)
        with torch.no_grad():
            model.weight.add_(1.0)
        with pytest.raises(RuntimeError, match="injected"):
            mgr.save(step=2)
        monkeypatch.setattr(dcp, "save", real_save)
        names = sorted(os.listdir(tmp_path))
        finished = [n for n in names if not n.startswith("tmp")]
        assert finished == good, names                      # no entry for step 2, step 1 untouched
        with torch.no_grad():
            model.weight.zero_()
        mgr.load()
        torch.testing.assert_close(model.weight.detach(), before)
    finally:
        dist.destroy_process_group()


def test_checkpoint_swap_interrupted_between_renames_falls_back_to_previous(tmp_path, monkeypatch):
    """The writer dies after the previous checkpoint was set aside and before the new one took its
    name: load() finds the set-aside copy."""
    import shutil

    import torch.distributed as dist

    from dion_b200 import training

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29930 - os.getpid() % 50))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        model = torch.nn.Linear(8, 8, bias=False)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)

        class Loader:
            def state_dict(self):
                return {"pos": 3}

            def load_state_dict(self, sd):
                self.loaded = sd

        mgr = training.CheckpointManager(str(tmp_path), model, opt, Loader(), Loader())
        mgr.save(step=1)
        before = model.weight.detach().clone()
        path = os.path.join(str(tmp_path), mgr.DEFAULT_NAME)

        real_rename = os.rename
        calls = []

        def dying_rename(src, dst):
            if path not in (str(src), str(dst)):
                return real_rename(src, dst)  # the checkpoint writer's own renames inside its directory
            calls.append((src, dst))
            if len(calls) == 2:  # the first rename set the old checkpoint aside; the second never happens
                raise RuntimeError("injected: writer died between the renames")
            return real_rename(src, dst)

        monkeypatch.setattr(os, "rename", dying_rename)
        with torch.no_grad():
            model.weight.add_(1.0)
        with pytest.raises(RuntimeError, match="injected"):
            mgr.save(step=2)
        monkeypatch.setattr(os, "rename", real_rename)
        assert not os.path.isdir(path) and os.path.isdir(path + mgr.OLD_SUFFIX)
        with torch.no_grad():
            model.weight.zero_()
        mgr.load()
        torch.testing.assert_close(model.weight.detach(), before)
        # the next complete save cleans up
        mgr.save(step=3)
        assert os.path.isdir(path) and not os.path.isdir(path + mgr.OLD_SUFFIX)
        shutil.rmtree(path)
    finally:
        dist.destroy_process_group()


def test_reduce_scatter_hook_hands_out_symmetric_inputs_and_ordinary_outputs(monkeypatch):
    """Bookkeeping of the FSDP2 reduce-scatter hook, with a stand-in for the symmetric arena: the
    first buffer FSDP asks for (world * n elements) comes from alternating slots of the arena, the
    second one (n elements) is ordinary memory that may outlive the call, and requests the kernel
    cannot serve fall back to ordinary memory as well."""
    from dion_b200.parallel import fsdp_comm, symm

    class FakeArena:
        def __init__(self, nbytes):
            self.buf = torch.zeros(symm._FLAG_BYTES + nbytes, dtype=torch.uint8)

    class FakeSlots:
        def __init__(self):
            self.arena, self.slot_bytes, self.grown = None, 0, 0

        def ensure(self, nbytes):
            if self.arena is None or nbytes > self.slot_bytes:
                self.slot_bytes = max(1024, nbytes)
                self.arena = FakeArena(2 * self.slot_bytes)
                self.grown += 1
            return True

        def slot_offset(self, index):
            return symm._FLAG_BYTES + index * self.slot_bytes

    rs = fsdp_comm.SymmReduceScatter.__new__(fsdp_comm.SymmReduceScatter)
    rs.device, rs.world = torch.device("cpu"), 4
    rs._slots, rs._next, rs._events, rs._live = FakeSlots(), 0, [None, None], {}
    rs._pending_numel, rs._generation, rs.kernel_calls, rs.fallback_calls = None, 0, 0, 0

    monkeypatch.setattr(fsdp_comm, "_is_cuda", lambda device: True)   # the stand-in arena lives on the host
    a_in = rs.allocate((4 * 64,), dtype=torch.float32, device="cpu")
    a_out_ptr_is_slot = a_in.data_ptr() in rs._live
    assert a_out_ptr_is_slot and rs._pending_numel == 256
    base = rs._slots.arena.buf.data_ptr()
    assert a_in.data_ptr() == base + rs._slots.slot_offset(0)
    # the output request (pending / world elements) is served from ordinary memory and clears the pending mark
    out = rs.allocate((64,), dtype=torch.float32, device="cpu")
    assert rs._pending_numel is None and out.data_ptr() not in rs._live
    assert not (base <= out.data_ptr() < base + rs._slots.arena.buf.numel())
    # the next input goes to the other slot
    b_in = rs.allocate((4 * 64,), dtype=torch.float32, device="cpu")
    assert b_in.data_ptr() == base + rs._slots.slot_offset(1)
    rs.allocate((64,), dtype=torch.float32, device="cpu")
    # a size that is not a multiple of world * 16 bytes is never taken from the arena
    odd = rs.allocate((4 * 3,), dtype=torch.float32, device="cpu")
    assert odd.data_ptr() not in rs._live


def test_arena_sizing_converges_in_one_regrowth():
    """An arena that is too small records the total need of the step, not just the first request
    that failed, so the next arena fits every buffer of the step."""
    from dion_b200.parallel import symm

    def fake(capacity):
        a = symm.SymmetricArena.__new__(symm.SymmetricArena)
        a.capacity, a.cursor, a.high_water, a._views, a._guards = capacity, 0, 0, {}, []
        a.buf = torch.zeros(symm._FLAG_BYTES + capacity, dtype=torch.uint8)
        return a

    requests = [((1000,), torch.float32), ((3000,), torch.bfloat16), ((500, 4), torch.float32), ((7,), torch.float32)]
    small = fake(12000)
    got = [small.alloc(shape, dt) for shape, dt in requests]
    assert got[0] is not None and got[1] is not None and got[2] is None and got[3] is None
    need = small.high_water
    assert need >= 4000 + 6000 + 8000 + 28
    big = fake(int(need * 1.25))
    views = [big.alloc(shape, dt) for shape, dt in requests]
    assert all(v is not None for v in views)
    assert all(big.offset_of(v) is not None and big.offset_of(v) % 256 == 0 for v in views)
    big.reset()
    assert big.alloc((10,), torch.float32).data_ptr() == views[0].data_ptr()


def test_heartbeat_reports_departed_and_stalled_ranks_before_a_step_is_launched():
    import time

    import torch.distributed as dist

    from dion_b200.utils.health import RankFailure, StepHeartbeat

    store = dist.HashStore()
    a = StepHeartbeat(store, 0, 3, max_lag=2, stale_after_s=0.05)
    b = StepHeartbeat(store, 1, 3, max_lag=2, stale_after_s=0.05)
    c = StepHeartbeat(store, 2, 3, max_lag=2, stale_after_s=0.05)
    for step in range(3):
        for hb in (a, b, c):
            hb.check(step)
            hb.beat(step)
    b.leave()                                  # orderly departure between steps
    with pytest.raises(RankFailure) as e:
        a.check(3)
    assert e.value.ranks == [1]
    # rank 2 stops beating: tolerated while it is within max_lag or its beat is fresh ...
    store.set("dion_b200/heartbeat/1", f"9:{time.time()}")
    for step in range(3, 5):
        a.beat(step)
    a.check(5)
    time.sleep(0.08)
    a.beat(5)
    with pytest.raises(RankFailure) as e:      # ... and reported once it trails and went silent
        a.check(6)
    assert e.value.ranks == [2]
