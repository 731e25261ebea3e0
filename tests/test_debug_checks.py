"""Debug aids that stand in for a memory checker: guard words behind the buffers of a symmetric arena, and
the debug build of the kernels (bounds checks that report through the status word)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_arena_guard_words_catch_a_write_past_the_end_of_a_buffer(monkeypatch):
    import torch.distributed as dist

    from dion_b200.ops.runtime import DionKernelError
    from dion_b200.parallel import symm

    monkeypatch.setattr(symm, "_DEBUG", True)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29800 + os.getpid() % 100))
    dev = torch.device("cuda", 0)
    own = not dist.is_initialized()
    if own:
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        arena = symm.SymmetricArena(dist.group.WORLD, 1 << 20, dev)
        a = arena.alloc((1000,), torch.float32)
        b = arena.alloc((64, 3), torch.bfloat16)
        a.fill_(1.0)
        b.fill_(2.0)
        arena.reset()                     # guards intact: no complaint
        a = arena.alloc((1000,), torch.float32)
        b = arena.alloc((64, 3), torch.bfloat16)
        off = arena.offset_of(a)
        arena.buf[off + 4000 + 7] = 0     # one byte past the end of `a`
        with pytest.raises(DionKernelError, match="guard behind buffer 0"):
            arena.reset()
    finally:
        if own:
            dist.destroy_process_group()


@pytest.mark.gpu
def test_debug_build_of_the_kernels_runs_clean():
    """The library compiled with -DDION_B200_DEBUG (bounds / consistency checks in the kernels) gives the same
    results and leaves the status word clear on correct launches."""
    lib = os.path.join(ROOT, "dion_b200", "_C_debug", "dion_b200_C_debug.so")
    if not os.path.exists(lib):
        pytest.skip("the debug build is not in the tree (DION_B200_DEBUG=1 python -c 'import __graft_entry__ as g; g.build()')")
    code = """
import torch
from dion_b200 import ops
from dion_b200.ops import _ext
assert _ext.DEBUG and _ext.library_path().name == 'dion_b200_C_debug.so'
a = torch.randn(3, 300, 200, device='cuda'); b = torch.randn(3, 200, 160, device='cuda')
ref = a.double() @ b.double()
out = ops.gemm(a, b, split3=True)
assert ((out.double() - ref).abs().max() / ref.abs().max()) < 2e-5
x = torch.randn(2, 512, 768, device='cuda').bfloat16()
g = ops.gemm(x, x.transpose(1, 2), symmetric=True)
assert torch.equal(g, g.transpose(1, 2))
P = torch.randn(4, 1024, 512, device='cuda')
Z, info = ops.chol_inverse(P.transpose(1, 2) @ P)
Q = P @ Z.transpose(1, 2)
assert (Q.transpose(1, 2) @ Q - torch.eye(512, device='cuda')).abs().max() < 5e-3 and int(info.sum()) == 0
slots = torch.randn(3, 4, 64, 32, device='cuda'); o = torch.empty(4, 64, 32, device='cuda')
ops.slot_reduce(slots, o, None, None, [], 1.0)
assert torch.equal(o, slots[0] + slots[1] + slots[2])
ops.check_status()
print('DEBUG BUILD OK')
"""
    env = dict(os.environ, DION_B200_DEBUG="1", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "DEBUG BUILD OK" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
