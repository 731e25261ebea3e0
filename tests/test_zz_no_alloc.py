"""The allocation-free C entry point (dion_chol_inverse_noalloc) against the regular
chol_inverse op.

Some callers of this library cannot allocate device memory - code inside a capture or
replay region of a framework that forbids allocation, latency-critical loops that cannot
afford the device synchronisation an allocation implies, hosts that pre-allocate a fixed
budget.  For them the library exports one C symbol whose scratch memory is a fixed array
inside the library image.  This test calls that symbol through ctypes, exactly as such a
caller would, and checks its output against the allocating entry point on two calls in a
row (the second call reuses the scratch the first one dirtied).

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch


def _library():
    from dion_b200.ops import _ext

    _ext.load(required=True)
    lib = ctypes.CDLL(str(_ext.library_path()))
    fn = lib.dion_chol_inverse_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p]
    lib.dion_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _gram(batch, m, r, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    P = torch.randn(batch, m, r, device="cuda", generator=g)
    return P, (P.transpose(-1, -2) @ P).contiguous()


@pytest.mark.gpu
def test_noalloc_entry_point_matches_regular_op_twice():
    from dion_b200 import ops

    lib, fn = _library()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (batch, r, seed) in enumerate([(6, 192, 1), (3, 256, 2)]):
        P, G = _gram(batch, 4 * r, r, seed)
        Z_ref, info_ref = ops.chol_inverse(G, 1e-6)
        Z = torch.empty_like(Z_ref)
        info = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
        rc = fn(G.data_ptr(), Z.data_ptr(), info.data_ptr(), batch, r, G.stride(1), G.stride(0), 1e-6, stream)
        assert rc == 0, lib.dion_noalloc_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(Z, Z_ref, rtol=1e-5, atol=1e-6)
        assert torch.equal(info, info_ref)
        Q = P @ Z.transpose(-1, -2)
        eye = torch.eye(r, device="cuda")
        assert (Q.transpose(-1, -2) @ Q - eye).abs().max() < 5e-3, f"call {call}"


@pytest.mark.gpu
def test_noalloc_entry_point_rejects_oversized_requests():
    lib, fn = _library()
    G = torch.eye(8, device="cuda").repeat(2, 1, 1).contiguous()
    Z = torch.empty_like(G)
    info = torch.zeros(2, dtype=torch.int32, device="cuda")
    # 2048 matrices of 64 x 64 would need 8 Mi floats of scratch: four times the built-in array
    rc = fn(G.data_ptr(), Z.data_ptr(), info.data_ptr(), 2048, 64, 64, 64 * 64, 1e-6, None)
    assert rc == 1
    msg = lib.dion_noalloc_last_error().decode()
    assert "exceeds the built-in scratch" in msg
    rc = fn(None, Z.data_ptr(), info.data_ptr(), 1, 8, 8, 64, 1e-6, None)
    assert rc == 1 and lib.dion_noalloc_last_error().decode() != ""
