"""Multi-process tests: host-side distributed logic on CPU (gloo, 2 ranks) and the same
cases plus the symmetric-memory kernels on GPUs (NCCL).  Every case runs in child
processes launched through torchrun; a rank that fails makes the launcher exit non-zero."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    """A port the kernel just handed out as free (two test processes running side by side cannot be
    given the same one, unlike a port derived from the process id)."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(cases, nproc, force_cpu, timeout=600, multicast=False):
    env = dict(os.environ)
    env["DION_TEST_FORCE_CPU"] = "1" if force_cpu else "0"
    env.setdefault("TORCHDYNAMO_DISABLE", "1")
    # in-tree kernels on plain peer loads / stores and NCCL without NVLS: a rank that dies
    # must not leave multicast bindings behind
    env["DION_B200_MULTICAST"] = "1" if multicast else "0"
    env["NCCL_NVLS_ENABLE"] = "0"
    env["DION_TEST_SOFT_FAIL"] = "1" if multicast else "0"
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "dist_worker.py"), *cases]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    tail = (res.stdout[-3000:] + "\n" + res.stderr[-3000:])
    assert res.returncode == 0 and "ALL OK" in res.stdout, tail


@pytest.mark.parametrize("case", ["dion_ddp", "muon_ddp", "fsdp", "fsdp_comm", "tp", "tp_sp", "structured", "checkpoint",
                                  "functional"])
def test_cpu_two_ranks(case):
    _launch([case], nproc=2, force_cpu=True)


@pytest.mark.parametrize("case", ["fsdp", "dion_ddp", "functional"])
def test_cpu_four_ranks(case):
    """The same cases with four ranks: batches that do not split evenly over the ranks, shares padded with
    zero matrices."""
    _launch([case], nproc=4, force_cpu=True, timeout=900)


def test_cpu_four_ranks_hybrid_meshes():
    _launch(["hybrid"], nproc=4, force_cpu=True, timeout=900)


@pytest.mark.gpu
def test_gpu_hybrid_meshes():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least 4 GPUs")
    _launch(["hybrid"], nproc=4, force_cpu=False, timeout=240)


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["symm", "dion_ddp", "muon_ddp", "fsdp", "fsdp_comm", "tp", "checkpoint"])
def test_gpu_ranks(case):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    # two ranks: the rank count these cases have been run with on GPUs (four ranks: the hybrid case above)
    _launch([case], nproc=2, force_cpu=False)


@pytest.mark.gpu
def test_gpu_symmetric_kernels_with_multimem():
    """The multimem.ld_reduce / multimem.st instantiations of the collectives (the default outside the
    tests).  No rank leaves early in this case: failures are recorded, the ranks agree on the verdict,
    tear down in order and only then exit non-zero."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch(["symm_multicast"], nproc=2, force_cpu=False, multicast=True)


@pytest.mark.gpu
@pytest.mark.skipif(os.environ.get("DION_B200_TP_FUSED_GATHER") != "1",
                    reason="the all-gather inside the GEMM kernel is opt-in (DION_B200_TP_FUSED_GATHER=1)")
def test_gpu_gemm_with_fused_all_gather():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch(["gemm_gather", "tp_sp"], nproc=2, force_cpu=False)
