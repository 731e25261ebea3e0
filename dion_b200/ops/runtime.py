"""Per-device runtime state shared by the CUDA ops: the device status word that
kernels set when a bounded wait gives up, and small cached workspaces."""

from __future__ import annotations

from typing import Dict

import torch

from . import _ext


class DionKernelError(RuntimeError):
    """A kernel reported a device-side failure (e.g. a pipeline or peer wait ran out)."""


_STATUS_NAMES = {
    1: "TMA producer wait timed out",
    2: "MMA issuer wait timed out",
    3: "epilogue wait timed out",
    4: "peer flag wait timed out",
    5: "bad kernel argument",
    6: "a bounds check of the debug build failed",
}

_status: Dict[int, torch.Tensor] = {}


def use_cuda_kernels(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU; raises if the extension is missing there."""
    if not t.is_cuda:
        return False
    _ext.load(required=True)
    return True


def status_tensor(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronising check of the device status word; raises DionKernelError if set."""
    if not torch.cuda.is_available():
        return
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        return
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise DionKernelError(f"dion_b200 kernel failure on cuda:{idx}: {_STATUS_NAMES.get(code, code)}")


def launch_count() -> int:
    """Kernel launches issued by this library in this process so far."""
    if not _ext.load(required=False):
        return 0
    return int(torch.ops.dion_b200.launch_count())
