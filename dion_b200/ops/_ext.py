"""Build and load the in-tree CUDA extension (``dion_b200/_C/dion_b200_C.so``).

The library is compiled for sm_100a only and registers its kernels as
``torch.ops.dion_b200.*``.  ``load()`` never compiles implicitly on a machine that has
a GPU but no built library: it raises, so that a silent PyTorch fallback cannot hide a
missing build.  ``build()`` cross-compiles and works without a GPU.
"""

from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import Optional

import torch

_PKG_DIR = Path(__file__).resolve().parent.parent
_SRC_DIR = _PKG_DIR / "csrc"
# DION_B200_DEBUG=1 selects the debug build: the same sources compiled with -DDION_B200_DEBUG, which turns on
# the bounds / consistency checks of the kernels (they report through the status word, nothing traps).  It
# lives beside the regular library, so both can exist in one tree; build it with
# `DION_B200_DEBUG=1 python -c "import __graft_entry__ as g; g.build()"`.
DEBUG = os.environ.get("DION_B200_DEBUG", "0") == "1"
_BUILD_DIR = _PKG_DIR / ("_C_debug" if DEBUG else "_C")
_LIB_NAME = "dion_b200_C_debug" if DEBUG else "dion_b200_C"
_SOURCES = ["bindings.cpp", "gemm.cu", "optim_kernels.cu", "nn_kernels.cu", "linalg.cu", "comm_kernels.cu",
            "noalloc.cu", "attention.cu", "dion_fused.cu", "llama_kernels.cu"]

_lock = threading.Lock()
_loaded: Optional[bool] = None
_load_error: Optional[str] = None


def sources() -> list[Path]:
    return [_SRC_DIR / s for s in _SOURCES if (_SRC_DIR / s).exists()]


def library_path() -> Path:
    return _BUILD_DIR / f"{_LIB_NAME}.so"


def _is_stale() -> bool:
    lib = library_path()
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(_SRC_DIR.glob("*.cu")) + list(_SRC_DIR.glob("*.cuh")) + list(_SRC_DIR.glob("*.h")) + list(
        _SRC_DIR.glob("*.cpp"))
    return any(p.stat().st_mtime > t for p in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every CUDA source for sm_100a into one shared library, in-tree."""
    from torch.utils import cpp_extension

    if not force and not _is_stale():
        return library_path()
    _BUILD_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=_LIB_NAME,
        sources=[str(p) for p in sources()],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=[
            "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "--expt-relaxed-constexpr", "-Xptxas", "-v",
        ] + (["-DDION_B200_DEBUG"] if DEBUG else []),
        build_directory=str(_BUILD_DIR),
        is_python_module=False,
        verbose=verbose,
    )
    return library_path()


def load(required: Optional[bool] = None) -> bool:
    """Load the shared library.  Returns True when the CUDA ops are registered.

    ``required`` defaults to ``torch.cuda.is_available()``: on a GPU machine a missing
    library is an error, on a CPU-only machine the callers use the PyTorch reference
    implementations (tests and host-side logic only).
    """
    global _loaded, _load_error
    if required is None:
        required = torch.cuda.is_available()
    with _lock:
        if _loaded is None:
            lib = library_path()
            if lib.exists():
                try:
                    torch.ops.load_library(str(lib))
                    _loaded = True
                except OSError as e:  # pragma: no cover - depends on the machine
                    _loaded = False
                    _load_error = f"{type(e).__name__}: {e}"
            else:
                _loaded = False
                _load_error = f"{lib} does not exist; run `python -c 'import __graft_entry__ as g; g.build()'`"
    if required and not _loaded:
        raise RuntimeError(f"dion_b200 CUDA extension is not available: {_load_error}")
    return bool(_loaded)


def is_loaded() -> bool:
    return bool(_loaded)
