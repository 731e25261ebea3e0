"""Kernel front ends.  CUDA tensors run the in-tree sm_100a kernels; CPU tensors run
PyTorch implementations of the same semantics (host-side tests and numerical oracles)."""

from . import _ext, runtime  # noqa: F401
from .dion_fused import dion_q_norm, dion_r_post, dion_r_post_reference, slot_reduce  # noqa: F401
from .gemm import gemm, gemm_reference  # noqa: F401
from .linalg import chol_inverse, chol_inverse_reference, col_sumsq, refine_prep, split_tf32  # noqa: F401
from .multi_tensor import (  # noqa: F401
    adamw_update,
    adamw_update_reference,
    cast_copy,
    dion_accumulate,
    lion_update,
    lion_update_reference,
    muon_apply,
    muon_momentum,
)
from .runtime import DionKernelError, check_status, launch_count  # noqa: F401
