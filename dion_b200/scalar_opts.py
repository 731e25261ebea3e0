"""The reference's ``dion.scalar_opts`` under its own names (dion/scalar_opts.py:6-187): AdamW and Lion updates
of one tensor or of a list of tensors, hyper-parameters as numbers or 0-dim tensors.  CUDA lists are updated by
one multi-tensor kernel launch (csrc/optim_kernels.cu)."""

from .optim.functional import adamw_update, adamw_update_foreach, lion_update, lion_update_foreach  # noqa: F401
