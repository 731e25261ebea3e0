"""The reference's ``dion.dion`` import path: the batched :class:`Dion` optimizer and the free functions its
update is made of (dion/dion.py:34-1602)."""

from .optim.dion import Dion, DionMixedPrecisionConfig, _DionParamConfig  # noqa: F401
from .optim.functional import (  # noqa: F401
    adamw_update_allreduce_grad,
    all_reduce_replicate_mesh,
    column_normalize,
    distributed_orthogonalize,
    fix_all_zero_or_nan,
    foreach_baddbmm_,
    generate_random_sketch_matrix,
    lion_update_allreduce_grad,
    local_column_sum_sq,
    orthogonalize,
    tensor_list_to_batch,
    update_Q_matrix_,
)
