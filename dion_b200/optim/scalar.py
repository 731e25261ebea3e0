"""Single-tensor AdamW and Lion updates used by the reference-style (per-parameter)
optimizers; the batched optimizers use ops.adamw_update / ops.lion_update on lists.
Math: dion/scalar_opts.py:6-86."""

from __future__ import annotations

from torch import Tensor

from .. import ops


def adamw_update(X: Tensor, G: Tensor, M: Tensor, V: Tensor, lr: float, beta1: float, beta2: float,
                 weight_decay: float, step: int, epsilon: float) -> None:
    ops.adamw_update([X], [G], [M], [V], lr=float(lr), beta1=float(beta1), beta2=float(beta2),
                     weight_decay=float(weight_decay), step=int(step), epsilon=float(epsilon))


def lion_update(X: Tensor, G: Tensor, M: Tensor, lr: float, beta1: float, beta2: float,
                weight_decay: float) -> None:
    ops.lion_update([X], [G], [M], lr=float(lr), beta1=float(beta1), beta2=float(beta2),
                    weight_decay=float(weight_decay))
