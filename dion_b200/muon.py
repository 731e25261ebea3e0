"""The reference's ``dion.muon`` import path: the :class:`Muon` optimizer, its learning-rate scalings and the
free functions its update is made of (dion/muon.py:25-647)."""

from .optim.functional import (  # noqa: F401
    adamw_update_foreach_async,
    lion_update_foreach_async,
    muon_update_newton_schulz,
    muon_update_post_orthogonalize,
    muon_update_pre_orthogonalize,
)
from .optim.muon import Muon, adjust_lr_keller_muon, adjust_lr_rms_norm, adjust_lr_spectral_norm  # noqa: F401
from .optim.newton_schulz import zeropower_via_newtonschulz5  # noqa: F401
