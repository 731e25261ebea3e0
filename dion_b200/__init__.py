"""dion_b200: Blackwell-native orthonormal-update optimizers (Dion, Muon) and the training
stack around them.  Public names match the reference package (dion/__init__.py:1-6)."""

from .optim import (  # noqa: F401
    Dion,
    DionMixedPrecisionConfig,
    DionReference,
    DionSimple,
    Muon,
    MuonKellerJordan,
    MuonReference,
)

__version__ = "0.1.0"
