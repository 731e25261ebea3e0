"""The reference's ``dion.dion_simple`` import path (dion/dion_simple.py:11-141): the single-device textbook
Dion as ``Dion`` and its update rule as ``dion_update``."""

from .optim.dion_simple import DionSimple, dion_simple_update  # noqa: F401

Dion = DionSimple
dion_update = dion_simple_update
