"""The reference's ``dion.muon_reference`` import path (dion/muon_reference.py:11-330)."""

from .optim.muon_reference import MuonKellerJordan, MuonReference, zeropower_fixed_coeffs  # noqa: F401

Muon = MuonReference
zeropower_via_newtonschulz5 = zeropower_fixed_coeffs
