"""The reference's ``dion.newton_schulz_triton`` import path (dion/newton_schulz_triton.py:134-374).  The
kernels behind these names are the symmetric tcgen05 GEMMs of csrc/gemm.cu, not Triton programs; the names are
kept so that ``Muon(..., newton_schulz_func=newton_schulz_triton)`` and scripts that call ``ns_line_1`` /
``ns_line_2`` run unchanged."""

from .optim.newton_schulz import (  # noqa: F401
    newton_schulz,
    ns_line_1,
    ns_line_2,
    zeropower_via_newtonschulz5,
)

newton_schulz_triton = newton_schulz
