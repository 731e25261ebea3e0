from .dion import Dion, DionMixedPrecisionConfig  # noqa: F401
from .dion_reference import DionReference  # noqa: F401
from .dion_simple import DionSimple  # noqa: F401
from .muon import Muon  # noqa: F401
from .muon_reference import MuonKellerJordan, MuonReference  # noqa: F401
from .newton_schulz import newton_schulz, zeropower_via_newtonschulz5  # noqa: F401
