"""Locate the unmodified reference package (for oracle tests); None when unavailable."""
import importlib
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_reference():
    # the install made for the benchmark's reference arm, or a checkout named by DION_REFERENCE_PATH
    cands = [os.path.join(_ROOT, "baseline", "_ref")]
    if os.environ.get("DION_REFERENCE_PATH"):
        cands.append(os.environ["DION_REFERENCE_PATH"])
    for cand in cands:
        if os.path.isdir(os.path.join(cand, "dion")):
            # a different package called `dion` may be installed in site-packages
            if cand in sys.path:
                sys.path.remove(cand)
            sys.path.insert(0, cand)
            sys.modules.pop("dion", None)
            try:
                mod = importlib.import_module("dion")
            except Exception:  # pragma: no cover
                return None
            if os.path.abspath(mod.__file__).startswith(os.path.abspath(cand)):
                return mod
            return None
    return None
