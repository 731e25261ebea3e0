"""Host compiler selection for code that goes through torch.compile (the reference arms of the benchmarks).

Inductor builds small host-side C++ files with OpenMP.  On some images the first ``g++`` on ``PATH`` cannot do
that (its ``libgomp.spec`` is missing) while the distribution's compiler can; Inductor honours ``CXX``.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import tempfile


def can_openmp(cxx: str) -> bool:
    """True when `cxx` compiles and links a trivial program with -fopenmp."""
    try:
        with tempfile.TemporaryDirectory() as d:
            src = os.path.join(d, "t.cpp")
            with open(src, "w") as f:
                f.write("int main() { return 0; }\n")
            return subprocess.run([cxx, "-fopenmp", src, "-o", os.path.join(d, "t")], capture_output=True,
                                  timeout=60).returncode == 0
    except Exception:
        return False


def ensure_openmp_cxx() -> str:
    """Point ``CXX`` at a compiler that can build OpenMP code, if the current choice cannot.  Returns the
    compiler in effect ('' when none was found)."""
    current = os.environ.get("CXX") or shutil.which("g++") or ""
    if current and can_openmp(current):
        return current
    for cand in ("/usr/bin/g++", "/usr/bin/clang++", "/usr/bin/g++-13", "/usr/bin/g++-12"):
        if os.path.exists(cand) and can_openmp(cand):
            os.environ["CXX"] = cand
            return cand
    return ""
