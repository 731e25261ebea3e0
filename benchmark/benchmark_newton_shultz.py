"""The reference's file name (benchmark/benchmark_newton_shultz.py) for `benchmark/benchmark_newton_schulz.py`;
same options."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from benchmark_newton_schulz import main  # noqa: E402

if __name__ == "__main__":
    main()
