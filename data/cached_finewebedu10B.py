"""`python data/cached_finewebedu10B.py [num_train_shards]`: the reference's script name for
`python data/cached_fineweb.py --version edu10B [num_train_shards]` (data/cached_finewebedu10B.py there)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from cached_fineweb import main  # noqa: E402

if __name__ == "__main__":
    main(["--version", "edu10B", *sys.argv[1:]])
