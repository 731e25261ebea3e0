"""Write uniform-random token shards in the FineWeb shard format.

    python data/synthetic.py --out data/synthetic --train-tokens 100000000 --val-tokens 10485760
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dion_b200.models.data import write_synthetic_shards

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--vocab-size", type=int, default=50304)
    ap.add_argument("--train-tokens", type=int, default=100_000_000)
    ap.add_argument("--val-tokens", type=int, default=10_485_760)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    write_synthetic_shards(a.out, a.vocab_size, a.train_tokens, a.val_tokens, a.seed)
    print(f"wrote shards to {a.out}")
