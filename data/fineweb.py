"""Tokenise FineWeb / FineWeb-edu with the GPT-2 tokenizer into shards of 100M tokens
(`fineweb_val_000000.bin`, `fineweb_train_000001.bin`, ...).  Needs `datasets`, `tiktoken`
and network access.  Shard format: see dion_b200.models.data.write_datafile
(reference: data/fineweb.py:32-155).

    python data/fineweb.py --version 10B --shard_size 100000000
"""
import argparse
import multiprocessing as mp
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dion_b200.models.data import write_datafile

_enc = None


def _tokenize(doc):
    global _enc
    if _enc is None:
        import tiktoken

        _enc = tiktoken.get_encoding("gpt2")
    eot = _enc._special_tokens["<|endoftext|>"]
    toks = np.array([eot] + _enc.encode_ordinary(doc["text"]))
    assert (0 <= toks).all() and (toks < 2 ** 16).all(), "token dictionary too large for uint16"
    return toks.astype(np.uint16)


def main():
    ap = argparse.ArgumentParser(description="FineWeb dataset preprocessing")
    ap.add_argument("-v", "--version", type=str, default="10B", help="10B, 100B, edu10B or edu100B")
    ap.add_argument("-s", "--shard_size", type=int, default=10 ** 8)
    args = ap.parse_args()
    names = {"10B": ("HuggingFaceFW/fineweb", "sample-10BT", "fineweb10B"),
             "100B": ("HuggingFaceFW/fineweb", "sample-100BT", "fineweb100B"),
             "edu10B": ("HuggingFaceFW/fineweb-edu", "sample-10BT", "finewebedu10B"),
             "edu100B": ("HuggingFaceFW/fineweb-edu", "sample-100BT", "finewebedu100B")}
    repo, remote, local = names[args.version]
    from datasets import load_dataset

    out_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), local)
    os.makedirs(out_dir, exist_ok=True)
    ds = load_dataset(repo, name=remote, split="train")
    shard = np.empty((args.shard_size,), dtype=np.uint16)
    fill, index = 0, 0
    with mp.Pool(max(1, (os.cpu_count() or 2) - 2)) as pool:
        for toks in pool.imap(_tokenize, ds, chunksize=16):
            while len(toks) > 0:
                take = min(len(toks), args.shard_size - fill)
                shard[fill:fill + take] = toks[:take]
                fill += take
                toks = toks[take:]
                if fill == args.shard_size:
                    split = "val" if index == 0 else "train"
                    write_datafile(os.path.join(out_dir, f"fineweb_{split}_{index:06d}.bin"), shard)
                    index, fill = index + 1, 0
    if fill:
        split = "val" if index == 0 else "train"
        write_datafile(os.path.join(out_dir, f"fineweb_{split}_{index:06d}.bin"), shard[:fill])


if __name__ == "__main__":
    main()
