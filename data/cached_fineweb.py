"""Download pre-tokenised GPT-2 FineWeb shards from the Hugging Face hub (network needed).

    python data/cached_fineweb.py --version 10B [num_train_shards]

Versions: 10B -> kjj0/fineweb10B-gpt2, 100B -> kjj0/fineweb100B-gpt2,
edu10B -> kjj0/finewebedu10B-gpt2 (references: data/cached_fineweb10B.py,
data/cached_fineweb100B.py, data/cached_finewebedu10B.py).
"""
import argparse
import os

REPOS = {"10B": ("kjj0/fineweb10B-gpt2", "fineweb10B", "fineweb", 103),
         "100B": ("kjj0/fineweb100B-gpt2", "fineweb100B", "fineweb", 1030),
         "edu10B": ("kjj0/finewebedu10B-gpt2", "finewebedu10B", "finewebedu", 99)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--version", default="10B", choices=sorted(REPOS))
    ap.add_argument("num_chunks", nargs="?", type=int, default=None)
    a = ap.parse_args(argv)
    from huggingface_hub import hf_hub_download

    repo, local, prefix, total = REPOS[a.version]
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), local)
    os.makedirs(out, exist_ok=True)

    def get(name):
        if not os.path.exists(os.path.join(out, name)):
            hf_hub_download(repo_id=repo, filename=name, repo_type="dataset", local_dir=out)

    get(f"{prefix}_val_{0:06d}.bin")
    for i in range(1, (a.num_chunks or total) + 1):
        get(f"{prefix}_train_{i:06d}.bin")


if __name__ == "__main__":
    main()
