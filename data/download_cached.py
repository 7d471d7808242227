#!/usr/bin/env python
"""Fetch pre-tokenized GPT-2 shards from the Hugging Face hub instead of tokenizing locally
(the role of data/cached_fineweb10B.py, cached_fineweb100B.py and cached_finewebedu10B.py in the
reference).  Needs ``huggingface_hub`` and network access.

    python data/download_cached.py fineweb10B [num_train_chunks]
    python data/download_cached.py fineweb100B 200
    python data/download_cached.py finewebedu10B
"""
from __future__ import annotations

import os
import sys

# name -> (hub dataset, file prefix, number of 100M-token training chunks in the full set)
DATASETS = {
    "fineweb10B": ("kjj0/fineweb10B-gpt2", "fineweb", 103),
    "fineweb100B": ("kjj0/fineweb100B-gpt2", "fineweb", 1030),
    "finewebedu10B": ("kjj0/finewebedu10B-gpt2", "finewebedu", 99),
}


def shard_names(prefix: str, num_train: int):
    yield f"{prefix}_val_{0:06d}.bin"
    for i in range(1, num_train + 1):
        yield f"{prefix}_train_{i:06d}.bin"


def fetch(name: str, num_train: int | None = None, root: str | None = None) -> str:
    if name not in DATASETS:
        raise SystemExit(f"unknown dataset {name!r}; choose from {sorted(DATASETS)}")
    repo, prefix, full = DATASETS[name]
    num_train = full if num_train is None else min(num_train, full)
    local = os.path.join(root or os.path.dirname(os.path.abspath(__file__)), name)
    try:
        from huggingface_hub import hf_hub_download
    except ImportError as exc:  # pragma: no cover - optional dependency
        raise SystemExit("huggingface_hub is required: pip install huggingface_hub") from exc
    for fname in shard_names(prefix, num_train):
        if not os.path.exists(os.path.join(local, fname)):
            hf_hub_download(repo_id=repo, filename=fname, repo_type="dataset", local_dir=local)
    return local


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    fetch(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else None)
