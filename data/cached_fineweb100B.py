#!/usr/bin/env python
"""`python data/cached_fineweb100B.py [num_train_chunks]`: fetch the pre-tokenized fineweb100B shards (the command
line of the reference's script of the same name); the work is done by download_cached.fetch."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from download_cached import fetch  # noqa: E402

if __name__ == "__main__":
    fetch("fineweb100B", int(sys.argv[1]) if len(sys.argv) > 1 else None)
