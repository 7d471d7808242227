#!/usr/bin/env python
"""`python data/fineweb.py [-s SHARD_SIZE]`: tokenize FineWeb-edu into `.bin` shards (the command
line of the reference's script of the same name); the work is done by prepare_fineweb.main."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from prepare_fineweb import main  # noqa: E402

if __name__ == "__main__":
    main()
