#!/usr/bin/env python
"""``torchrun --standalone --nproc_per_node=N train.py --config configs/dion2_160m.yaml [flags]``.
Thin launcher; the trainer lives in ``dion_b200.trainer``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from dion_b200.trainer import main  # noqa: E402

if __name__ == "__main__":
    main()
