"""Forwarder: optimizer base class and LR scaling (reference module dion/megabatch_base.py)."""
import dion_b200.optim.ortho_base as _m
from dion_b200.optim.ortho_base import *  # noqa: F401,F403
from dion_b200.parallel.megabatch import megabatch_orthogonalize_async  # noqa: E402,F401


def __getattr__(name):
    return getattr(_m, name)
