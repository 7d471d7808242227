"""Forwarder: AdamW / Lion updates (reference module dion/scalar_opts.py)."""
import dion_b200.optim.scalar_opts as _m
from dion_b200.optim.scalar_opts import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
