"""Forwarder: unbatched Dion (reference module dion/dion_reference.py)."""
import dion_b200.optim.dion_reference as _m
from dion_b200.optim.dion_reference import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
