"""Forwarder: Dion3 alias (reference module dion/dion3.py)."""
import dion_b200.optim.dion3 as _m
from dion_b200.optim.dion3 import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
