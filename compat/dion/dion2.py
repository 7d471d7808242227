"""Forwarder: Dion2 (reference module dion/dion2.py)."""
import dion_b200.optim.dion2 as _m
from dion_b200.optim.dion2 import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
