"""Forwarder: NorDion2 (reference module dion/nordion2.py)."""
import dion_b200.optim.nordion2 as _m
from dion_b200.optim.nordion2 import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
