"""Forwarder: batched low-rank Dion (reference module dion/dion.py)."""
import dion_b200.optim.dion as _m
from dion_b200.optim.dion import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
