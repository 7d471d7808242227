"""Forwarder: single-device Dion (reference module dion/dion_simple.py)."""
import dion_b200.optim.dion_simple as _m
from dion_b200.optim.dion_simple import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
