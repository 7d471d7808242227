"""Forwarder: Polar Express drivers (reference module dion/polar_express.py)."""
import dion_b200.ops.newton_schulz as _m
from dion_b200.ops.newton_schulz import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
