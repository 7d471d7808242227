"""Forwarder: all-gather Muon (reference module dion/muon_reference.py)."""
import dion_b200.optim.muon_reference as _m
from dion_b200.optim.muon_reference import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
