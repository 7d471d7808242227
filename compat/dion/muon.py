"""Forwarder: Muon optimizer (reference module dion/muon.py)."""
import dion_b200.optim.muon as _m
from dion_b200.optim.muon import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
