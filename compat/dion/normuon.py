"""Forwarder: NorMuon (reference module dion/normuon.py)."""
import dion_b200.optim.normuon as _m
from dion_b200.optim.normuon import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
