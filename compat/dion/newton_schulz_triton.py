"""Forwarder: Newton-Schulz drivers (reference module dion/newton_schulz_triton.py; the kernels here are CUDA, not Triton)."""
import dion_b200.ops.newton_schulz as _m
from dion_b200.ops.newton_schulz import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
