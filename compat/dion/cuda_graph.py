"""Forwarder: CudaGraphOptimizer (reference module dion/cuda_graph.py)."""
import dion_b200.optim.cuda_graph as _m
from dion_b200.optim.cuda_graph import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
