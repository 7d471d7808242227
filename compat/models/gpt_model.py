"""Forwarder: GPT decoder and its parallelization (reference module models/gpt_model.py)."""
import dion_b200.models.gpt as _m
from dion_b200.models.gpt import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)
