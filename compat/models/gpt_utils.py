"""Forwarder: token-shard data loaders (reference module models/gpt_utils.py)."""
import dion_b200.models.data as _m
from dion_b200.models.data import *  # noqa: F401,F403


def __getattr__(name):
    return getattr(_m, name)

_load_data_shard = _m._read_shard      # the reference's name of the shard reader
