"""Dion3 is the public name of NorDion2 (reference: dion/dion3.py:16)."""
from .nordion2 import NorDion2

Dion3 = NorDion2

__all__ = ["Dion3"]
