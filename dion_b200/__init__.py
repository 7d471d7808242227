"""dion_b200: Blackwell-native orthonormal optimizers.

Public names match the reference package (dion/__init__.py:1-10): ``Muon``, ``Dion2``,
``NorMuon``, ``NorDion2``, ``Dion3``, ``Dion``, ``DionMixedPrecisionConfig``, ``DionSimple``,
``DionReference``, ``MuonReference`` and ``CudaGraphOptimizer``.
"""
__version__ = "0.1.0"

_LAZY = {
    "Muon": ("dion_b200.optim.muon", "Muon"),
    "NorMuon": ("dion_b200.optim.normuon", "NorMuon"),
    "Dion2": ("dion_b200.optim.dion2", "Dion2"),
    "NorDion2": ("dion_b200.optim.nordion2", "NorDion2"),
    "Dion3": ("dion_b200.optim.dion3", "Dion3"),
    "Dion": ("dion_b200.optim.dion", "Dion"),
    "DionMixedPrecisionConfig": ("dion_b200.optim.dion", "DionMixedPrecisionConfig"),
    "DionSimple": ("dion_b200.optim.dion_simple", "Dion"),
    "DionReference": ("dion_b200.optim.dion_reference", "Dion"),
    "MuonReference": ("dion_b200.optim.muon_reference", "Muon"),
    "MuonKellerJordan": ("dion_b200.optim.muon_reference", "MuonKellerJordan"),
    "CudaGraphOptimizer": ("dion_b200.optim.cuda_graph", "CudaGraphOptimizer"),
}

__all__ = list(_LAZY)


def __getattr__(name):
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(f"module 'dion_b200' has no attribute {name!r}")
    import importlib

    value = getattr(importlib.import_module(target[0]), target[1])
    globals()[name] = value
    return value
