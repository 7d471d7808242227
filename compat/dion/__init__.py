"""Import-name compatibility: ``from dion import Muon, Dion2, Dion, NorMuon, ...`` resolves to the
classes of ``dion_b200`` (same constructor arguments, param-group keys and state_dict layout as
the reference's dion/__init__.py:1-10)."""
import dion_b200 as _impl

__version__ = _impl.__version__
__all__ = [n for n in _impl.__all__]


def __getattr__(name):
    if name in _impl.__all__:
        value = getattr(_impl, name)
        globals()[name] = value
        return value
    raise AttributeError(f"module 'dion' has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | set(__all__))
