"""dion_b200: Blackwell-native orthonormal optimizers (Muon, Dion2, NorMuon, NorDion2, Dion)."""
__version__ = "0.1.0"
