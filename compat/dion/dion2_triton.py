"""Forwarder: fused Dion2 apply ``x = a*x - b*u[map]`` (reference module dion/dion2_triton.py; the
kernel here is CUDA, ``dion_b200.ops.foreach.dion2_post``)."""
from dion_b200.ops.foreach import dion2_post  # noqa: F401
from dion_b200.optim.dion2 import dion2_post_orthogonalize  # noqa: F401

dion2_post_orthogonalize_triton = dion2_post_orthogonalize
