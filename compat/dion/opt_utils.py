"""Forwarder: cooperative task runtime and DTensor helpers (reference module dion/opt_utils.py)."""
from dion_b200.parallel.async_runtime import AsyncRuntime, AsyncTask  # noqa: F401
from dion_b200.utils.tensors import (  # noqa: F401
    as_scalar_tensor, create_param_batches, dtensor_from_local, lm_head_lr_scale, pad_batch,
    to_local)
