"""Capture ``optimizer.step()`` in a CUDA graph and replay it.

The megabatch optimizers issue a fixed sequence of kernels per step with no host
synchronization, read their learning rate (and optionally weight decay) from persistent device
tensors and advance AdamW's bias-correction counter on the device, so one captured graph stays
valid for the whole run while a stock ``torch.optim`` scheduler keeps filling the LR tensor
outside the graph.  Behaviour follows dion/cuda_graph.py:88-313 of the reference:

* the first ``warmup_steps`` steps run eagerly (they allocate state, workspaces and exchange
  buffers); the next step is captured and replayed once; later steps only replay;
* capture refuses to start while a ``requires_grad`` parameter has ``.grad is None`` - such a
  parameter would be left out of the graph for good;
* gradients must live in stable ``.grad`` buffers: ``zero_grad`` always zeroes in place;
* ``release()`` drops the graph (``add_param_group`` / ``load_state_dict`` call it too); call
  it before ``destroy_process_group()`` when the graph holds collectives;
* a group that starts carrying a hyper-parameter as a device tensor after capture raises
  instead of silently replaying the value baked at capture.
"""
from __future__ import annotations

import warnings
from collections import OrderedDict
from typing import Callable, Optional

import torch


class CudaGraphOptimizer(torch.optim.Optimizer):
    """``torch.optim.Optimizer`` facade around ``optimizer`` with captured steps.  All state
    lives in the inner optimizer; ``param_groups`` is shared, so an LR scheduler may be built on
    either object."""

    def __init__(self, optimizer: torch.optim.Optimizer, warmup_steps: int = 10,
                 capture_error_mode: str = "thread_local"):
        if warmup_steps < 1:
            raise ValueError(
                f"warmup_steps must be >= 1, got {warmup_steps}. Capture needs at least one "
                "eager step to have allocated the optimizer state and communication buffers.")
        # Optimizer.__init__ is skipped on purpose: this object owns no parameters.  The hook
        # tables it would create are still expected by torch's profiling wrappers.
        self.optimizer = optimizer
        self.warmup_steps = warmup_steps
        self.capture_error_mode = capture_error_mode
        self._step_count = 0
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._captured_hyperparam_count = 0
        self._warned_set_to_none = False
        for name in ("_optimizer_step_pre_hooks", "_optimizer_step_post_hooks",
                     "_optimizer_state_dict_pre_hooks", "_optimizer_state_dict_post_hooks",
                     "_optimizer_load_state_dict_pre_hooks",
                     "_optimizer_load_state_dict_post_hooks"):
            setattr(self, name, OrderedDict())

    # -- delegation ---------------------------------------------------------------------------
    def __getattr__(self, name):
        if name == "optimizer":
            raise AttributeError(name)
        return getattr(self.optimizer, name)

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @param_groups.setter
    def param_groups(self, value):
        self.optimizer.param_groups = value

    @property
    def state(self):
        return self.optimizer.state

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state_dict):
        self.release()
        return self.optimizer.load_state_dict(state_dict)

    def add_param_group(self, param_group):
        self.release()
        return self.optimizer.add_param_group(param_group)

    def zero_grad(self, set_to_none: bool = False):
        if set_to_none and not self._warned_set_to_none:
            self._warned_set_to_none = True
            warnings.warn(
                "CudaGraphOptimizer needs stable .grad buffers for graph replay; ignoring "
                "set_to_none=True and zeroing in place.", RuntimeWarning)
        self.optimizer.zero_grad(set_to_none=False)

    # -- graph lifetime -----------------------------------------------------------------------
    def release(self) -> None:
        """Drop the captured graph; the next steps warm up and capture again."""
        graph, self._graph = self._graph, None
        self._captured_hyperparam_count = 0
        self._step_count = 0
        if graph is not None:
            torch.cuda.synchronize()
            graph.reset()

    def _live_hyperparam_count(self) -> int:
        tensors = getattr(self.optimizer, "_hyperparam_tensors", None)
        return len(tensors) if tensors is not None else 0

    def _check_live_hyperparams_unchanged(self) -> None:
        if self._live_hyperparam_count() != self._captured_hyperparam_count:
            raise RuntimeError(
                "a param group started carrying a hyperparameter as a live device tensor after "
                "the CUDA graph was captured (weight_decay=Tensor is the way in). The captured "
                "graph baked the previous host value and cannot read the new tensor. Opt in "
                "before the first capture, or call release() to re-capture.")

    def _check_params_have_grads(self) -> None:
        missing = [
            f"group {gi}[{pi}] shape {tuple(p.shape)}"
            for gi, group in enumerate(self.param_groups)
            for pi, p in enumerate(group["params"])
            if p.requires_grad and p.grad is None
        ]
        if missing:
            shown = ", ".join(missing[:5]) + (f", ... (+{len(missing) - 5} more)" if len(missing) > 5 else "")
            raise RuntimeError(
                f"{len(missing)} parameter(s) require a gradient but have .grad=None at CUDA graph "
                f"capture, so replay would never update them: {shown}. Capture after every "
                "parameter has taken part in a backward pass (raise warmup_steps), or set "
                "requires_grad=False on the ones that are meant to be frozen.")

    def _sync_host_hyperparams(self) -> None:
        sync = getattr(self.optimizer, "_sync_hyperparam_tensors", None)
        if sync is not None:
            sync()

    def _capture(self) -> None:
        self._check_params_have_grads()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        # A failed capture leaves self._graph unset, so nothing half-built is ever replayed.
        with torch.cuda.graph(graph, capture_error_mode=self.capture_error_mode):
            self.optimizer.step()
        self._graph = graph
        self._captured_hyperparam_count = self._live_hyperparam_count()
        graph.replay()

    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._step_count < self.warmup_steps:
            self.optimizer.step()
        else:
            self._sync_host_hyperparams()
            if self._graph is None:
                self._capture()
            else:
                self._check_live_hyperparams_unchanged()
                self._graph.replay()
                advance = getattr(self.optimizer, "_advance_host_step_counters", None)
                if advance is not None:
                    advance()
        self._step_count += 1
        return loss
