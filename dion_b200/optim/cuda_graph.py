"""Replay ``optimizer.step()`` from a CUDA graph.

The megabatch optimizers of this package issue the same kernels every step, never synchronize
with the host, read learning rate (and, when opted in, weight decay) from persistent device
tensors and keep AdamW's bias-correction counter on the device.  One recording therefore stays
valid for a whole run while an ordinary ``torch.optim`` scheduler keeps refreshing the LR tensor
between replays.  What this wrapper guarantees (the behaviours of dion/cuda_graph.py:88-313 in
the reference):

* ``warmup_steps`` eager steps come first: they allocate optimizer state, workspaces and
  exchange buffers.  The following step is recorded and executed by one replay; every later step
  is a replay.
* Recording is refused while a trainable parameter has no ``.grad``: it would be left out of the
  recording for good.  A refused or failed recording leaves nothing behind that could be replayed.
* Gradients have to keep their buffers, so ``zero_grad`` always zeroes in place.
* ``release()`` discards the recording (``add_param_group`` and ``load_state_dict`` do it
  implicitly).  Call it before ``destroy_process_group()`` when the recording holds collectives.
* A hyper-parameter that turns into a live device tensor only after the recording was made is an
  error, not a silent replay of the stale value.
"""
from __future__ import annotations

import warnings
from collections import OrderedDict
from typing import Callable, List, Optional

import torch

_HOOK_TABLES = (
    "_optimizer_step_pre_hooks", "_optimizer_step_post_hooks",
    "_optimizer_state_dict_pre_hooks", "_optimizer_state_dict_post_hooks",
    "_optimizer_load_state_dict_pre_hooks", "_optimizer_load_state_dict_post_hooks",
)


def _call_if_present(obj, name: str):
    fn = getattr(obj, name, None)
    return fn() if fn is not None else None


def supports_graph_replay(optimizer) -> bool:
    """True for optimizers whose step stays correct when replayed from a recording: learning rate
    in persistent device tensors refreshed through ``_sync_hyperparam_tensors``, AdamW counters
    on the device, host counters advanced through ``_advance_host_step_counters`` (the megabatch
    family).  Optimizers that pass ``group["lr"]`` or a step count to their kernels as host
    numbers (legacy Dion, DionReference, DionSimple, MuonReference, plain torch optimizers)
    would replay the values of the recorded step for ever."""
    return (callable(getattr(optimizer, "_sync_hyperparam_tensors", None))
            and callable(getattr(optimizer, "_advance_host_step_counters", None)))


def require_graph_replay_support(optimizer, what: str) -> None:
    if not supports_graph_replay(optimizer):
        raise TypeError(
            f"{what} needs an optimizer that keeps its learning rate and step counters in device "
            f"tensors (Muon, NorMuon, Dion2, NorDion2); {type(optimizer).__name__} passes them "
            f"as host numbers, so a replayed step would train at the recorded step's learning "
            f"rate and bias correction.  Run it without a CUDA graph.")


class CudaGraphOptimizer(torch.optim.Optimizer):
    """A ``torch.optim.Optimizer`` face on ``optimizer`` whose steps are recorded once and then
    replayed.  It owns no parameters or state of its own: ``param_groups`` and ``state`` are the
    inner optimizer's, so a scheduler can be attached to either object."""

    def __init__(self, optimizer: torch.optim.Optimizer, warmup_steps: int = 10,
                 capture_error_mode: str = "thread_local"):
        if warmup_steps < 1:
            raise ValueError(
                f"warmup_steps must be >= 1, got {warmup_steps}: at least one eager step has to "
                "run before a recording so that state and communication buffers exist.")
        # torch.optim.Optimizer.__init__ is deliberately not called (there are no parameters to
        # register); torch's profiling wrappers only need the hook tables to exist.
        for table in _HOOK_TABLES:
            setattr(self, table, OrderedDict())
        self.optimizer = optimizer
        self.warmup_steps = warmup_steps
        self.capture_error_mode = capture_error_mode
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._steps_taken = 0
        self._live_tensors_at_capture = 0
        self._told_about_set_to_none = False

    # -- everything else is the inner optimizer's ----------------------------------------------
    def __getattr__(self, name):
        if name == "optimizer":           # not constructed yet (e.g. during unpickling)
            raise AttributeError(name)
        return getattr(self.optimizer, name)

    param_groups = property(lambda self: self.optimizer.param_groups,
                            lambda self, groups: setattr(self.optimizer, "param_groups", groups))
    state = property(lambda self: self.optimizer.state)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state_dict):
        self.release()
        return self.optimizer.load_state_dict(state_dict)

    def add_param_group(self, param_group):
        self.release()
        return self.optimizer.add_param_group(param_group)

    def zero_grad(self, set_to_none: bool = False):
        if set_to_none and not self._told_about_set_to_none:
            self._told_about_set_to_none = True
            warnings.warn("a recorded step reads the gradients at fixed addresses: "
                          "set_to_none=True is ignored and gradients are zeroed in place.",
                          RuntimeWarning)
        self.optimizer.zero_grad(set_to_none=False)

    # -- recording -----------------------------------------------------------------------------
    def release(self) -> None:
        """Forget the recording; the next steps warm up and record again."""
        old, self._graph = self._graph, None
        self._steps_taken = 0
        self._live_tensors_at_capture = 0
        if old is not None:
            torch.cuda.synchronize()
            old.reset()

    def _on_cuda(self) -> bool:
        for group in self.param_groups:
            for p in group["params"]:
                return p.is_cuda
        return False

    def _count_live_tensors(self) -> int:
        return len(getattr(self.optimizer, "_hyperparam_tensors", None) or ())

    def _params_without_grad(self) -> List[str]:
        return [f"group {g}[{i}] shape {tuple(p.shape)}"
                for g, group in enumerate(self.param_groups)
                for i, p in enumerate(group["params"])
                if p.requires_grad and p.grad is None]

    def _record(self) -> None:
        require_graph_replay_support(self.optimizer, "CudaGraphOptimizer")
        orphans = self._params_without_grad()
        if orphans:
            listed = ", ".join(orphans[:5])
            if len(orphans) > 5:
                listed += f", ... (+{len(orphans) - 5} more)"
            raise RuntimeError(
                f"cannot record the optimizer step: {len(orphans)} trainable parameter(s) have "
                f"no .grad yet and would never be updated by replays: {listed}.  Record after "
                "every parameter has received a gradient (more warmup_steps), or freeze the "
                "ones that are meant to stay fixed (requires_grad=False).")
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode=self.capture_error_mode):
            self.optimizer.step()
        # Only a completed recording is kept.
        self._graph = graph
        self._live_tensors_at_capture = self._count_live_tensors()
        graph.replay()   # recording executed nothing on the device; this is that step's work

    def _replay(self) -> None:
        if self._count_live_tensors() != self._live_tensors_at_capture:
            raise RuntimeError(
                "a hyper-parameter became a live device tensor after the step was recorded "
                "(assigning a Tensor weight_decay is the way in); the recording holds the old "
                "host value and cannot see the tensor.  Opt in before the first recording or "
                "call release() to record again.")
        _call_if_present(self.optimizer, "_poll_device_status")
        self._graph.replay()
        _call_if_present(self.optimizer, "_snapshot_device_status")
        _call_if_present(self.optimizer, "_advance_host_step_counters")

    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._steps_taken < self.warmup_steps or not self._on_cuda():
            self.optimizer.step()      # warm-up, or nothing to record: parameters live on the host
        else:
            _call_if_present(self.optimizer, "_sync_hyperparam_tensors")
            if self._graph is None:
                self._record()
            else:
                self._replay()
        self._steps_taken += 1
        return loss
