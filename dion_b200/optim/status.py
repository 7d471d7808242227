"""How an optimizer learns that one of its kernels gave up on a wait.

The kernels of this package never hang: a wait that runs out of time (a peer GPU that never
delivered, a pipeline stage that never arrived) records a code in a device status word, and the
kernels that would have consumed the missing data leave weights and state untouched.  The host
learns of it without a synchronization of its own: each step ends with an asynchronous copy of
the record to pinned memory and begins by looking at the last copy that has landed, so an error
raises at the start of one of the next steps.  ``check_device_status()`` (blocking) is for the
points where the host synchronizes anyway, e.g. before a checkpoint.  The reference has no
counterpart: it avoids hangs by keeping every collective uniform
(dion/megabatch_base.py:716-782) and relies on NCCL's watchdog otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..utils.tensors import to_local


class DeviceStatusMixin:
    def _status_device(self) -> Optional[torch.device]:
        dev = getattr(self, "_status_dev", False)
        if dev is False:
            dev = None
            for group in self.param_groups:
                if group["params"]:
                    loc = to_local(group["params"][0])
                    dev = loc.device if loc.is_cuda else None
                    break
            self._status_dev = dev
        return dev

    def _poll_device_status(self) -> None:
        dev = self._status_device()
        if dev is not None:
            from ..ops import gemm

            gemm.poll_status(dev)

    def _snapshot_device_status(self) -> None:
        dev = self._status_device()
        if dev is not None:
            from ..ops import gemm

            gemm.snapshot_status(dev)

    def check_device_status(self) -> None:
        """Synchronize and raise if any kernel of this package reported a timeout."""
        dev = self._status_device()
        if dev is not None:
            from ..ops import gemm

            gemm.check_status(dev)
