"""Token loaders for the trainer.

* ``DistributedDataLoader``  strided reader over ``.bin`` shards in the reference's format
  (256 x int32 header with magic 20240520 and version 1, then uint16 tokens;
  models/gpt_utils.py:27-104), with a checkpointable position per data-parallel rank.
* ``ArithmeticDistributedDataLoader``  header-less uint16 files (models/gpt_utils.py:107-168).
* ``SyntheticDataLoader``  uniform-random token ids from a fixed seed, for benchmarks and tests.
* ``write_datafile``  writes a shard in the same format (data/fineweb.py:32-60).

Every loader stages its batch in pinned host memory and copies it to the GPU with one
asynchronous transfer; on a machine without a GPU the tensors stay on the CPU.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

MAGIC = 20240520
VERSION = 1
HEADER_INTS = 256


def write_datafile(filename: str, tokens) -> None:
    """Write ``tokens`` (values < 2**16) as one shard."""
    toks = np.asarray(tokens)
    assert toks.size < 2 ** 31, "token count too large"
    assert toks.min(initial=0) >= 0 and toks.max(initial=0) < 2 ** 16, "tokens must fit uint16"
    header = np.zeros(HEADER_INTS, dtype=np.int32)
    header[0], header[1], header[2] = MAGIC, VERSION, toks.size
    with open(filename, "wb") as f:
        f.write(header.tobytes())
        f.write(toks.astype(np.uint16).tobytes())


def _read_shard(filename: str) -> np.ndarray:
    with open(filename, "rb") as f:
        header = np.frombuffer(f.read(HEADER_INTS * 4), dtype=np.int32)
        if header[0] != MAGIC:
            raise ValueError(f"{filename}: magic number mismatch in the data .bin file")
        if header[1] != VERSION:
            raise ValueError(f"{filename}: unsupported version {header[1]}")
        tokens = np.frombuffer(f.read(), dtype=np.uint16)
    if len(tokens) != header[2]:
        raise ValueError(f"{filename}: header claims {header[2]} tokens, file holds {len(tokens)}")
    return tokens


class _DeviceStager:
    """Pinned host buffer pair + async copy of an (inputs, targets) batch."""

    def __init__(self, B: int, T: int, device: Optional[torch.device]):
        self.device = device
        self.use_cuda = device is not None and device.type == "cuda"
        self.host = torch.empty((2, B, T), dtype=torch.int64)
        if self.use_cuda:
            self.host = self.host.pin_memory()

    def push(self, window: np.ndarray, B: int, T: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``window`` holds ``B*T + 1`` consecutive tokens."""
        w = torch.from_numpy(window.astype(np.int64))
        self.host[0].copy_(w[:-1].view(B, T))
        self.host[1].copy_(w[1:].view(B, T))
        if self.use_cuda:
            dev = self.host.to(self.device, non_blocking=True)
            return dev[0], dev[1]
        return self.host[0].clone(), self.host[1].clone()

    def bytes_per_batch(self) -> int:
        return self.host.numel() * self.host.element_size()


def _default_device() -> Optional[torch.device]:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None


class DistributedDataLoader:
    def __init__(self, filename_pattern: str, B: int, T: int, dp_rank: int, dp_world_size: int,
                 device: Optional[torch.device] = None):
        self.B, self.T = B, T
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self.files = sorted(glob.glob(filename_pattern))
        if not self.files:
            raise FileNotFoundError(
                f"Could not find any files matching the pattern {filename_pattern}")
        self._stager = _DeviceStager(B, T, device if device is not None else _default_device())
        self.reset()

    def _open(self, shard: int) -> None:
        self.current_shard = shard % len(self.files)
        self.current_position = self.dp_rank * self.B * self.T
        self.tokens = _read_shard(self.files[self.current_shard])

    def reset(self) -> None:
        self._open(0)

    def advance(self) -> None:
        self._open(self.current_shard + 1)

    def next_batch(self):
        span = self.B * self.T
        window = self.tokens[self.current_position:self.current_position + span + 1]
        out = self._stager.push(window, self.B, self.T)
        self.current_position += span * self.dp_world_size
        if self.current_position + span * self.dp_world_size + 1 > len(self.tokens):
            self.advance()
        return out

    def state_dict(self) -> Dict[str, int]:
        return {
            f"current_shard_rank_{self.dp_rank}": self.current_shard,
            f"current_position_rank_{self.dp_rank}": self.current_position,
            "dataloader_world_size": self.dp_world_size,
        }

    def load_state_dict(self, state: dict) -> None:
        if state.get("dataloader_world_size") != self.dp_world_size:
            raise NotImplementedError(
                "DistributedDataLoader does not support redistributing checkpoints to a different "
                f"world size. Current process has world size {self.dp_world_size}, but checkpoint "
                f"has size {state.get('dataloader_world_size')}.")
        shard = state[f"current_shard_rank_{self.dp_rank}"]
        position = state[f"current_position_rank_{self.dp_rank}"]
        self._open(shard)
        self.current_position = position


class ArithmeticDistributedDataLoader:
    """Header-less uint16 ``{split}.bin``: strided circular reading when the file is long enough,
    random windows otherwise."""

    def __init__(self, data_dir: str, B: int, T: int, rank: int, world_size: int,
                 split: str = "train", device: Optional[torch.device] = None):
        self.B, self.T, self.rank, self.world_size = B, T, rank, world_size
        path = os.path.join(data_dir, f"{split}.bin")
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        self.tokens = np.fromfile(path, dtype=np.uint16)
        self.ntok = len(self.tokens)
        self._stager = _DeviceStager(B, T, device if device is not None else _default_device())
        self.reset()

    def reset(self) -> None:
        self.pos = self.rank * self.B * self.T

    def next_batch(self):
        need = self.B * self.T + 1
        if self.ntok >= need:
            idx = (self.pos + np.arange(need)) % self.ntok
            self.pos = (self.pos + self.world_size * self.B * self.T) % self.ntok
            return self._stager.push(self.tokens[idx], self.B, self.T)
        hi = self.ntok - self.T - 1
        assert hi > 0, f"split too small: ntok={self.ntok}, need at least T+1={self.T + 1}"
        starts = np.random.randint(0, hi + 1, size=self.B)
        x = np.stack([self.tokens[s:s + self.T] for s in starts]).astype(np.int64)
        y = np.stack([self.tokens[s + 1:s + self.T + 1] for s in starts]).astype(np.int64)
        st = self._stager
        st.host[0].copy_(torch.from_numpy(x))
        st.host[1].copy_(torch.from_numpy(y))
        if st.use_cuda:
            dev = st.host.to(st.device, non_blocking=True)
            return dev[0], dev[1]
        return st.host[0].clone(), st.host[1].clone()


class SyntheticDataLoader:
    """Uniform-random token ids in ``[0, vocab_size)``; the stream is a function of
    ``(seed, rank, step)`` only, so runs are reproducible and ranks see different data."""

    def __init__(self, B: int, T: int, vocab_size: int, dp_rank: int = 0, dp_world_size: int = 1,
                 seed: int = 0, device: Optional[torch.device] = None):
        self.B, self.T, self.vocab_size = B, T, vocab_size
        self.dp_rank, self.dp_world_size, self.seed = dp_rank, dp_world_size, seed
        self.step = 0
        self._stager = _DeviceStager(B, T, device if device is not None else _default_device())

    def reset(self) -> None:
        self.step = 0

    def next_batch(self):
        rng = np.random.default_rng([self.seed, self.dp_rank, self.step])
        self.step += 1
        window = rng.integers(0, self.vocab_size, size=self.B * self.T + 1, dtype=np.int64)
        return self._stager.push(window, self.B, self.T)

    def bytes_per_batch(self) -> int:
        return self._stager.bytes_per_batch()

    def state_dict(self) -> Dict[str, int]:
        return {f"step_rank_{self.dp_rank}": self.step, "dataloader_world_size": self.dp_world_size}

    def load_state_dict(self, state: dict) -> None:
        if state.get("dataloader_world_size") != self.dp_world_size:
            raise NotImplementedError("SyntheticDataLoader cannot change world size on resume")
        self.step = state[f"step_rank_{self.dp_rank}"]
