"""Token-shard data loading for the GPT trainer.

Shard format (models/gpt_utils.py:7-37, data/fineweb.py:32-60): a header of 256 int32
(``[0] = 20240520`` magic, ``[1] = 1`` version, ``[2] = number of tokens``) followed by the
tokens as uint16.  :class:`DistributedDataLoader` walks rank-strided windows of ``B*T + 1``
tokens exactly like the reference loader (same positions, same shard roll-over, same
state-dict keys), but reads through a memory map, stages each batch in pinned host memory
and issues the host-to-device copy on a side stream one batch ahead, so the training stream
never waits for the copy.
"""

from __future__ import annotations

import glob
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

SHARD_MAGIC = 20240520
SHARD_VERSION = 1
HEADER_INTS = 256


def write_datafile(filename: str, toks) -> None:
    """Write one token shard (header + uint16 tokens)."""
    n = len(toks)
    assert n < 2 ** 31, "token count too large"
    header = np.zeros(HEADER_INTS, dtype=np.int32)
    header[0], header[1], header[2] = SHARD_MAGIC, SHARD_VERSION, n
    arr = toks if isinstance(toks, np.ndarray) and toks.dtype == np.uint16 else None
    if arr is None:
        arr = np.asarray(toks)
        assert arr.min(initial=0) >= 0 and arr.max(initial=0) < 2 ** 16, "token dictionary too large for uint16"
        arr = arr.astype(np.uint16)
    with open(filename, "wb") as f:
        f.write(header.tobytes())
        f.write(arr.tobytes())


def write_synthetic_shards(data_dir: str, vocab_size: int, train_tokens: int, val_tokens: int, seed: int = 0,
                           prefix: str = "fineweb") -> None:
    """Uniform-random token shards named like the FineWeb ones (``<prefix>_train_000001.bin``,
    ``<prefix>_val_000000.bin``), for benchmarks and tests without a dataset."""
    os.makedirs(data_dir, exist_ok=True)
    rng = np.random.default_rng(seed)
    for name, n in ((f"{prefix}_val_000000.bin", val_tokens), (f"{prefix}_train_000001.bin", train_tokens)):
        write_datafile(os.path.join(data_dir, name), rng.integers(0, vocab_size, size=n, dtype=np.uint16))


def _read_header(filename: str) -> int:
    with open(filename, "rb") as f:
        header = np.frombuffer(f.read(HEADER_INTS * 4), dtype=np.int32)
    if header[0] != SHARD_MAGIC:
        raise ValueError(f"{filename}: magic number mismatch in the data .bin file")
    if header[1] != SHARD_VERSION:
        raise ValueError(f"{filename}: unsupported version {header[1]}")
    return int(header[2])


def _map_shard(filename: str) -> np.ndarray:
    ntok = _read_header(filename)
    tokens = np.memmap(filename, dtype=np.uint16, mode="r", offset=HEADER_INTS * 4)
    if len(tokens) != ntok:
        raise ValueError(f"{filename}: number of tokens read does not match header")
    return tokens


class DistributedDataLoader:
    """Rank ``dp_rank`` of ``dp_world_size`` reads windows ``[pos, pos + B*T + 1)`` with
    ``pos`` starting at ``dp_rank * B * T`` and advancing by ``B * T * dp_world_size``; when
    the next window would not fit, the loader moves to the next shard
    (models/gpt_utils.py:40-104)."""

    def __init__(self, filename_pattern: str, B: int, T: int, dp_rank: int, dp_world_size: int,
                 device: Optional[torch.device] = None, prefetch: bool = True):
        self.dp_rank = dp_rank
        self.dp_world_size = dp_world_size
        self.B = B
        self.T = T
        self.files = sorted(glob.glob(filename_pattern))
        if len(self.files) < 1:
            raise FileNotFoundError(f"Could not find any files matching the pattern {filename_pattern}")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self._cuda = self.device.type == "cuda"
        self._prefetch = prefetch and self._cuda
        self._stream = torch.cuda.Stream(device=self.device) if self._cuda else None
        self._pinned = [torch.empty(B * T + 1, dtype=torch.int64).pin_memory() for _ in range(2)] if self._cuda else None
        self._slot = 0
        self._slot_events = [None, None]
        self._staged: Optional[Tuple[torch.Tensor, torch.Tensor, torch.cuda.Event]] = None
        self.reset()

    # -- position bookkeeping (identical to the reference)
    def _load_tokens_for_current_shard(self):
        self.tokens = _map_shard(self.files[self.current_shard])

    def reset(self):
        self.current_shard = 0
        self.current_position = self.dp_rank * self.B * self.T
        self._load_tokens_for_current_shard()
        self._staged = None

    def advance(self):
        self.current_shard = (self.current_shard + 1) % len(self.files)
        self.current_position = self.dp_rank * self.B * self.T
        self._load_tokens_for_current_shard()

    def _take_window(self) -> np.ndarray:
        n = self.B * self.T
        buf = self.tokens[self.current_position:self.current_position + n + 1]
        self.current_position += n * self.dp_world_size
        if self.current_position + (n * self.dp_world_size + 1) > len(self.tokens):
            self.advance()
        return buf

    # -- staging
    def _stage(self):
        """Copy the next window into pinned memory and start its transfer on the side stream."""
        state_before = (self.current_shard, self.current_position)
        buf = self._take_window()
        slot = self._slot
        self._slot ^= 1
        if self._slot_events[slot] is not None:
            self._slot_events[slot].synchronize()  # the copy that last read this pinned buffer is done
        pinned = self._pinned[slot]
        pinned.numpy()[:] = buf  # uint16 -> int64 while copying into the pinned buffer
        with torch.cuda.stream(self._stream):
            dev = pinned.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._slot_events[slot] = ev
        return dev, ev, state_before

    def next_batch(self) -> Tuple[torch.Tensor, torch.Tensor]:
        B, T = self.B, self.T
        if not self._cuda:
            buf = torch.from_numpy(self._take_window().astype(np.int64))
            return buf[:-1].view(B, T), buf[1:].view(B, T)
        if self._staged is None:
            self._staged = self._stage()
        dev, ev, _ = self._staged
        torch.cuda.current_stream(self.device).wait_event(ev)
        dev.record_stream(torch.cuda.current_stream(self.device))
        self._staged = self._stage() if self._prefetch else None
        return dev[:-1].view(B, T), dev[1:].view(B, T)

    @property
    def h2d_bytes_per_batch(self) -> int:
        return (self.B * self.T + 1) * 8

    # -- checkpointing (keys of models/gpt_utils.py:84-104)
    def state_dict(self) -> Dict[str, int]:
        shard, pos = self.current_shard, self.current_position
        if self._staged is not None:  # a prefetched, not yet consumed batch must be replayed after resume
            shard, pos = self._staged[2]
        return {
            f"current_shard_rank_{self.dp_rank}": shard,
            f"current_position_rank_{self.dp_rank}": pos,
            "dataloader_world_size": self.dp_world_size,
        }

    def load_state_dict(self, state_dict: dict):
        world = state_dict.get("dataloader_world_size")
        if world != self.dp_world_size:
            raise NotImplementedError(
                f"DistributedDataLoader does not support redistributing checkpoints to a different world size. "
                f"Current process has world size {self.dp_world_size}, but checkpoint has size {world}.")
        self.current_shard = state_dict[f"current_shard_rank_{self.dp_rank}"]
        self.current_position = state_dict[f"current_position_rank_{self.dp_rank}"]
        self._load_tokens_for_current_shard()
        self._staged = None


class ArithmeticDistributedDataLoader:
    """Loader for one headerless uint16 file ``<data_dir>/<split>.bin``: rank-strided windows
    with circular wrap-around when the file holds at least ``B*T + 1`` tokens, otherwise ``B``
    random windows of length ``T`` (models/gpt_utils.py:107-168)."""

    def __init__(self, data_dir: str, B: int, T: int, rank: int, world_size: int, split: str = "train",
                 device: Optional[torch.device] = None):
        self.B, self.T, self.rank, self.world_size = B, T, rank, world_size
        path = os.path.join(data_dir, f"{split}.bin")
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        self.tokens = np.fromfile(path, dtype=np.uint16).astype(np.int64)
        self.ntok = len(self.tokens)
        self.pos = rank * B * T
        if device is None:
            device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)

    def reset(self):
        self.pos = self.rank * self.B * self.T

    def next_batch(self) -> Tuple[torch.Tensor, torch.Tensor]:
        B, T = self.B, self.T
        need = B * T + 1
        if self.ntok >= need:
            idx = (self.pos + np.arange(need)) % self.ntok
            buf = self.tokens[idx]
            self.pos = (self.pos + self.world_size * B * T) % self.ntok
            x = torch.from_numpy(buf[:-1]).view(B, T)
            y = torch.from_numpy(buf[1:]).view(B, T)
        else:
            max_start = self.ntok - T - 1
            assert max_start > 0, f"split too small: ntok={self.ntok}, need at least T+1={T + 1}"
            starts = np.random.randint(0, max_start + 1, size=B)
            x = torch.from_numpy(np.stack([self.tokens[s:s + T] for s in starts]))
            y = torch.from_numpy(np.stack([self.tokens[s + 1:s + T + 1] for s in starts]))
        return x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
