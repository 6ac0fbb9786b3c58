"""Token data: ArrayRecord shards (+ ``.lengths.npy`` sidecars) or a ``.npy`` token file, read as fixed
``(batch, seq)`` blocks with a one-token overlap for labels (lyra/data.py:30-115).

Reading, record indexing and prefetch run in the native runtime (``csrc/io``): each block is filled by a
worker thread straight into a pinned host buffer, so the training loop's host-to-device copy is a
single asynchronous transfer. Block order comes from ``IndexSampler`` (sequential or a seeded
per-epoch shuffle, rank-strided like Grain's ``ShardOptions(drop_remainder=True)``) whose position is
the loader state stored in checkpoints.
"""

from __future__ import annotations

import ctypes
import json
import os
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from lyra_b200.ops import native

TOKEN_DTYPE = np.dtype("<i4")
LENGTHS_SUFFIX = ".lengths.npy"


@dataclass(frozen=True, kw_only=True)
class DataLoaderConfig:
    shuffle: bool = False
    seed: int = 42
    num_epochs: int | None = 1
    worker_count: int = 2


# --------------------------------------------------------------------------- shard writer
class ArrayRecordWriter:
    """One record per ``write`` call (``group_size:1``)."""

    def __init__(self, path: str | os.PathLike, group_size: int = 1):
        lib = native.io()
        lib.lyra_ar_writer_open.restype = ctypes.c_void_p
        self._lib = lib
        self._h = lib.lyra_ar_writer_open(str(path).encode(), group_size)
        if not self._h:
            raise OSError(f"cannot open {path} for writing")

    def write(self, data: bytes) -> None:
        if self._lib.lyra_ar_writer_write(ctypes.c_void_p(self._h), data, ctypes.c_longlong(len(data))) != 0:
            raise OSError("ArrayRecord write failed")

    def close(self) -> None:
        if self._h:
            rc = self._lib.lyra_ar_writer_close(ctypes.c_void_p(self._h))
            self._h = None
            if rc != 0:
                raise OSError("ArrayRecord close failed")


class ShardWriter:
    """Writes one record per document, starting a new shard every ``tokens_per_shard`` tokens, and a
    ``<shard>.lengths.npy`` int64 sidecar with the record lengths (data/prepare_climbmix.py:34-63)."""

    def __init__(self, directory: Path, tokens_per_shard: int) -> None:
        self.directory = Path(directory)
        self.tokens_per_shard = tokens_per_shard
        self.index = 0
        self.writer: ArrayRecordWriter | None = None
        self.lengths: list[int] = []
        self.count = 0

    def write(self, tokens: list[int]) -> None:
        while tokens:
            if self.writer is None:
                self.path = self.directory / f"shard-{self.index:05d}.array_record"
                self.writer = ArrayRecordWriter(self.path, 1)
            room = self.tokens_per_shard - self.count
            chunk, tokens = tokens[:room], tokens[room:]
            self.writer.write(np.asarray(chunk, dtype=TOKEN_DTYPE).tobytes())
            self.lengths.append(len(chunk))
            self.count += len(chunk)
            if self.count == self.tokens_per_shard:
                self.close()

    def close(self) -> None:
        if self.writer is None:
            return
        self.writer.close()
        np.save(str(self.path) + LENGTHS_SUFFIX, np.asarray(self.lengths, dtype=np.int64))
        print(f"Wrote {self.path} ({self.count:,} tokens)", flush=True)
        self.index, self.writer, self.lengths, self.count = self.index + 1, None, [], 0


# --------------------------------------------------------------------------- block source
class TokenBlocks:
    """Random access to ``(batch, seq)`` blocks of a token stream."""

    def __init__(self, path: Path, batch_size: int, seq_len: int):
        self.path = Path(path)
        self.shape = (batch_size, seq_len)
        self.size = batch_size * seq_len
        lib = native.io()
        lib.lyra_tokens_open.restype = ctypes.c_void_p
        lib.lyra_tokens_open_raw.restype = ctypes.c_void_p
        lib.lyra_tokens_count.restype = ctypes.c_longlong
        self._lib = lib
        if self.path.suffix == ".npy":
            arr = np.load(self.path, mmap_mode="r")
            if arr.dtype != TOKEN_DTYPE or arr.ndim != 1:
                raise ValueError(f"{self.path}: expected a 1-D int32 token array, found {arr.dtype} {arr.shape}")
            self._src = lib.lyra_tokens_open_raw(str(self.path).encode(), ctypes.c_longlong(arr.offset), ctypes.c_longlong(arr.shape[0]))
        else:
            shards = sorted(str(s) for s in self.path.glob("*.array_record")) if self.path.is_dir() else [str(self.path)]
            if not shards:
                raise FileNotFoundError(f"no *.array_record shards in {self.path}")
            arr_t = (ctypes.c_char_p * len(shards))(*[s.encode() for s in shards])
            self._src = lib.lyra_tokens_open(len(shards), arr_t)
            if self._src:
                sidecar = sum(int(np.load(s + LENGTHS_SUFFIX).sum()) for s in shards if os.path.exists(s + LENGTHS_SUFFIX))
                total = lib.lyra_tokens_count(ctypes.c_void_p(self._src))
                if sidecar and sidecar != total:
                    raise ValueError(f"{self.path}: lengths sidecars give {sidecar:,} tokens, records hold {total:,}")
        if not self._src:
            raise OSError(f"cannot open token source {self.path}")
        self.token_count = int(lib.lyra_tokens_count(ctypes.c_void_p(self._src)))

    def __len__(self) -> int:
        return (self.token_count - 1) // self.size

    def __repr__(self) -> str:
        return f"TokenBlocks({self.path}, shape={self.shape})"

    def read(self, start: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=TOKEN_DTYPE)
        rc = self._lib.lyra_tokens_read(ctypes.c_void_p(self._src), ctypes.c_longlong(start), ctypes.c_longlong(count),
                                        out.ctypes.data_as(ctypes.c_void_p))
        if rc != 0:
            raise IndexError(f"token range [{start}, {start + count}) out of bounds or unreadable")
        return out

    def __getitem__(self, index: int) -> dict[str, np.ndarray]:
        tokens = self.read(index * self.size, self.size + 1)
        return {"input_ids": tokens[:-1].reshape(self.shape), "labels": tokens[1:].reshape(self.shape)}


# --------------------------------------------------------------------------- sampler
class IndexSampler:
    """Deterministic block order with a serialisable position. Rank ``r`` of ``n`` takes positions ``r, r+n, ...``
    of each epoch's (optionally shuffled) order; the remainder of an epoch that does not divide is dropped."""

    def __init__(self, num_records: int, *, shuffle: bool, seed: int, num_epochs: int | None, shard_index: int = 0, shard_count: int = 1):
        self.num_records = num_records
        self.shuffle, self.seed, self.num_epochs = shuffle, seed, num_epochs
        self.shard_index, self.shard_count = shard_index, shard_count
        self.per_epoch = num_records // shard_count
        self.position = 0  # number of indices already handed out on this rank
        self._epoch_cache: tuple[int, np.ndarray] | None = None

    def _order(self, epoch: int) -> np.ndarray:
        if self._epoch_cache is None or self._epoch_cache[0] != epoch:
            if self.shuffle:
                order = np.random.Generator(np.random.Philox(key=self.seed + epoch)).permutation(self.num_records)
            else:
                order = np.arange(self.num_records)
            self._epoch_cache = (epoch, order)
        return self._epoch_cache[1]

    def index_at(self, position: int) -> int | None:
        if self.per_epoch == 0:
            return None
        epoch, within = divmod(position, self.per_epoch)
        if self.num_epochs is not None and epoch >= self.num_epochs:
            return None
        return int(self._order(epoch)[within * self.shard_count + self.shard_index])


# --------------------------------------------------------------------------- loader
class DataLoader:
    def __init__(self, path, batch_size: int, seq_len: int, *, config: DataLoaderConfig, shard_index: int = 0, shard_count: int = 1,
                 pin_memory: bool | None = None, quiet: bool = False):
        source = TokenBlocks(Path(path), batch_size, seq_len)
        self.source = source
        self.config = config
        self.token_count = source.token_count
        self.block_count = len(source)
        if not quiet:
            print(f"Loaded {self.token_count:,} tokens from {path} ({self.block_count:,} blocks of {batch_size} x {seq_len})")
        self.sampler = IndexSampler(self.block_count, shuffle=config.shuffle, seed=config.seed, num_epochs=config.num_epochs,
                                    shard_index=shard_index, shard_count=shard_count)
        lib = source._lib
        lib.lyra_loader_create.restype = ctypes.c_void_p
        self._lib = lib
        self._loader = lib.lyra_loader_create(ctypes.c_void_p(source._src), ctypes.c_longlong(source.size), max(config.worker_count, 1))
        self._depth = 4
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        self._buffers = [torch.empty(source.size + 1, dtype=torch.int32, pin_memory=pin) for _ in range(self._depth + 2)]
        self._free = list(range(len(self._buffers)))
        self._inflight: list[tuple[int, int]] = []  # (ticket, buffer index)
        self._submitted = 0  # sampler position of the next block to submit

    # -- state ------------------------------------------------------------------------------
    def get_state(self) -> bytes:
        return json.dumps({"position": self.sampler.position, "seed": self.config.seed, "shuffle": self.config.shuffle}).encode()

    def set_state(self, state: bytes) -> None:
        self._drain()
        self.sampler.position = int(json.loads(state.decode())["position"])
        self._submitted = self.sampler.position

    def check_steps(self, steps: int, accumulation_steps: int) -> None:
        needed = steps * accumulation_steps
        if self.config.num_epochs is not None and needed > self.sampler.per_epoch * self.config.num_epochs:
            raise ValueError(
                f"{steps:,} steps need {needed:,} blocks, but {self.token_count:,} tokens give {self.block_count:,} per epoch. "
                "Download more data or train for fewer steps."
            )

    # -- iteration --------------------------------------------------------------------------
    def _drain(self) -> None:
        for ticket, buf in self._inflight:
            self._lib.lyra_loader_wait(ctypes.c_void_p(self._loader), ticket)
            self._free.append(buf)
        self._inflight.clear()

    def _fill(self) -> None:
        while len(self._inflight) < self._depth and len(self._free) > 1:
            index = self.sampler.index_at(self._submitted)
            if index is None:
                return
            buf = self._free.pop(0)
            ticket = self._lib.lyra_loader_submit(ctypes.c_void_p(self._loader), ctypes.c_longlong(index),
                                                  ctypes.c_void_p(self._buffers[buf].data_ptr()))
            self._inflight.append((ticket, buf))
            self._submitted += 1

    def __iter__(self):
        return self

    def next_pinned(self) -> torch.Tensor:
        """Next block as a pinned int32 tensor of ``B*T + 1`` tokens. The buffer is reused after a few calls."""
        if self._submitted < self.sampler.position:
            self._submitted = self.sampler.position
        self._fill()
        if not self._inflight:
            raise StopIteration
        ticket, buf = self._inflight.pop(0)
        if self._lib.lyra_loader_wait(ctypes.c_void_p(self._loader), ticket) != 0:
            raise OSError("token block read failed")
        self.sampler.position += 1
        self._free.append(buf)
        self._fill()
        return self._buffers[buf]

    def __next__(self) -> tuple[np.ndarray, np.ndarray]:
        tokens = self.next_pinned().numpy().copy()
        shape = self.source.shape
        return tokens[:-1].reshape(shape), tokens[1:].reshape(shape)

    def close(self) -> None:
        if getattr(self, "_loader", None):
            self._drain()
            self._lib.lyra_loader_destroy(ctypes.c_void_p(self._loader))
            self._loader = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
