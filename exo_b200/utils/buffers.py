"""Re-sequencing buffers, keyed back-off and the append-only disk event log.

* ``OrderedBuffer`` / ``MultiSourceBuffer`` — hold out-of-order indexed items until the gap closes
  (reference ``src/exo/utils/event_buffer.py:4-70``; a duplicate index must carry an equal item).
* ``KeyedBackoff`` — per-key exponential back-off, 0.5 s doubling to 10 s by default
  (reference ``src/exo/utils/keyed_backoff.py``).
* ``DiskEventLog`` — length-prefixed msgpack records, sparse offset index for ``read_range``,
  rotation of the previous log to a compressed archive keeping the 5 newest
  (reference ``src/exo/utils/disk_event_log.py:62-187``; gzip stands in for zstd, which is not
  available in this environment).
"""
from __future__ import annotations

import gzip
import os
import shutil
import struct
import time
from collections.abc import Hashable, Iterator
from pathlib import Path
from typing import Any, Generic, TypeVar

import msgpack

T = TypeVar("T")
K = TypeVar("K", bound=Hashable)


class OrderedBuffer(Generic[T]):
    def __init__(self, start: int = 0) -> None:
        self.next_idx = start
        self.store: dict[int, T] = {}

    def ingest(self, idx: int, item: T) -> None:
        if idx < self.next_idx:
            return
        if idx in self.store:
            assert self.store[idx] == item, f"conflicting items for index {idx}"
            return
        self.store[idx] = item

    def drain(self) -> list[T]:
        out: list[T] = []
        while self.next_idx in self.store:
            out.append(self.store.pop(self.next_idx))
            self.next_idx += 1
        return out

    def drain_indexed(self) -> list[tuple[int, T]]:
        out: list[tuple[int, T]] = []
        while self.next_idx in self.store:
            out.append((self.next_idx, self.store.pop(self.next_idx)))
            self.next_idx += 1
        return out

    @property
    def has_gap(self) -> bool:
        return bool(self.store) and self.next_idx not in self.store


class MultiSourceBuffer(Generic[K, T]):
    """One ``OrderedBuffer`` per source; ``drain`` returns what became contiguous, source by source."""

    def __init__(self) -> None:
        self.buffers: dict[K, OrderedBuffer[T]] = {}

    def ingest(self, idx: int, item: T, source: K) -> None:
        self.buffers.setdefault(source, OrderedBuffer()).ingest(idx, item)

    def drain(self) -> list[T]:
        out: list[T] = []
        for b in self.buffers.values():
            out.extend(b.drain())
        return out


class KeyedBackoff(Generic[K]):
    def __init__(self, base: float = 0.5, cap: float = 10.0) -> None:
        self.base, self.cap = base, cap
        self.attempts: dict[K, int] = {}
        self.not_before: dict[K, float] = {}

    def should_proceed(self, key: K) -> bool:
        return time.monotonic() >= self.not_before.get(key, 0.0)

    def record_attempt(self, key: K) -> int:
        n = self.attempts.get(key, 0)
        self.attempts[key] = n + 1
        self.not_before[key] = time.monotonic() + min(self.cap, self.base * (2 ** n))
        return n + 1

    def attempts_for(self, key: K) -> int:
        return self.attempts.get(key, 0)

    def reset(self, key: K) -> None:
        self.attempts.pop(key, None)
        self.not_before.pop(key, None)


class DiskEventLog:
    """Append-only log of msgpack-able records with O(1) amortised range reads."""
    ARCHIVES = 5
    INDEX_EVERY = 256

    def __init__(self, directory: str | Path, name: str = "events.bin") -> None:
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.path = self.dir / name
        self.rotate()
        self.f = open(self.path, "ab+")
        self.count = 0
        self.offsets: list[int] = []  # byte offset of every INDEX_EVERY-th record

    def rotate(self) -> None:
        """Move a non-empty previous log into a compressed archive, keep the newest ``ARCHIVES``."""
        if self.path.exists() and self.path.stat().st_size > 0:
            dst = self.dir / f"{self.path.stem}.{int(time.time() * 1000)}.bin.gz"
            with open(self.path, "rb") as src, gzip.open(dst, "wb", compresslevel=3) as out:
                shutil.copyfileobj(src, out)
            self.path.unlink()
        old = sorted(self.dir.glob(f"{self.path.stem}.*.bin.gz"))
        for p in old[:-self.ARCHIVES] if len(old) > self.ARCHIVES else []:
            p.unlink(missing_ok=True)

    def append(self, record: Any) -> int:
        blob = msgpack.packb(record, use_bin_type=True)
        if self.count % self.INDEX_EVERY == 0:
            self.f.seek(0, os.SEEK_END)
            self.offsets.append(self.f.tell())
        self.f.write(struct.pack("<I", len(blob)))
        self.f.write(blob)
        self.count += 1
        return self.count - 1

    def flush(self) -> None:
        self.f.flush()

    def read_range(self, start: int, end: int | None = None) -> Iterator[Any]:
        """Records ``[start, end)`` (``end`` defaults to the current count)."""
        end = self.count if end is None else min(end, self.count)
        if start >= end:
            return
        self.f.flush()
        slot = start // self.INDEX_EVERY
        with open(self.path, "rb") as r:
            r.seek(self.offsets[slot])
            i = slot * self.INDEX_EVERY
            while i < end:
                hdr = r.read(4)
                if len(hdr) < 4:
                    return
                (n,) = struct.unpack("<I", hdr)
                blob = r.read(n)
                if i >= start:
                    yield msgpack.unpackb(blob, raw=False)
                i += 1

    def read_all(self) -> list[Any]:
        return list(self.read_range(0))

    def __len__(self) -> int:
        return self.count

    def close(self) -> None:
        try:
            self.f.flush()
            self.f.close()
        except ValueError:
            pass
