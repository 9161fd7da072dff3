"""Span tracing for runner ranks and Chrome-trace export.

``with trace("recv 0", rank, "comms"):`` records ``(name, start_us, duration_us, rank, category)``
in a per-process buffer; nested spans compose their categories (``sync/compute``); nothing is
recorded unless ``EXO_TRACING_ENABLED=true`` (reference ``src/exo/shared/tracing.py:79-119``).
When ``cuda=True`` the span is timed with CUDA events on the current stream instead of the host
clock, so asynchronous kernels are attributed to the span that launched them.  Buffers are shipped
to the master as ``TracesCollected`` events, merged, and written as Chrome-trace JSON
(reference ``tracing.py:130-238``); ``compute_stats`` feeds ``/v1/traces/{task}/stats``.
"""
from __future__ import annotations

import json
import time
from collections.abc import Generator, Iterable
from contextlib import contextmanager
from contextvars import ContextVar
from dataclasses import dataclass, field
from pathlib import Path

from . import constants

_category: ContextVar[str | None] = ContextVar("exo_trace_category", default=None)


@dataclass(frozen=True)
class TraceEvent:
    name: str
    start_us: int
    duration_us: int
    rank: int
    category: str


@dataclass
class CategoryStats:
    total_us: int = 0
    count: int = 0
    min_us: int = 0
    max_us: int = 0

    def add(self, d: int) -> None:
        self.min_us = d if self.count == 0 else min(self.min_us, d)
        self.max_us = d if self.count == 0 else max(self.max_us, d)
        self.total_us += d
        self.count += 1

    @property
    def avg_us(self) -> float:
        return self.total_us / self.count if self.count else 0.0


@dataclass
class TraceStats:
    total_wall_time_us: int = 0
    by_category: dict[str, CategoryStats] = field(default_factory=dict)
    by_rank: dict[int, dict[str, CategoryStats]] = field(default_factory=dict)


_buffer: list[TraceEvent] = []
_pending_cuda: list[tuple[str, int, int, str, object, object]] = []
enabled = constants.EXO_TRACING_ENABLED


def set_enabled(on: bool) -> None:
    global enabled
    enabled = on


@contextmanager
def trace(name: str, rank: int, category: str = "compute", cuda: bool = False) -> Generator[None, None, None]:
    if not enabled:
        yield
        return
    parent = _category.get()
    full = f"{parent}/{category}" if parent else category
    token = _category.set(full)
    start_us = int(time.time() * 1_000_000)
    t0 = time.perf_counter()
    ev0 = ev1 = None
    if cuda:
        import torch
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push(name)
        ev0.record()
    try:
        yield
    finally:
        _category.reset(token)
        if cuda:
            import torch
            ev1.record()
            torch.cuda.nvtx.range_pop()
            _pending_cuda.append((name, start_us, rank, full, ev0, ev1))
        else:
            _buffer.append(TraceEvent(name, start_us, int((time.perf_counter() - t0) * 1_000_000), rank, full))


def _resolve_cuda() -> None:
    """Turn finished CUDA-event pairs into spans (called when the buffer is read)."""
    if not _pending_cuda:
        return
    import torch
    torch.cuda.synchronize()
    for name, start_us, rank, cat, e0, e1 in _pending_cuda:
        _buffer.append(TraceEvent(name, start_us, int(e0.elapsed_time(e1) * 1000), rank, cat))
    _pending_cuda.clear()


def get_trace_buffer() -> list[TraceEvent]:
    _resolve_cuda()
    return list(_buffer)


def clear_trace_buffer() -> None:
    _buffer.clear()
    _pending_cuda.clear()


def to_chrome_trace(events: Iterable[TraceEvent]) -> dict:
    out = []
    for e in events:
        out.append({"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.duration_us,
                    "pid": 0, "tid": e.rank, "args": {"rank": e.rank}})
    return {"traceEvents": out, "displayTimeUnit": "ms"}


def export_trace(events: Iterable[TraceEvent], path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(to_chrome_trace(events)))


def load_trace_file(path: Path) -> list[TraceEvent]:
    raw = json.loads(path.read_text())
    return [TraceEvent(e["name"], int(e["ts"]), int(e["dur"]), int(e.get("tid", 0)), e.get("cat", ""))
            for e in raw.get("traceEvents", []) if e.get("ph") == "X"]


def compute_stats(events: Iterable[TraceEvent]) -> TraceStats:
    evs = list(events)
    st = TraceStats()
    if not evs:
        return st
    st.total_wall_time_us = max(e.start_us + e.duration_us for e in evs) - min(e.start_us for e in evs)
    for e in evs:
        st.by_category.setdefault(e.category, CategoryStats()).add(e.duration_us)
        st.by_rank.setdefault(e.rank, {}).setdefault(e.category, CategoryStats()).add(e.duration_us)
    return st
