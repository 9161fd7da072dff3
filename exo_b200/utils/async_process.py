"""Child processes for asyncio code: spawn, pump stdout/stderr, stop with escalation.

``AsyncProcess`` runs a picklable target in a ``spawn``-context child whose stdout/stderr are
pipes the parent reads line by line; ``faulthandler`` is enabled in the child; ``stop()`` sends
SIGTERM repeatedly and then SIGKILL (reference ``src/exo/utils/async_process.py:40-289``:
10 × SIGTERM, then SIGKILL).  ``TaskGroup`` is a small restartable wrapper around
``anyio`` task groups (reference ``src/exo/utils/task_group.py``).
"""
from __future__ import annotations

import faulthandler
import multiprocessing as mp
import os
import signal
import sys
import time
from collections.abc import AsyncIterator, Awaitable, Callable
from typing import Any

import anyio


def _child_main(target: Callable[..., Any], args: tuple, out_conn: Any, err_conn: Any) -> None:
    # the pipe ends arrive as multiprocessing Connections (the only way to hand an fd to a spawned
    # child); from here on they are plain stdout / stderr
    os.dup2(out_conn.fileno(), 1)
    os.dup2(err_conn.fileno(), 2)
    out_conn.close()
    err_conn.close()
    sys.stdout = os.fdopen(1, "w", buffering=1, closefd=False)
    sys.stderr = os.fdopen(2, "w", buffering=1, closefd=False)
    faulthandler.enable(file=sys.stderr, all_threads=True)
    target(*args)


class AsyncProcess:
    TERM_ATTEMPTS = 10
    TERM_INTERVAL = 0.3

    def __init__(self, target: Callable[..., Any], args: tuple = (), name: str | None = None, daemon: bool = True):
        self.ctx = mp.get_context("spawn")
        out_r, out_w = self.ctx.Pipe(duplex=False)
        err_r, err_w = self.ctx.Pipe(duplex=False)
        self._out_r, self._err_r = os.dup(out_r.fileno()), os.dup(err_r.fileno())
        out_r.close()
        err_r.close()
        self.proc = self.ctx.Process(target=_child_main, args=(target, args, out_w, err_w), name=name, daemon=daemon)
        self._w = (out_w, err_w)
        self.started = False

    def start(self) -> None:
        self.proc.start()
        for c in self._w:
            c.close()
        self.started = True

    @property
    def pid(self) -> int | None:
        return self.proc.pid

    def is_alive(self) -> bool:
        return self.proc.is_alive()

    @property
    def exitcode(self) -> int | None:
        return self.proc.exitcode

    async def _lines(self, fd: int) -> AsyncIterator[str]:
        f = os.fdopen(fd, "rb", buffering=0, closefd=True)
        buf = b""
        try:
            while True:
                chunk = await anyio.to_thread.run_sync(f.read, 65536, abandon_on_cancel=True)
                if not chunk:
                    break
                buf += chunk
                *lines, buf = buf.split(b"\n")
                for ln in lines:
                    yield ln.decode("utf-8", "replace")
            if buf:
                yield buf.decode("utf-8", "replace")
        finally:
            try:
                f.close()
            except OSError:
                pass

    def stdout_lines(self) -> AsyncIterator[str]:
        return self._lines(self._out_r)

    def stderr_lines(self) -> AsyncIterator[str]:
        return self._lines(self._err_r)

    async def wait(self, poll: float = 0.05) -> int | None:
        while self.proc.is_alive():
            await anyio.sleep(poll)
        self.proc.join(timeout=0)
        return self.proc.exitcode

    async def stop(self) -> int | None:
        """SIGTERM up to ``TERM_ATTEMPTS`` times, then SIGKILL.  Returns the exit code."""
        if not self.started:
            return None
        for _ in range(self.TERM_ATTEMPTS):
            if not self.proc.is_alive():
                break
            try:
                os.kill(self.proc.pid, signal.SIGTERM)  # type: ignore[arg-type]
            except ProcessLookupError:
                break
            deadline = time.monotonic() + self.TERM_INTERVAL
            while self.proc.is_alive() and time.monotonic() < deadline:
                await anyio.sleep(0.02)
        if self.proc.is_alive():
            try:
                os.kill(self.proc.pid, signal.SIGKILL)  # type: ignore[arg-type]
            except ProcessLookupError:
                pass
            while self.proc.is_alive():
                await anyio.sleep(0.02)
        self.proc.join(timeout=1)
        return self.proc.exitcode


class TaskGroup:
    """An anyio task group that can be entered, cancelled and entered again."""

    def __init__(self) -> None:
        self._tg: anyio.abc.TaskGroup | None = None
        self._cm: Any = None

    async def __aenter__(self) -> "TaskGroup":
        self._cm = anyio.create_task_group()
        self._tg = await self._cm.__aenter__()
        return self

    async def __aexit__(self, *exc: Any) -> bool | None:
        try:   # children may keep spawning siblings while the group waits for them
            return await self._cm.__aexit__(*exc)
        finally:
            self._cm, self._tg = None, None

    def start_soon(self, fn: Callable[..., Awaitable[Any]], *args: Any) -> None:
        assert self._tg is not None, "task group is not running"
        self._tg.start_soon(fn, *args)

    def cancel_tasks(self) -> None:
        if self._tg is not None:
            self._tg.cancel_scope.cancel()

    @property
    def running(self) -> bool:
        return self._tg is not None
