"""Typed channels: in-process (anyio memory streams with cloneable ends) and cross-process
(``multiprocessing`` queues with an end-of-stream sentinel).

Same roles as the reference's ``src/exo/utils/channels.py:110-424`` (``channel()``, ``Sender.clone``,
``Receiver.collect``, ``mp_channel()``, closed-channel errors) — the control plane is built on
them: every component owns the receiving end of its inbox and hands out cloned senders.
"""
from __future__ import annotations

import multiprocessing as mp
import queue
from math import inf
from typing import Any, Generic, TypeVar

import anyio
from anyio import BrokenResourceError, ClosedResourceError, EndOfStream, WouldBlock
from anyio.streams.memory import MemoryObjectReceiveStream, MemoryObjectSendStream

T = TypeVar("T")


class ChannelClosed(Exception):
    pass


class Sender(Generic[T]):
    def __init__(self, stream: MemoryObjectSendStream[T]):
        self._s = stream

    async def send(self, item: T) -> None:
        try:
            await self._s.send(item)
        except (BrokenResourceError, ClosedResourceError) as e:
            raise ChannelClosed("receiver is gone") from e

    def send_nowait(self, item: T) -> None:
        try:
            self._s.send_nowait(item)
        except (BrokenResourceError, ClosedResourceError) as e:
            raise ChannelClosed("receiver is gone") from e

    def clone(self) -> "Sender[T]":
        return Sender(self._s.clone())

    def close(self) -> None:
        self._s.close()

    def __enter__(self) -> "Sender[T]":
        return self

    def __exit__(self, *a: Any) -> None:
        self.close()


class Receiver(Generic[T]):
    def __init__(self, stream: MemoryObjectReceiveStream[T]):
        self._r = stream

    async def receive(self) -> T:
        try:
            return await self._r.receive()
        except (EndOfStream, ClosedResourceError) as e:
            raise ChannelClosed("all senders are gone") from e

    def receive_nowait(self) -> T:
        try:
            return self._r.receive_nowait()
        except (EndOfStream, ClosedResourceError) as e:
            raise ChannelClosed("all senders are gone") from e

    def collect(self) -> list[T]:
        """Everything that is queued right now, without waiting."""
        out: list[T] = []
        while True:
            try:
                out.append(self._r.receive_nowait())
            except (WouldBlock, EndOfStream, ClosedResourceError):
                return out

    async def receive_at_least(self, n: int) -> list[T]:
        out = self.collect()
        while len(out) < n:
            out.append(await self.receive())
            out.extend(self.collect())
        return out

    def clone(self) -> "Receiver[T]":
        return Receiver(self._r.clone())

    def close(self) -> None:
        self._r.close()

    def __aiter__(self) -> "Receiver[T]":
        return self

    async def __anext__(self) -> T:
        try:
            return await self.receive()
        except ChannelClosed:
            raise StopAsyncIteration from None

    def __enter__(self) -> "Receiver[T]":
        return self

    def __exit__(self, *a: Any) -> None:
        self.close()


def channel(max_buffer_size: float = inf) -> tuple[Sender[Any], Receiver[Any]]:
    s, r = anyio.create_memory_object_stream(max_buffer_size)
    return Sender(s), Receiver(r)


# ------------------------------------------------------------------------------------------------
# cross-process
# ------------------------------------------------------------------------------------------------
class _Eos:
    """End-of-stream marker (pickles to itself)."""

    def __reduce__(self):
        return (_Eos, ())


class MpSender(Generic[T]):
    def __init__(self, q: "mp.Queue[Any]"):
        self._q = q
        self._closed = False

    def send(self, item: T) -> None:
        if self._closed:
            raise ChannelClosed("sender closed")
        self._q.put(item)

    async def send_async(self, item: T) -> None:
        await anyio.to_thread.run_sync(self.send, item)

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            try:
                self._q.put(_Eos())
            except (ValueError, OSError):
                pass

    def join(self) -> None:
        self._q.close()
        self._q.join_thread()


class MpReceiver(Generic[T]):
    def __init__(self, q: "mp.Queue[Any]"):
        self._q = q
        self._done = False

    def receive(self, timeout: float | None = None) -> T:
        if self._done:
            raise ChannelClosed("stream ended")
        try:
            item = self._q.get(timeout=timeout)
        except queue.Empty:
            raise TimeoutError from None
        if isinstance(item, _Eos):
            self._done = True
            raise ChannelClosed("stream ended")
        return item

    def receive_nowait(self) -> T:
        if self._done:
            raise ChannelClosed("stream ended")
        try:
            item = self._q.get_nowait()
        except queue.Empty:
            raise WouldBlock from None
        if isinstance(item, _Eos):
            self._done = True
            raise ChannelClosed("stream ended")
        return item

    def collect(self) -> list[T]:
        out: list[T] = []
        while True:
            try:
                out.append(self.receive_nowait())
            except (WouldBlock, ChannelClosed):
                return out

    async def receive_async(self, poll: float = 0.2) -> T:
        """Awaitable receive that stays cancellable (polls a worker thread with a short timeout)."""
        while True:
            try:
                return await anyio.to_thread.run_sync(self.receive, poll, abandon_on_cancel=True)
            except TimeoutError:
                continue

    def close(self) -> None:
        self._done = True


def mp_channel(ctx: Any = None, maxsize: int = 0) -> tuple[MpSender[Any], MpReceiver[Any]]:
    q = (ctx or mp.get_context("spawn")).Queue(maxsize)
    return MpSender(q), MpReceiver(q)
