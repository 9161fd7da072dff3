"""asyncio transport over the native bus (`_exo_native.Bus`) for ``exo_b200.routing.router``.

The C++ side queues events and signals an eventfd; here the running loop watches that fd, so
``recv()`` is a plain await.  Publishing hands the frame to a worker thread because the native
call blocks until every subscribed peer has taken it (back-pressure), with the GIL released.
"""
from __future__ import annotations

import asyncio
from typing import Any

import anyio

from ..utils.channels import ChannelClosed


def load_native():
    from . import _exo_native  # built by exo_b200.build
    return _exo_native


class NativeTransport:
    def __init__(self, identity: str, namespace: str, listen_port: int = 0, discovery_port: int = 0):
        self.native = load_native()
        self.bus = self.native.Bus(identity, namespace, listen_port, discovery_port)
        self._closed = False
        self._ready: asyncio.Event | None = None
        self._loop: asyncio.AbstractEventLoop | None = None

    @property
    def listen_port(self) -> int:
        return self.bus.listen_port

    def connect(self, host: str, port: int) -> bool:
        return self.bus.connect(host, port)

    def _arm(self) -> None:
        if self._loop is None:
            self._loop = asyncio.get_running_loop()
            self._ready = asyncio.Event()
            self._loop.add_reader(self.bus.event_fd, self._ready.set)

    async def recv(self) -> tuple[str, Any]:
        self._arm()
        assert self._ready is not None
        while True:
            if self._closed:
                raise ChannelClosed("bus closed")
            ev = self.bus.try_recv()
            if ev is not None:
                if ev[0] == "message":
                    return "message", (ev[1], ev[2])
                if ev[0] == "connection":
                    return "connection", (ev[1], ev[2])
                return "discovered", (ev[1], ev[2])
            self._ready.clear()
            if self.bus.try_recv is None:  # pragma: no cover
                continue
            await self._ready.wait()

    async def publish(self, topic: str, data: bytes) -> None:
        await anyio.to_thread.run_sync(self.bus.publish, topic, bytes(data))

    async def subscribe(self, topic: str) -> None:
        self.bus.subscribe(topic)

    async def unsubscribe(self, topic: str) -> None:
        self.bus.unsubscribe(topic)

    def peers(self) -> list[str]:
        return list(self.bus.peers())

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        if self._loop is not None:
            try:
                self._loop.remove_reader(self.bus.event_fd)
            except (RuntimeError, ValueError):
                pass
            if self._ready is not None:
                self._loop.call_soon_threadsafe(self._ready.set)
        self.bus.close()
