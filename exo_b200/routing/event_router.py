"""Reliable, ordered event transport between one node's components and the master.

Outbound: every local producer gets its own origin id and a contiguous ``origin_idx`` stream;
an event stays "out for delivery" until the master echoes it in the global stream and is re-sent
if that takes more than 5 s.  Inbound: global events of the current session coming from the
master are re-sequenced; a gap that does not close triggers a NACK — a ``RequestEventLog`` from
the first missing index — with exponential back-off from 0.5 s to 10 s (reference
``src/exo/routing/event_router.py:62-181``).
"""
from __future__ import annotations

import random

import anyio

from ..shared.base import EventId, SessionId, SystemId
from ..shared.events import Event, GlobalForwarderEvent, IndexedEvent, LocalForwarderEvent
from ..shared.messages import ForwarderCommand, RequestEventLog
from ..utils.buffers import OrderedBuffer
from ..utils.channels import ChannelClosed, Receiver, Sender, channel

RESEND_AFTER = 5.0
NACK_BASE, NACK_CAP = 0.5, 10.0


class EventRouter:
    def __init__(self, session_id: SessionId, command_sender: Sender[ForwarderCommand],
                 external_inbound: Receiver[GlobalForwarderEvent], external_outbound: Sender[LocalForwarderEvent],
                 resend_after: float = RESEND_AFTER, nack_base: float = NACK_BASE, nack_cap: float = NACK_CAP):
        self.session_id = session_id
        self.command_sender, self.ext_in, self.ext_out = command_sender, external_inbound, external_outbound
        self.system_id = SystemId()
        self.subscribers: list[Sender[IndexedEvent]] = []
        self.out_for_delivery: dict[EventId, tuple[float, LocalForwarderEvent]] = {}
        self.resend_after, self.nack_base, self.nack_cap = resend_after, nack_base, nack_cap
        self._producers: list[tuple[SystemId, Receiver[Event]]] = []
        self._nack_attempts = 0
        self._nack_scope: anyio.CancelScope | None = None
        self._tg: anyio.abc.TaskGroup | None = None

    # ---- wiring ----
    def sender(self) -> Sender[Event]:
        s, r = channel()
        sid = SystemId()
        if self._tg is None:
            self._producers.append((sid, r))
        else:
            self._tg.start_soon(self._ingest, sid, r)
        return s

    def receiver(self) -> Receiver[IndexedEvent]:
        s, r = channel()
        self.subscribers.append(s)
        return r

    # ---- outbound ----
    async def _ingest(self, origin: SystemId, recv: Receiver[Event]) -> None:
        idx = 0
        async for ev in recv:
            fe = LocalForwarderEvent(origin_idx=idx, origin=origin, session=self.session_id, event=ev)
            idx += 1
            self.out_for_delivery[ev.event_id] = (anyio.current_time(), fe)
            await self.ext_out.send(fe)

    async def _resend_loop(self) -> None:
        while True:
            await anyio.sleep(min(1.0 + random.random(), max(0.05, self.resend_after / 2)))
            now = anyio.current_time()
            for eid, (t, fe) in list(self.out_for_delivery.items()):
                if now > t + self.resend_after:
                    self.out_for_delivery[eid] = (now, fe)
                    await self.ext_out.send(fe)

    # ---- inbound ----
    async def _nack(self, since_idx: int) -> None:
        with anyio.CancelScope() as scope:
            self._nack_scope = scope
            delay = min(self.nack_cap, self.nack_base * (2.0 ** self._nack_attempts))
            self._nack_attempts += 1
            try:
                await anyio.sleep(delay)
                await self.command_sender.send(ForwarderCommand(origin=self.system_id,
                                                                command=RequestEventLog(since_idx=max(0, since_idx))))
            finally:
                if self._nack_scope is scope:
                    self._nack_scope = None

    async def _inbound(self) -> None:
        buf: OrderedBuffer[Event] = OrderedBuffer()
        async for ge in self.ext_in:
            if ge.session != self.session_id or ge.origin != self.session_id.master_node_id:
                continue
            buf.ingest(ge.origin_idx, ge.event)
            self.out_for_delivery.pop(ge.event.event_id, None)
            drained = buf.drain_indexed()
            if drained:
                self._nack_attempts = 0
                if self._nack_scope is not None:
                    self._nack_scope.cancel()
            elif buf.has_gap and self._nack_scope is None:
                assert self._tg is not None
                self._tg.start_soon(self._nack, buf.next_idx)
                continue
            for idx, ev in drained:
                dead = []
                for s in self.subscribers:
                    try:
                        await s.send(IndexedEvent(idx=idx, event=ev))
                    except ChannelClosed:
                        dead.append(s)
                for s in dead:
                    self.subscribers.remove(s)

    async def run(self) -> None:
        try:
            async with anyio.create_task_group() as tg:
                self._tg = tg
                for sid, r in self._producers:
                    tg.start_soon(self._ingest, sid, r)
                self._producers = []
                tg.start_soon(self._inbound)
                tg.start_soon(self._resend_loop)
        except ChannelClosed:
            pass
        finally:
            self._tg = None
            for s in self.subscribers:
                s.close()

    def shutdown(self) -> None:
        if self._tg is not None:
            self._tg.cancel_scope.cancel()
