"""Typed pub/sub between the components of a node and between nodes.

A ``Router`` owns a set of typed topics.  Publishing on a topic fans out to local subscribers and,
depending on the topic's policy, to the network transport; inbound network frames are decoded
with the topic's model and fanned out locally.  Peer appearance/disappearance reported by the
transport is republished on the local-only ``connection_messages`` topic (reference
``src/exo/routing/router.py:34-240`` and ``topics.py:40-51``: six topics, JSON payloads,
``Always``/``Never`` publish policies, a warning above 1 MiB per message).

Transports: ``LoopbackHub`` joins several routers inside one process (tests, single-controller
deployments); ``exo_b200.native.bus`` is the C++ socket bus for separate processes.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Generic, Protocol, TypeVar

import anyio
from pydantic import TypeAdapter

from ..shared import constants
from ..shared.base import NodeId
from ..shared.election import ConnectionMessage, ElectionMessage
from ..shared.events import GlobalForwarderEvent, LocalForwarderEvent
from ..shared.messages import ForwarderCommand, ForwarderDownloadCommand
from ..utils.channels import ChannelClosed, Receiver, Sender, channel

log = logging.getLogger("exo.router")
T = TypeVar("T")


class PublishPolicy(str, Enum):
    Never = "Never"      # local subscribers only
    Always = "Always"    # local subscribers and the network


@dataclass(frozen=True)
class TypedTopic(Generic[T]):
    name: str
    model: Any
    policy: PublishPolicy = PublishPolicy.Always

    def adapter(self) -> TypeAdapter:
        return TypeAdapter(self.model)


GLOBAL_EVENTS = TypedTopic(constants.TOPIC_GLOBAL_EVENTS, GlobalForwarderEvent)
LOCAL_EVENTS = TypedTopic(constants.TOPIC_LOCAL_EVENTS, LocalForwarderEvent)
COMMANDS = TypedTopic(constants.TOPIC_COMMANDS, ForwarderCommand)
ELECTION_MESSAGES = TypedTopic(constants.TOPIC_ELECTION, ElectionMessage)
DOWNLOAD_COMMANDS = TypedTopic(constants.TOPIC_DOWNLOAD_COMMANDS, ForwarderDownloadCommand)
CONNECTION_MESSAGES = TypedTopic(constants.TOPIC_CONNECTIONS, ConnectionMessage, PublishPolicy.Never)
ALL_TOPICS = (GLOBAL_EVENTS, LOCAL_EVENTS, COMMANDS, ELECTION_MESSAGES, DOWNLOAD_COMMANDS, CONNECTION_MESSAGES)


class Transport(Protocol):
    """What a router needs from the network."""

    async def publish(self, topic: str, data: bytes) -> None: ...
    async def recv(self) -> tuple[str, Any]: ...   # ("message", (topic, data)) | ("connection", (peer, up))
    async def subscribe(self, topic: str) -> None: ...
    def close(self) -> None: ...


class LoopbackHub:
    """Joins routers of one process: a published frame reaches every *other* attached router."""

    def __init__(self) -> None:
        self.ports: dict[NodeId, "LoopbackPort"] = {}

    def attach(self, node_id: NodeId) -> "LoopbackPort":
        port = LoopbackPort(self, node_id)
        for other in self.ports.values():
            other._inbox_s.send_nowait(("connection", (node_id, True)))
            port._inbox_s.send_nowait(("connection", (other.node_id, True)))
        self.ports[node_id] = port
        return port

    def detach(self, node_id: NodeId) -> None:
        if self.ports.pop(node_id, None) is not None:
            for other in self.ports.values():
                other._inbox_s.send_nowait(("connection", (node_id, False)))


class LoopbackPort:
    def __init__(self, hub: LoopbackHub, node_id: NodeId):
        self.hub, self.node_id = hub, node_id
        self._inbox_s, self._inbox_r = channel()
        self.topics: set[str] = set()
        self.drop: Any = None   # test hook: callable(topic, data) -> True to lose the frame

    async def publish(self, topic: str, data: bytes) -> None:
        for nid, port in list(self.hub.ports.items()):
            if nid != self.node_id and topic in port.topics:
                if port.drop is not None and port.drop(topic, data):
                    continue
                port._inbox_s.send_nowait(("message", (topic, data)))

    async def recv(self) -> tuple[str, Any]:
        return await self._inbox_r.receive()

    async def subscribe(self, topic: str) -> None:
        self.topics.add(topic)

    def close(self) -> None:
        self.hub.detach(self.node_id)


class TopicRouter(Generic[T]):
    def __init__(self, topic: TypedTopic[T]):
        self.topic = topic
        self.adapter = topic.adapter()
        self.local: list[Sender[T]] = []

    async def deliver(self, item: T) -> None:
        dead = []
        for s in self.local:
            try:
                await s.send(item)
            except ChannelClosed:
                dead.append(s)
        for s in dead:
            self.local.remove(s)


class Router:
    def __init__(self, node_id: NodeId, transport: Transport | None = None):
        self.node_id, self.transport = node_id, transport
        self.topics: dict[str, TopicRouter[Any]] = {}
        self._pending_ingest: list[tuple[TypedTopic[Any], Receiver[Any]]] = []
        self._tg: anyio.abc.TaskGroup | None = None

    def register_topic(self, topic: TypedTopic[Any]) -> None:
        self.topics.setdefault(topic.name, TopicRouter(topic))

    def sender(self, topic: TypedTopic[T]) -> Sender[T]:
        """A sender whose items go to local subscribers and (policy permitting) to the network."""
        self.register_topic(topic)
        s, r = channel()
        if self._tg is None:
            self._pending_ingest.append((topic, r))   # started by run()
        else:
            self._tg.start_soon(self._ingest, topic, r)
        return s

    def receiver(self, topic: TypedTopic[T]) -> Receiver[T]:
        self.register_topic(topic)
        s, r = channel()
        self.topics[topic.name].local.append(s)
        return r

    async def _ingest(self, topic: TypedTopic[Any], recv: Receiver[Any]) -> None:
        tr = self.topics[topic.name]
        async for item in recv:
            await tr.deliver(item)
            if topic.policy == PublishPolicy.Always and self.transport is not None:
                data = tr.adapter.dump_json(item)
                if len(data) > (1 << 20):
                    log.warning("message of %d bytes on topic %s", len(data), topic.name)
                await self.transport.publish(topic.name, data)

    async def _network_in(self) -> None:
        assert self.transport is not None
        while True:
            try:
                kind, payload = await self.transport.recv()
            except ChannelClosed:
                return
            if kind == "message":
                name, data = payload
                tr = self.topics.get(name)
                if tr is None:
                    continue
                try:
                    item = tr.adapter.validate_json(data)
                except ValueError as e:
                    log.warning("undecodable frame on %s: %s", name, e)
                    continue
                await tr.deliver(item)
            elif kind == "connection":
                peer, up = payload
                tr = self.topics.get(CONNECTION_MESSAGES.name)
                if tr is not None:
                    await tr.deliver(ConnectionMessage(node_id=NodeId(str(peer)), connected=bool(up)))

    async def run(self) -> None:
        async with anyio.create_task_group() as tg:
            self._tg = tg
            if self.transport is not None:
                for name, tr in self.topics.items():
                    if tr.topic.policy == PublishPolicy.Always:
                        await self.transport.subscribe(name)
                tg.start_soon(self._network_in)
            for topic, r in self._pending_ingest:
                tg.start_soon(self._ingest, topic, r)
            self._pending_ingest = []
            await anyio.sleep_forever()

    def shutdown(self) -> None:
        if self._tg is not None:
            self._tg.cancel_scope.cancel()
        if self.transport is not None:
            self.transport.close()


def make_router(node_id: NodeId, transport: Transport | None = None) -> Router:
    r = Router(node_id, transport)
    for t in ALL_TOPICS:
        r.register_topic(t)
    return r
