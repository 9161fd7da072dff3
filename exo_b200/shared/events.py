"""Events, the global ``State`` and the pure fold ``apply(state, indexed_event)``.

Only the master orders events; every component keeps a ``State`` that is the fold of ``apply`` over
the indexed log (reference: event union ``src/exo/shared/types/events.py:149-172``, state
``src/exo/shared/types/state.py:30-94``, fold ``src/exo/shared/apply.py:82-136``: strict index
contiguity, pass-through events, per-family handlers).  NVLink telemetry is folded into topology
edges here the way the reference folds RDMA interface reports (``apply.py:410-463``).
"""
from __future__ import annotations

import copy
from collections.abc import Mapping, Sequence
from datetime import datetime, timezone
from typing import Any, cast

from pydantic import ConfigDict, Field, field_serializer, field_validator
from pydantic.alias_generators import to_camel

from .base import (CommandId, EventId, FrozenModel, InstanceId, InstanceLinkId, ModelId, NodeId, RunnerId, SessionId,
                   SystemId, TaggedModel, TaskId)
from .cards import Backend, ModelCard
from .messages import Task, TaskStatus
from .topology import Connection, NvlinkConnection, Topology, TopologySnapshot
from .wire import (Chunk, DiskUsage, DownloadProgress, GatheredInfo, InputImageChunk, Instance, InstanceLink,
                   MemoryUsage, MiscData, NodeBackends, NodeDiskUsage, NodeIdentity, NodeMemory, NodeNetworkInfo,
                   NodeNetworkInterfaces, NodeNvlink, NodeNvlinkInfo, NodePerformance, NodeRdmaCtlStatus,
                   NodeThunderboltInfo, RdmaCtlStatus, RunnerReady, RunnerShutdown, RunnerStatus,
                   StaticNodeInformation, SystemPerformanceProfile, ThunderboltBridgeStatus)


class BaseEvent(TaggedModel):
    event_id: EventId = Field(default_factory=EventId)


class TestEvent(BaseEvent):
    __test__ = False


class TaskCreated(BaseEvent):
    task_id: TaskId
    task: Task


class TaskAcknowledged(BaseEvent):
    task_id: TaskId


class TaskDeleted(BaseEvent):
    task_id: TaskId


class TaskStatusUpdated(BaseEvent):
    task_id: TaskId
    task_status: TaskStatus


class TaskFailed(BaseEvent):
    task_id: TaskId
    error_type: str
    error_message: str


class InstanceCreated(BaseEvent):
    instance: Instance


class InstanceDeleted(BaseEvent):
    instance_id: InstanceId


class RunnerStatusUpdated(BaseEvent):
    runner_id: RunnerId
    runner_status: RunnerStatus


class NodeTimedOut(BaseEvent):
    node_id: NodeId


class NodeGatheredInfo(BaseEvent):
    node_id: NodeId
    when: str  # ISO timestamp, overwritten by the master when it indexes the event
    info: GatheredInfo


class NodeDownloadProgress(BaseEvent):
    download_progress: DownloadProgress


class ChunkGenerated(BaseEvent):
    command_id: CommandId
    chunk: Chunk


class InputChunkReceived(BaseEvent):
    command_id: CommandId
    chunk: InputImageChunk


class TopologyEdgeCreated(BaseEvent):
    conn: Connection


class TopologyEdgeDeleted(BaseEvent):
    conn: Connection


class CustomModelCardAdded(BaseEvent):
    model_card: ModelCard


class CustomModelCardDeleted(BaseEvent):
    model_id: ModelId


class TraceEventData(FrozenModel):
    name: str
    start_us: int
    duration_us: int
    rank: int
    category: str


class TracesCollected(BaseEvent):
    task_id: TaskId
    rank: int
    traces: list[TraceEventData]


class TracesMerged(BaseEvent):
    task_id: TaskId
    traces: list[TraceEventData]


class InstanceLinkCreated(BaseEvent):
    link: InstanceLink


class InstanceLinkDeleted(BaseEvent):
    link_id: InstanceLinkId


Event = (TestEvent | TaskCreated | TaskStatusUpdated | TaskFailed | TaskDeleted | TaskAcknowledged | InstanceCreated
         | InstanceDeleted | RunnerStatusUpdated | NodeTimedOut | NodeGatheredInfo | NodeDownloadProgress
         | ChunkGenerated | InputChunkReceived | TopologyEdgeCreated | TopologyEdgeDeleted | TracesCollected
         | TracesMerged | CustomModelCardAdded | CustomModelCardDeleted | InstanceLinkCreated | InstanceLinkDeleted)

PASS_THROUGH = (TestEvent, ChunkGenerated, TaskAcknowledged, InputChunkReceived, TracesCollected, TracesMerged)


class IndexedEvent(FrozenModel):
    idx: int = Field(ge=0)
    event: Event


class GlobalForwarderEvent(FrozenModel):
    origin_idx: int = Field(ge=0)
    origin: NodeId
    session: SessionId
    event: Event


class LocalForwarderEvent(FrozenModel):
    origin_idx: int = Field(ge=0)
    origin: SystemId
    session: SessionId
    event: Event


class State(FrozenModel):
    """Global cluster state; ``topology`` travels as a snapshot."""
    model_config = ConfigDict(alias_generator=to_camel, validate_by_name=True, extra="forbid", strict=True,
                              arbitrary_types_allowed=True, serialize_by_alias=True)
    instances: Mapping[InstanceId, Instance] = {}
    runners: Mapping[RunnerId, RunnerStatus] = {}
    downloads: Mapping[NodeId, Sequence[DownloadProgress]] = {}
    tasks: Mapping[TaskId, Task] = {}
    last_seen: Mapping[NodeId, datetime] = {}
    topology: Topology = Field(default_factory=Topology)
    last_event_applied_idx: int = Field(default=-1, ge=-1)
    node_identities: Mapping[NodeId, NodeIdentity] = {}
    node_memory: Mapping[NodeId, MemoryUsage] = {}
    node_disk: Mapping[NodeId, DiskUsage] = {}
    node_system: Mapping[NodeId, SystemPerformanceProfile] = {}
    node_network: Mapping[NodeId, NodeNetworkInfo] = {}
    node_thunderbolt: Mapping[NodeId, NodeThunderboltInfo] = {}
    node_thunderbolt_bridge: Mapping[NodeId, ThunderboltBridgeStatus] = {}
    node_rdma_ctl: Mapping[NodeId, NodeRdmaCtlStatus] = {}
    node_backends: Mapping[NodeId, list[Backend]] = {}
    node_nvlink: Mapping[NodeId, NodeNvlinkInfo] = {}
    thunderbolt_bridge_cycles: Sequence[Sequence[NodeId]] = []
    instance_links: Mapping[InstanceLinkId, InstanceLink] = {}
    prefill_server_ports: Mapping[RunnerId, int] = {}
    custom_model_cards: Mapping[ModelId, ModelCard] = {}

    @field_serializer("topology", mode="plain")
    def _enc_topology(self, v: Topology) -> TopologySnapshot:
        return v.to_snapshot()

    @field_validator("topology", mode="before")
    @classmethod
    def _dec_topology(cls, v: object) -> Topology:
        if isinstance(v, Topology):
            return v
        if isinstance(v, TopologySnapshot):
            return Topology.from_snapshot(v)
        if isinstance(v, Mapping):
            return Topology.from_snapshot(TopologySnapshot(**cast(dict[str, Any], v)))
        raise TypeError("Invalid representation for Topology field in State")


# ------------------------------------------------------------------------------------------------
# the fold
# ------------------------------------------------------------------------------------------------
def _without(m: Mapping, key) -> dict:
    return {k: v for k, v in m.items() if k != key}


def _gathered(ev: NodeGatheredInfo, st: State) -> State:
    n, info = ev.node_id, ev.info
    try:
        when = datetime.fromisoformat(ev.when)
    except ValueError:
        when = datetime.now(tz=timezone.utc)
    topo = st.topology
    if not topo.contains_node(n):
        topo = copy.deepcopy(topo)
        topo.add_node(n)
    upd: dict[str, Any] = {"last_seen": {**st.last_seen, n: when}, "topology": topo}
    ident = st.node_identities.get(n, NodeIdentity())
    if isinstance(info, NodeMemory):
        upd["node_memory"] = {**st.node_memory, n: info.memory}
    elif isinstance(info, NodePerformance):
        upd["node_system"] = {**st.node_system, n: info.profile}
    elif isinstance(info, NodeDiskUsage):
        upd["node_disk"] = {**st.node_disk, n: info.disk_usage}
    elif isinstance(info, NodeNetworkInterfaces):
        upd["node_network"] = {**st.node_network, n: NodeNetworkInfo(interfaces=info.ifaces)}
    elif isinstance(info, StaticNodeInformation):
        upd["node_identities"] = {**st.node_identities, n: ident.model_copy(update={
            "model_id": info.model, "chip_id": info.chip, "os_version": info.os_version,
            "os_build_version": info.os_build_version})}
    elif isinstance(info, MiscData):
        upd["node_identities"] = {**st.node_identities, n: ident.model_copy(update={"friendly_name": info.friendly_name})}
    elif isinstance(info, NodeBackends):
        upd["node_backends"] = {**st.node_backends, n: list(info.backends)}
    elif isinstance(info, RdmaCtlStatus):
        upd["node_rdma_ctl"] = {**st.node_rdma_ctl, n: NodeRdmaCtlStatus(enabled=info.enabled)}
    elif isinstance(info, NodeNvlink):
        nv = {**st.node_nvlink, n: info.info}
        upd["node_nvlink"] = nv
        # NVLink edges exist between two nodes once both sides have reported the other as a P2P peer
        topo = copy.deepcopy(topo)
        by_gpu = {v.gpu_index: k for k, v in nv.items()}
        for conn in [c for c in topo.out_edges(n) if isinstance(c.edge, NvlinkConnection)]:
            topo.remove_connection(conn)
        for p in info.info.peers:
            peer = by_gpu.get(p.peer_gpu)
            if peer is None or not p.p2p:
                continue
            back = [q for q in nv[peer].peers if q.peer_gpu == info.info.gpu_index and q.p2p]
            if not back:
                continue
            topo.add_connection(Connection(source=n, sink=peer, edge=NvlinkConnection(
                source_gpu=info.info.gpu_index, sink_gpu=p.peer_gpu, gbps=p.gbps, links=p.links)))
            if not any(isinstance(e, NvlinkConnection) for e in topo.get_all_connections_between(peer, n)):
                topo.add_connection(Connection(source=peer, sink=n, edge=NvlinkConnection(
                    source_gpu=p.peer_gpu, sink_gpu=info.info.gpu_index, gbps=back[0].gbps, links=back[0].links)))
        upd["topology"] = topo
    return st.model_copy(update=upd)


def _node_timed_out(ev: NodeTimedOut, st: State) -> State:
    topo = copy.deepcopy(st.topology)
    topo.remove_node(ev.node_id)
    upd: dict[str, Any] = {"topology": topo}
    for f in ("last_seen", "downloads", "node_identities", "node_memory", "node_disk", "node_system", "node_network",
              "node_thunderbolt", "node_thunderbolt_bridge", "node_rdma_ctl", "node_backends", "node_nvlink"):
        upd[f] = _without(getattr(st, f), ev.node_id)
    return st.model_copy(update=upd)


def event_apply(ev: Event, st: State) -> State:
    if isinstance(ev, PASS_THROUGH):
        return st
    if isinstance(ev, TaskCreated):
        return st.model_copy(update={"tasks": {**st.tasks, ev.task_id: ev.task}})
    if isinstance(ev, TaskDeleted):
        return st.model_copy(update={"tasks": _without(st.tasks, ev.task_id)})
    if isinstance(ev, TaskStatusUpdated):
        if ev.task_id not in st.tasks:
            return st
        upd: dict[str, Any] = {"task_status": ev.task_status}
        t = st.tasks[ev.task_id]
        if ev.task_status != TaskStatus.Failed and hasattr(t, "error_type"):
            upd.update(error_type=None, error_message=None)
        return st.model_copy(update={"tasks": {**st.tasks, ev.task_id: t.model_copy(update=upd)}})
    if isinstance(ev, TaskFailed):
        if ev.task_id not in st.tasks or not hasattr(st.tasks[ev.task_id], "error_type"):
            return st
        t = st.tasks[ev.task_id].model_copy(update={"error_type": ev.error_type, "error_message": ev.error_message})
        return st.model_copy(update={"tasks": {**st.tasks, ev.task_id: t}})
    if isinstance(ev, InstanceCreated):
        return st.model_copy(update={"instances": {**st.instances, ev.instance.instance_id: ev.instance}})
    if isinstance(ev, InstanceDeleted):
        links: dict[InstanceLinkId, InstanceLink] = {}
        for lid, link in st.instance_links.items():
            pre = [i for i in link.prefill_instances if i != ev.instance_id]
            dec = [i for i in link.decode_instances if i != ev.instance_id]
            if pre and dec:
                links[lid] = link if (pre == list(link.prefill_instances) and dec == list(link.decode_instances)) \
                    else link.model_copy(update={"prefill_instances": pre, "decode_instances": dec})
        return st.model_copy(update={"instances": _without(st.instances, ev.instance_id), "instance_links": links})
    if isinstance(ev, InstanceLinkCreated):
        return st.model_copy(update={"instance_links": {**st.instance_links, ev.link.link_id: ev.link}})
    if isinstance(ev, InstanceLinkDeleted):
        return st.model_copy(update={"instance_links": _without(st.instance_links, ev.link_id)})
    if isinstance(ev, RunnerStatusUpdated):
        if isinstance(ev.runner_status, RunnerShutdown):
            return st.model_copy(update={"runners": _without(st.runners, ev.runner_id),
                                         "prefill_server_ports": _without(st.prefill_server_ports, ev.runner_id)})
        upd = {"runners": {**st.runners, ev.runner_id: ev.runner_status}}
        if isinstance(ev.runner_status, RunnerReady) and ev.runner_status.prefill_server_port is not None:
            upd["prefill_server_ports"] = {**st.prefill_server_ports, ev.runner_id: ev.runner_status.prefill_server_port}
        return st.model_copy(update=upd)
    if isinstance(ev, NodeTimedOut):
        return _node_timed_out(ev, st)
    if isinstance(ev, NodeDownloadProgress):
        dp = ev.download_progress
        cur = list(st.downloads.get(dp.node_id, ()))
        for i, old in enumerate(cur):
            if old.shard_metadata.model_card.model_id == dp.shard_metadata.model_card.model_id:
                cur[i] = dp
                break
        else:
            cur.append(dp)
        return st.model_copy(update={"downloads": {**st.downloads, dp.node_id: cur}})
    if isinstance(ev, NodeGatheredInfo):
        return _gathered(ev, st)
    if isinstance(ev, TopologyEdgeCreated):
        topo = copy.deepcopy(st.topology)
        topo.add_connection(ev.conn)
        return st.model_copy(update={"topology": topo})
    if isinstance(ev, TopologyEdgeDeleted):
        topo = copy.deepcopy(st.topology)
        topo.remove_connection(ev.conn)
        return st.model_copy(update={"topology": topo})
    if isinstance(ev, CustomModelCardAdded):
        return st.model_copy(update={"custom_model_cards": {**st.custom_model_cards, ev.model_card.model_id: ev.model_card}})
    if isinstance(ev, CustomModelCardDeleted):
        return st.model_copy(update={"custom_model_cards": _without(st.custom_model_cards, ev.model_id)})
    raise TypeError(f"unhandled event {type(ev).__name__}")


def apply(state: State, event: IndexedEvent) -> State:
    """Fold one indexed event; indices must be contiguous (the transport re-orders and NACKs gaps)."""
    assert state.last_event_applied_idx == event.idx - 1, \
        f"Expected event {state.last_event_applied_idx + 1} but received {event.idx}"
    return event_apply(event.event, state).model_copy(update={"last_event_applied_idx": event.idx})
