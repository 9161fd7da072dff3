"""The master: orders events, turns commands into events, prunes dead nodes.

One node of the cluster is elected master.  It is the only writer of the event log: local events
from every node are re-sequenced per origin, stamped, folded into its ``State``, appended to
disk and broadcast with a global index (reference ``src/exo/master/main.py:492-522``); commands
are turned into events (``:171-468``): a generation request goes to the serving instance with the
fewest in-flight tasks, placement commands go through the planner, ``RequestEventLog`` replays up
to 1000 logged events to a node that NACKed a gap (``:454-464``); every 10 s instances that
reference vanished nodes are deleted and nodes silent for 30 s are timed out (``:471-490``).
"""
from __future__ import annotations

from datetime import datetime, timedelta, timezone

import anyio
from pydantic import TypeAdapter

from ..shared import constants
from ..shared.base import CommandId, InstanceId, NodeId, SessionId, SystemId, TaskId
from ..shared.events import (ChunkGenerated, CustomModelCardAdded, CustomModelCardDeleted, Event, GlobalForwarderEvent,
                             IndexedEvent, InputChunkReceived, InstanceDeleted, InstanceLinkCreated,
                             InstanceLinkDeleted, LocalForwarderEvent, NodeGatheredInfo, NodeTimedOut, State,
                             TaskCreated, TaskDeleted, TaskStatusUpdated, TraceEventData, TracesCollected, TracesMerged,
                             apply)
from ..shared.messages import (AddCustomModelCard, CreateInstance, DeleteCustomModelCard, DeleteInstance,
                               DeleteInstanceLink, ForwarderCommand, ImageEdits, ImageEditsCommand, ImageGeneration,
                               ImageGenerationCommand, PlaceInstance, RequestEventLog, SendInputChunk, SetInstanceLink,
                               TaskCancelled, TaskFinished, TaskStatus, TestCommand, TextGeneration,
                               TextGenerationCommand)
from ..shared.wire import ErrorChunk, Instance, InstanceLink, RunnerReady, RunnerRunning
from ..utils.buffers import DiskEventLog, MultiSourceBuffer
from ..utils.channels import ChannelClosed, Receiver, Sender
from .placement import delete_instance, get_transition_events, place_instance

NODE_TIMEOUT = timedelta(seconds=30)
PLAN_INTERVAL = 10.0
REPLAY_LIMIT = 1000


class Master:
    def __init__(self, node_id: NodeId, session_id: SessionId, *, command_receiver: Receiver[ForwarderCommand],
                 local_event_receiver: Receiver[LocalForwarderEvent], global_event_sender: Sender[GlobalForwarderEvent],
                 log_dir=None, gpu_index: dict[NodeId, int] | None = None):
        self.node_id, self.session_id = node_id, session_id
        self.state = State()
        self._commands, self._local_events, self._global_out = command_receiver, local_event_receiver, global_event_sender
        self._buffer: MultiSourceBuffer[SystemId, Event] = MultiSourceBuffer()
        self._log = DiskEventLog(log_dir or constants.EXO_EVENT_LOG_DIR / "master")
        self._command_task: dict[CommandId, TaskId] = {}
        self._pending_traces: dict[TaskId, dict[int, list[TraceEventData]]] = {}
        self._expected_ranks: dict[TaskId, set[int]] = {}
        self.gpu_index = gpu_index or {}
        self._tg: anyio.abc.TaskGroup | None = None

    # ---- event path ----
    async def _emit(self, event: Event) -> None:
        """Index, fold, persist and broadcast one event."""
        idx = self.state.last_event_applied_idx + 1
        if isinstance(event, NodeGatheredInfo):
            event = event.model_copy(update={"when": datetime.now(tz=timezone.utc).isoformat()})
        self.state = apply(self.state, IndexedEvent(idx=idx, event=event))
        self._log.append(TypeAdapter(Event).dump_json(event).decode())
        await self._global_out.send(GlobalForwarderEvent(origin_idx=idx, origin=self.node_id, session=self.session_id,
                                                         event=event))
        if isinstance(event, TracesCollected):
            await self._collect_traces(event)

    async def _event_processor(self) -> None:
        async for fe in self._local_events:
            if fe.session != self.session_id:
                continue
            self._buffer.ingest(fe.origin_idx, fe.event, fe.origin)
            for ev in self._buffer.drain():
                await self._emit(ev)

    async def _collect_traces(self, ev: TracesCollected) -> None:
        got = self._pending_traces.setdefault(ev.task_id, {})
        got[ev.rank] = list(ev.traces)
        expected = self._expected_ranks.get(ev.task_id)
        if expected is not None and set(got) >= expected:
            merged = [t for r in sorted(got) for t in got[r]]
            self._pending_traces.pop(ev.task_id, None)
            self._expected_ranks.pop(ev.task_id, None)
            await self._emit(TracesMerged(task_id=ev.task_id, traces=merged))

    # ---- command path ----
    def _serving_instances(self, model: str) -> list[Instance]:
        """Instances of ``model`` whose runners are all Ready/Running."""
        out = []
        for inst in self.state.instances.values():
            if inst.shard_assignments.model_id != model:
                continue
            runners = inst.shard_assignments.runner_to_shard
            if all(isinstance(self.state.runners.get(r), (RunnerReady, RunnerRunning)) for r in runners):
                out.append(inst)
        return out

    def _pick_instance(self, model: str) -> Instance | None:
        """Least-loaded serving instance that is not reserved for prefill by an instance link."""
        prefill_only = {i for l in self.state.instance_links.values() for i in l.prefill_instances
                        if i not in l.decode_instances}
        cands = [i for i in self._serving_instances(model) if i.instance_id not in prefill_only] \
            or self._serving_instances(model)
        if not cands:
            return None
        load = {i.instance_id: 0 for i in cands}
        for t in self.state.tasks.values():
            if t.instance_id in load and t.task_status in (TaskStatus.Pending, TaskStatus.Running) \
                    and isinstance(t, (TextGeneration, ImageGeneration, ImageEdits)):
                load[t.instance_id] += 1
        return min(cands, key=lambda i: load[i.instance_id])

    def _prefill_endpoint_for(self, inst: Instance) -> str | None:
        for link in self.state.instance_links.values():
            if inst.instance_id not in link.decode_instances:
                continue
            for pid in link.prefill_instances:
                p = self.state.instances.get(pid)
                if p is None:
                    continue
                for rid, sm in p.shard_assignments.runner_to_shard.items():
                    port = self.state.prefill_server_ports.get(rid)
                    if sm.device_rank == 0 and port is not None:
                        return f"127.0.0.1:{port}"
        return None

    async def _generation(self, cmd, task_cls) -> None:
        inst = self._pick_instance(str(cmd.task_params.model))
        if inst is None:
            await self._emit(ChunkGenerated(command_id=cmd.command_id, chunk=ErrorChunk(
                model=cmd.task_params.model, error_message=f"No instance found for model {cmd.task_params.model}")))
            return
        params = cmd.task_params
        if task_cls is TextGeneration:
            ep = self._prefill_endpoint_for(inst)
            if ep is not None:
                params = params.model_copy(update={"prefill_endpoint": ep})
        task = task_cls(instance_id=inst.instance_id, command_id=cmd.command_id, task_params=params)
        self._command_task[cmd.command_id] = task.task_id
        self._expected_ranks[task.task_id] = {s.device_rank for s in inst.shard_assignments.runner_to_shard.values()}
        await self._emit(TaskCreated(task_id=task.task_id, task=task))

    async def _handle(self, cmd) -> None:
        st = self.state
        if isinstance(cmd, TestCommand):
            return
        if isinstance(cmd, TextGenerationCommand):
            await self._generation(cmd, TextGeneration)
        elif isinstance(cmd, ImageGenerationCommand):
            await self._generation(cmd, ImageGeneration)
        elif isinstance(cmd, ImageEditsCommand):
            await self._generation(cmd, ImageEdits)
        elif isinstance(cmd, PlaceInstance):
            target = place_instance(cmd, st.topology, st.instances, st.node_memory, st.node_backends,
                                    download_status=st.downloads,
                                    gpu_index={n: v.gpu_index for n, v in st.node_nvlink.items()} or self.gpu_index,
                                    node_nvlink=st.node_nvlink)
            for ev in get_transition_events(st.instances, target, st.tasks):
                await self._emit(ev)
        elif isinstance(cmd, CreateInstance):
            target = {**st.instances, cmd.instance.instance_id: cmd.instance}
            for ev in get_transition_events(st.instances, target, st.tasks):
                await self._emit(ev)
        elif isinstance(cmd, DeleteInstance):
            target = delete_instance(cmd, st.instances)
            for ev in get_transition_events(st.instances, target, st.tasks):
                await self._emit(ev)
        elif isinstance(cmd, SendInputChunk):
            await self._emit(InputChunkReceived(command_id=cmd.chunk.command_id, chunk=cmd.chunk))
        elif isinstance(cmd, TaskCancelled):
            tid = self._command_task.get(cmd.cancelled_command_id)
            if tid is not None and tid in st.tasks:
                await self._emit(TaskStatusUpdated(task_id=tid, task_status=TaskStatus.Cancelled))
        elif isinstance(cmd, TaskFinished):
            tid = self._command_task.pop(cmd.finished_command_id, None)
            if tid is not None and tid in st.tasks:
                await self._emit(TaskDeleted(task_id=tid))
        elif isinstance(cmd, AddCustomModelCard):
            await self._emit(CustomModelCardAdded(model_card=cmd.model_card))
        elif isinstance(cmd, DeleteCustomModelCard):
            await self._emit(CustomModelCardDeleted(model_id=cmd.model_id))
        elif isinstance(cmd, SetInstanceLink):
            await self._emit(InstanceLinkCreated(link=InstanceLink(link_id=cmd.link_id, prefill_instances=cmd.prefill_instances,
                                                                   decode_instances=cmd.decode_instances)))
        elif isinstance(cmd, DeleteInstanceLink):
            await self._emit(InstanceLinkDeleted(link_id=cmd.link_id))
        elif isinstance(cmd, RequestEventLog):
            end = min(len(self._log), cmd.since_idx + REPLAY_LIMIT)
            ta = TypeAdapter(Event)
            for i, raw in enumerate(self._log.read_range(cmd.since_idx, end), start=cmd.since_idx):
                await self._global_out.send(GlobalForwarderEvent(origin_idx=i, origin=self.node_id, session=self.session_id,
                                                                 event=ta.validate_json(raw)))

    async def _command_processor(self) -> None:
        async for fc in self._commands:
            try:
                await self._handle(fc.command)
            except ValueError as e:
                # planner / validation errors do not take the master down; the API learns through state
                self.last_error = str(e)

    # ---- housekeeping ----
    async def plan_once(self, now: datetime | None = None) -> None:
        now = now or datetime.now(tz=timezone.utc)
        alive = set(self.state.topology.list_nodes())
        for iid, inst in list(self.state.instances.items()):
            if any(n not in alive for n in inst.shard_assignments.node_to_runner):
                for ev in get_transition_events(self.state.instances, {k: v for k, v in self.state.instances.items() if k != iid},
                                                self.state.tasks):
                    await self._emit(ev)
        for n, seen in list(self.state.last_seen.items()):
            if now - seen > NODE_TIMEOUT:
                await self._emit(NodeTimedOut(node_id=n))

    async def _plan_loop(self) -> None:
        while True:
            await anyio.sleep(PLAN_INTERVAL)
            await self.plan_once()

    async def run(self) -> None:
        self.last_error: str | None = None
        try:
            async with anyio.create_task_group() as tg:
                self._tg = tg
                tg.start_soon(self._event_processor)
                tg.start_soon(self._command_processor)
                tg.start_soon(self._plan_loop)
        except ChannelClosed:
            pass
        finally:
            self._log.close()

    def shutdown(self) -> None:
        if self._tg is not None:
            self._tg.cancel_scope.cancel()
