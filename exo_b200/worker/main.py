"""The worker of a node: folds events into a local state copy, plans, and drives its runners.

Loop structure of the reference (``src/exo/worker/main.py:65-432``): an event applier (which also
assembles chunked image uploads into an image cache keyed by SHA-256), a planner tick every
100 ms that asks :func:`exo_b200.worker.plan.plan` for at most one task and carries it out, a
telemetry forwarder, a peer-reachability poll that creates and deletes socket edges, and a
reconciler that mirrors cluster-wide custom model cards onto disk.  An instance whose runner has
been created ``EXO_MAX_INSTANCE_RETRIES`` times without success is reported to the master for
deletion instead of being retried forever.
"""
from __future__ import annotations

import hashlib
from collections import defaultdict
from datetime import datetime, timezone

import anyio

from ..download.store import is_read_only_model_dir, resolve_existing_model
from ..shared import constants
from ..shared.base import CommandId, InstanceId, ModelId, NodeId, RunnerId, SystemId
from ..shared.cards import card_cache
from ..shared.events import (Event, IndexedEvent, InputChunkReceived, InstanceDeleted, NodeDownloadProgress,
                             NodeGatheredInfo, State, TaskCreated, TaskStatusUpdated, TopologyEdgeCreated,
                             TopologyEdgeDeleted, apply)
from ..shared.messages import (CancelTask, CreateRunner, DeleteInstance, DownloadModel, ForwarderCommand,
                               ForwarderDownloadCommand, ImageEdits, LoadModel, Shutdown, StartDownload, Task, TaskStatus,
                               TextGeneration)
from ..shared.topology import Connection, Multiaddr, SocketConnection
from ..shared.wire import DownloadCompleted, GatheredInfo, InputImageChunk
from ..utils.async_process import TaskGroup
from ..utils.buffers import KeyedBackoff
from ..utils.channels import ChannelClosed, Receiver, Sender, channel
from ..utils.info_gatherer import InfoGatherer, check_reachable
from .plan import plan
from .runner.supervisor import RunnerSupervisor

PLAN_INTERVAL_S = 0.1
REACHABILITY_INTERVAL_S = 10.0


class Worker:
    def __init__(self, node_id: NodeId, *, event_receiver: Receiver[IndexedEvent], event_sender: Sender[Event],
                 command_sender: Sender[ForwarderCommand], download_command_sender: Sender[ForwarderDownloadCommand],
                 api_port: int = 52415, info_gatherer: InfoGatherer | None = None, supervisor_factory=RunnerSupervisor.create,
                 poll_connections: bool = True):
        self.node_id, self.api_port = node_id, api_port
        self.event_receiver, self.event_sender = event_receiver, event_sender
        self.command_sender, self.download_command_sender = command_sender, download_command_sender
        self.state = State()
        self.runners: dict[RunnerId, RunnerSupervisor] = {}
        self.input_chunk_buffer: dict[CommandId, dict[int, InputImageChunk]] = {}
        self.input_chunk_counts: dict[CommandId, int] = {}
        self.image_cache: dict[str, str] = {}
        self._download_backoff: KeyedBackoff[ModelId] = KeyedBackoff(base=0.5, cap=10.0)
        self._instance_backoff: KeyedBackoff[InstanceId] = KeyedBackoff(base=0.5, cap=10.0)
        self._system_id = SystemId()
        self._synced_cards: set[ModelId] = set()
        self._tg = TaskGroup()
        self._stopped = anyio.Event()
        self._info_gatherer, self._make_supervisor, self._poll = info_gatherer, supervisor_factory, poll_connections

    # ---- lifecycle ----
    async def run(self) -> None:
        info_s, info_r = channel()
        gatherer = self._info_gatherer or InfoGatherer(info_s)
        gatherer.sender = info_s
        try:
            async with self._tg as tg:
                tg.start_soon(gatherer.run)
                tg.start_soon(self._forward_info, info_r)
                tg.start_soon(self._plan_loop)
                tg.start_soon(self._event_applier)
                if self._poll:
                    tg.start_soon(self._poll_connection_updates)
                tg.start_soon(self._reconcile_custom_cards)
        except* ChannelClosed:
            pass
        finally:
            self.event_sender.close()
            self.command_sender.close()
            self.download_command_sender.close()
            for r in list(self.runners.values()):
                with anyio.CancelScope(shield=True):
                    await r.shutdown(grace=0.5)
            self._stopped.set()

    async def shutdown(self) -> None:
        self._tg.cancel_tasks()
        await self._stopped.wait()

    # ---- inbound ----
    async def _forward_info(self, recv: Receiver[GatheredInfo]) -> None:
        with recv as infos:
            async for info in infos:
                await self.event_sender.send(NodeGatheredInfo(node_id=self.node_id, when=str(datetime.now(tz=timezone.utc)), info=info))

    def _on_input_chunk(self, ev: InputChunkReceived) -> None:
        cid = ev.command_id
        buf = self.input_chunk_buffer.setdefault(cid, {})
        self.input_chunk_counts.setdefault(cid, ev.chunk.total_chunks)
        buf[ev.chunk.chunk_index] = ev.chunk
        if len(buf) != self.input_chunk_counts[cid]:
            return
        per_image: dict[int, list[InputImageChunk]] = defaultdict(list)
        for ch in buf.values():
            per_image[ch.image_index].append(ch)
        for chunks in per_image.values():
            img = "".join(c.data for c in sorted(chunks, key=lambda c: c.chunk_index))
            self.image_cache[hashlib.sha256(img.encode("ascii")).hexdigest()] = img

    async def _event_applier(self) -> None:
        with self.event_receiver as events:
            async for ie in events:
                self.state = apply(self.state, ie)
                ev = ie.event
                if isinstance(ev, InstanceDeleted):
                    self._instance_backoff.reset(ev.instance_id)
                elif isinstance(ev, InputChunkReceived):
                    self._on_input_chunk(ev)

    async def _reconcile_custom_cards(self) -> None:
        while True:
            await anyio.sleep(1.0)
            target = dict(self.state.custom_model_cards)
            for mid, card in target.items():
                self._synced_cards.add(mid)
                if card_cache.get(mid) != card:
                    card_cache.save(card)
            # only cards that came from the cluster are removed with it; cards derived from local checkpoints stay
            for mid in [m for m in self._synced_cards if m not in target]:
                self._synced_cards.discard(mid)
                card_cache.pop(mid)

    # ---- planning ----
    async def _plan_loop(self) -> None:
        while True:
            await anyio.sleep(PLAN_INTERVAL_S)
            await self.plan_step()

    async def plan_step(self) -> Task | None:
        task = plan(self.node_id, self.runners, self.state.downloads, self.state.instances, self.state.runners,
                    self.state.tasks, self.input_chunk_buffer, self.image_cache, self._instance_backoff,
                    self._download_backoff)
        if task is None:
            return None
        if isinstance(task, CreateRunner) and self._instance_backoff.attempts_for(task.instance_id) >= constants.EXO_MAX_INSTANCE_RETRIES:
            await self.command_sender.send(ForwarderCommand(origin=self._system_id, command=DeleteInstance(instance_id=task.instance_id)))
            return None
        await self.event_sender.send(TaskCreated(task_id=task.task_id, task=task))
        await self._execute(task)
        return task

    async def _status(self, task: Task, status: TaskStatus) -> None:
        await self.event_sender.send(TaskStatusUpdated(task_id=task.task_id, task_status=status))

    async def _execute(self, task: Task) -> None:
        if isinstance(task, CreateRunner):
            sup = self._make_supervisor(task.bound_instance, self.event_sender.clone())
            self.runners[task.bound_instance.bound_runner_id] = sup
            self._tg.start_soon(sup.run)
            self._instance_backoff.record_attempt(task.instance_id)
            await self._status(task, TaskStatus.Complete)
        elif isinstance(task, DownloadModel):
            shard = task.shard_metadata
            mid = shard.model_card.model_id
            self._download_backoff.record_attempt(mid)
            found = await anyio.to_thread.run_sync(resolve_existing_model, mid, shard.model_card)
            if found is not None:
                await self.event_sender.send(NodeDownloadProgress(download_progress=DownloadCompleted(
                    node_id=self.node_id, shard_metadata=shard, model_directory=str(found), total=shard.model_card.storage_size,
                    read_only=is_read_only_model_dir(found))))
                await self._status(task, TaskStatus.Complete)
            else:
                await self.download_command_sender.send(ForwarderDownloadCommand(
                    origin=self._system_id, command=StartDownload(target_node_id=self.node_id, shard_metadata=shard)))
                await self._status(task, TaskStatus.Running)
        elif isinstance(task, Shutdown):
            sup = self.runners.pop(task.runner_id, None)
            if sup is None:
                return
            try:
                with anyio.fail_after(3):
                    await sup.start_task(task)
            except TimeoutError:
                await self._status(task, TaskStatus.TimedOut)
            finally:
                await sup.shutdown()
        elif isinstance(task, CancelTask):
            sup = self.runners.get(task.runner_id)
            if sup is not None:
                await sup.cancel_task(task.cancelled_task_id)
            await self._status(task, TaskStatus.Complete)
        elif isinstance(task, ImageEdits) and task.task_params.total_input_chunks > 0:
            chunks = self.input_chunk_buffer.pop(task.command_id, {})
            self.input_chunk_counts.pop(task.command_id, None)
            data = "".join(chunks[i].data for i in range(len(chunks)))
            await self._to_runner(task.model_copy(update={"task_params": task.task_params.model_copy(update={"image_data": data})}))
        elif isinstance(task, TextGeneration) and task.task_params.image_hashes:
            images = [self.image_cache[h] for _i, h in sorted(task.task_params.image_hashes.items())]
            self.input_chunk_buffer.pop(task.command_id, None)
            self.input_chunk_counts.pop(task.command_id, None)
            await self._to_runner(task.model_copy(update={"task_params": task.task_params.model_copy(update={"images": images})}))
        else:
            if isinstance(task, LoadModel) and (inst := self.state.instances.get(task.instance_id)) is not None:
                self._download_backoff.reset(inst.shard_assignments.model_id)
            await self._to_runner(task)

    async def _to_runner(self, task: Task) -> None:
        inst = self.state.instances.get(task.instance_id)
        if inst is None:
            return
        sup = self.runners.get(inst.shard_assignments.node_to_runner.get(self.node_id))
        if sup is not None:
            await sup.start_task(task)

    # ---- reachability → socket edges ----
    async def _poll_connection_updates(self) -> None:
        while True:
            try:
                await self.poll_connections_once()
            except ChannelClosed:
                return
            except Exception:  # noqa: BLE001 - a failing probe must not end the worker
                pass
            await anyio.sleep(REACHABILITY_INTERVAL_S)

    async def poll_connections_once(self) -> None:
        edges = {c.edge for c in self.state.topology.out_edges(self.node_id)}
        candidates = {str(n): sorted({i.ip_address for i in info.interfaces})
                      for n, info in self.state.node_network.items() if n != self.node_id}
        seen: dict[NodeId, set[str]] = defaultdict(set)
        async for ip, nid in check_reachable(candidates, self.api_port):
            node = NodeId(nid)
            if ip in seen[node]:
                continue
            seen[node].add(ip)
            proto = "ip4" if "." in ip else "ip6"
            edge = SocketConnection(sink_multiaddr=Multiaddr(address=f"/{proto}/{ip}/tcp/{self.api_port}"))
            if edge not in edges:
                await self.event_sender.send(TopologyEdgeCreated(conn=Connection(source=self.node_id, sink=node, edge=edge)))
        for conn in self.state.topology.out_edges(self.node_id):
            if not isinstance(conn.edge, SocketConnection) or conn.edge.sink_multiaddr.port != self.api_port:
                continue
            if conn.edge.sink_multiaddr.ip_address not in seen.get(conn.sink, set()):
                await self.event_sender.send(TopologyEdgeDeleted(conn=conn))
