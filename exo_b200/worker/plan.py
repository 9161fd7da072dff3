"""The worker's reconciler: a pure function from (cluster state, local runners) to the next task.

Rules are tried in a fixed priority order, the first that fires wins, one task per tick
(reference ``src/exo/worker/plan.py:47-72``):

  cancel → kill runner → create runner → download → connect → load → warm up → forward task

and their conditions are the reference's (``plan.py:75-362``): a runner is shut down when its
instance disappeared or it, or any peer of its instance, failed; a failed instance is re-created
with back-off, waiting for failed peers first; ranks 0..n-2 connect while everyone is Idle or
Connecting and the last rank joins once all the others are Connecting; the model is loaded once
every node of the instance has it on disk and all runners are Connected/Loading/Loaded; ranks > 0
warm up first and rank 0 last; generation tasks are forwarded only while *all* runners of the
instance are Ready or Running.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from typing import Protocol

from ..shared.base import CommandId, InstanceId, ModelId, NodeId, RunnerId, TaskId
from ..shared.messages import (CancelTask, ConnectToGroup, CreateRunner, DownloadModel, ImageEdits, ImageGeneration,
                               LoadModel, Shutdown, StartWarmup, Task, TaskStatus, TextGeneration)
from ..shared.wire import (BoundInstance, DownloadCompleted, DownloadFailed, DownloadOngoing, DownloadProgress,
                           Instance, RunnerConnected, RunnerConnecting, RunnerFailed, RunnerIdle, RunnerLoaded,
                           RunnerLoading, RunnerReady, RunnerRunning, RunnerStatus, RunnerWarmingUp)
from ..utils.buffers import KeyedBackoff

GENERATION = (TextGeneration, ImageGeneration, ImageEdits)


class RunnerView(Protocol):
    """What the planner needs to know about a local runner (a supervisor, or a fake in tests)."""
    bound_instance: BoundInstance
    status: RunnerStatus
    completed: set[TaskId]
    in_progress: set[TaskId]
    cancelled: set[TaskId]


class Ctx:
    def __init__(self, node_id, runners, downloads, instances, all_runners, tasks, input_chunks, image_cache,
                 instance_backoff, download_backoff):
        self.node_id: NodeId = node_id
        self.runners: Mapping[RunnerId, RunnerView] = runners
        self.downloads: Mapping[NodeId, Sequence[DownloadProgress]] = downloads
        self.instances: Mapping[InstanceId, Instance] = instances
        self.all: Mapping[RunnerId, RunnerStatus] = all_runners
        self.tasks: Mapping[TaskId, Task] = tasks
        self.input_chunks: Mapping[CommandId, Mapping[int, object]] = input_chunks
        self.image_cache: Mapping[str, str] = image_cache
        self.instance_backoff: KeyedBackoff[InstanceId] = instance_backoff
        self.download_backoff: KeyedBackoff[ModelId] = download_backoff

    def peers(self, r: RunnerView) -> list[RunnerId]:
        return list(r.bound_instance.instance.shard_assignments.runner_to_shard)

    def all_in(self, ids, kinds, default=None) -> bool:
        return all(isinstance(self.all.get(i, default), kinds) for i in ids)


def _cancel(c: Ctx) -> Task | None:
    for t in c.tasks.values():
        if t.task_status != TaskStatus.Cancelled:
            continue
        for rid, r in c.runners.items():
            if t.instance_id == r.bound_instance.instance.instance_id and t.task_id in r.in_progress \
                    and t.task_id not in r.cancelled:
                return CancelTask(instance_id=t.instance_id, cancelled_task_id=t.task_id, runner_id=rid)
    return None


def _kill(c: Ctx) -> Task | None:
    for r in c.runners.values():
        me = r.bound_instance.bound_runner_id
        iid = r.bound_instance.instance.instance_id
        gone = iid not in c.instances
        peer_failed = any(isinstance(c.all.get(p), RunnerFailed) for p in c.peers(r) if p != me)
        if gone or isinstance(r.status, RunnerFailed) or peer_failed:
            return Shutdown(instance_id=iid, runner_id=me)
    return None


def _create(c: Ctx) -> Task | None:
    for inst in c.instances.values():
        rid = inst.shard_assignments.node_to_runner.get(c.node_id)
        if rid is None or rid in c.runners:
            continue
        others_failed = any(isinstance(c.all.get(p), RunnerFailed)
                            for p in inst.shard_assignments.node_to_runner.values() if p != rid)
        if others_failed and not isinstance(c.all.get(rid), RunnerFailed):
            continue  # let the failed peers come down first
        if not c.instance_backoff.should_proceed(inst.instance_id):
            continue
        return CreateRunner(instance_id=inst.instance_id,
                            bound_instance=BoundInstance(instance=inst, bound_runner_id=rid, bound_node_id=c.node_id))
    return None


def _download(c: Ctx) -> Task | None:
    mine = {dp.shard_metadata.model_card.model_id: dp for dp in c.downloads.get(c.node_id, [])}
    for r in c.runners.values():
        mid = r.bound_instance.bound_shard.model_card.model_id
        known = isinstance(mine.get(mid), (DownloadOngoing, DownloadCompleted, DownloadFailed))
        if isinstance(r.status, RunnerIdle) and not known and c.download_backoff.should_proceed(mid):
            return DownloadModel(instance_id=r.bound_instance.instance.instance_id, shard_metadata=r.bound_instance.bound_shard)
    return None


def _connect(c: Ctx) -> Task | None:
    for r in c.runners.values():
        peers = c.peers(r)
        if len(peers) == 1 or not isinstance(r.status, RunnerIdle):
            continue
        if not c.all_in(peers, (RunnerConnecting, RunnerIdle, RunnerConnected)):   # Connected: a rendezvous that does not block
            continue
        sh = r.bound_instance.bound_shard
        me = r.bound_instance.bound_runner_id
        last = sh.device_rank == sh.world_size - 1
        if not last or c.all_in([p for p in peers if p != me], (RunnerConnecting, RunnerConnected)):
            return ConnectToGroup(instance_id=r.bound_instance.instance.instance_id)
    return None


def _load(c: Ctx) -> Task | None:
    for r in c.runners.values():
        sa = r.bound_instance.instance.shard_assignments
        on_disk = all(any(isinstance(dp, DownloadCompleted) and dp.shard_metadata.model_card.model_id == sa.model_id
                          for dp in c.downloads.get(n, [])) for n in sa.node_to_runner)
        if not on_disk:
            continue
        peers = c.peers(r)
        if len(peers) == 1:
            if isinstance(r.status, RunnerIdle):
                return LoadModel(instance_id=r.bound_instance.instance.instance_id)
            continue
        if isinstance(r.status, RunnerConnected) and c.all_in(peers, (RunnerConnected, RunnerLoading, RunnerLoaded)):
            return LoadModel(instance_id=r.bound_instance.instance.instance_id)
    return None


def _warmup(c: Ctx) -> Task | None:
    for r in c.runners.values():
        if not isinstance(r.status, RunnerLoaded):
            continue
        peers = c.peers(r)
        me = r.bound_instance.bound_runner_id
        rank = r.bound_instance.bound_shard.device_rank
        followers_ready = rank > 0 and c.all_in(peers, (RunnerLoaded, RunnerWarmingUp, RunnerReady))
        leader_ready = rank == 0 and c.all_in([p for p in peers if p != me], (RunnerWarmingUp, RunnerReady))
        if followers_ready or leader_ready:
            return StartWarmup(instance_id=r.bound_instance.instance.instance_id)
    return None


def _forward(c: Ctx) -> Task | None:
    for t in c.tasks.values():
        if not isinstance(t, GENERATION) or t.task_status not in (TaskStatus.Pending, TaskStatus.Running):
            continue
        if isinstance(t, ImageEdits) and t.task_params.total_input_chunks > 0 \
                and len(c.input_chunks.get(t.command_id, {})) < t.task_params.total_input_chunks:
            continue  # image upload still in flight
        if isinstance(t, TextGeneration) and t.task_params.image_hashes \
                and not all(h in c.image_cache for h in t.task_params.image_hashes.values()):
            continue
        for r in c.runners.values():
            if t.instance_id != r.bound_instance.instance.instance_id:
                continue
            if t.task_id in r.completed or t.task_id in r.in_progress:
                continue
            if isinstance(r.status, (RunnerReady, RunnerRunning)) and c.all_in(c.peers(r), (RunnerReady, RunnerRunning)):
                return t
    return None


RULES: tuple[Callable[[Ctx], Task | None], ...] = (_cancel, _kill, _create, _download, _connect, _load, _warmup, _forward)


def plan(node_id: NodeId, runners: Mapping[RunnerId, RunnerView],
         global_download_status: Mapping[NodeId, Sequence[DownloadProgress]], instances: Mapping[InstanceId, Instance],
         all_runners: Mapping[RunnerId, RunnerStatus], tasks: Mapping[TaskId, Task],
         input_chunk_buffer: Mapping[CommandId, Mapping[int, object]] | None = None,
         image_cache: Mapping[str, str] | None = None, instance_backoff: KeyedBackoff | None = None,
         download_backoff: KeyedBackoff | None = None) -> Task | None:
    c = Ctx(node_id, runners, global_download_status, instances, all_runners, tasks, input_chunk_buffer or {},
            image_cache or {}, instance_backoff or KeyedBackoff(), download_backoff or KeyedBackoff())
    for rule in RULES:
        t = rule(c)
        if t is not None:
            return t
    return None
