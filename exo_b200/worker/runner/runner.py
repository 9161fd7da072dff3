"""The runner: the child process's state machine around one engine.

Idle → Connecting → Connected → Loading → Loaded → WarmingUp → Ready ⇄ Running → ShuttingDown →
Shutdown, each transition reported as ``RunnerStatusUpdated`` (reference
``src/exo/worker/runner/runner.py:233-311``).  Tasks arrive on one queue; while requests are in
flight the loop alternates ``engine.step()`` with non-blocking polls of the task and cancel
queues (``:329-386``).  Every task is acknowledged when taken and completed/failed when done.
A single-rank instance skips the connect states.
"""
from __future__ import annotations

import time
import traceback
from collections.abc import Callable

from ...shared import tracing
from ...shared.base import TaskId
from ...shared.events import (ChunkGenerated, Event, RunnerStatusUpdated, TaskAcknowledged, TaskStatusUpdated,
                              TraceEventData, TracesCollected)
from ...shared.messages import (ConnectToGroup, GenerationTask, ImageEdits, ImageGeneration, LoadModel, Shutdown,
                                StartWarmup, Task, TaskStatus, TextGeneration)
from ...shared.wire import (BoundInstance, ErrorChunk, RunnerConnected, RunnerConnecting, RunnerFailed, RunnerIdle,
                            RunnerLoaded, RunnerLoading, RunnerReady, RunnerRunning, RunnerShutdown, RunnerShuttingDown,
                            RunnerStatus, RunnerWarmingUp)
from ...utils.channels import ChannelClosed, MpReceiver, MpSender
from ..engines.base import Builder, Cancelled, Engine, Finished

GENERATION = (TextGeneration, ImageGeneration, ImageEdits)


class Runner:
    def __init__(self, bound_instance: BoundInstance, builder: Builder, events: MpSender[Event],
                 tasks: MpReceiver[Task], cancels: MpReceiver[TaskId], idle_poll: float = 0.05):
        self.bound, self.builder = bound_instance, builder
        self.events, self.tasks, self.cancels = events, tasks, cancels
        self.runner_id = bound_instance.bound_runner_id
        self.rank = bound_instance.bound_shard.device_rank
        self.engine: Engine | None = None
        self.status: RunnerStatus = RunnerIdle()
        self.idle_poll = idle_poll
        self.active: dict[TaskId, GenerationTask] = {}
        self.single = len(bound_instance.instance.shard_assignments.runner_to_shard) == 1

    # ---- reporting ----
    def emit(self, ev: Event) -> None:
        self.events.send(ev)

    def set_status(self, st: RunnerStatus) -> None:
        self.status = st
        self.emit(RunnerStatusUpdated(runner_id=self.runner_id, runner_status=st))

    def _done(self, task: Task, status: TaskStatus = TaskStatus.Complete) -> None:
        self.emit(TaskStatusUpdated(task_id=task.task_id, task_status=status))

    # ---- lifecycle tasks ----
    def _connect(self, task: Task) -> None:
        self.set_status(RunnerConnecting())
        self.builder.connect()
        self.set_status(RunnerConnected())
        self._done(task)

    def _load(self, task: Task) -> None:
        total = 0
        for p in self.builder.load():
            total = p.total_layers
            self.set_status(RunnerLoading(layers_loaded=p.layers_loaded, total_layers=p.total_layers))
        self.engine = self.builder.build()
        self.set_status(RunnerLoaded())
        self._done(task)

    def _warmup(self, task: Task) -> None:
        assert self.engine is not None
        self.set_status(RunnerWarmingUp())
        self.engine.warmup()
        self.set_status(RunnerReady(prefill_server_port=getattr(self.engine, "prefill_server_port", None)))
        self._done(task)

    # ---- generation ----
    def _start_generation(self, task: GenerationTask) -> None:
        assert self.engine is not None
        self.active[task.task_id] = task
        self.emit(TaskStatusUpdated(task_id=task.task_id, task_status=TaskStatus.Running))
        self.engine.submit(task)
        if not isinstance(self.status, RunnerRunning):
            self.set_status(RunnerRunning())

    def _finish_generation(self, tid: TaskId, status: TaskStatus) -> None:
        task = self.active.pop(tid, None)
        if task is None:
            return
        if tracing.enabled and self.engine is not None:
            spans = self.engine.collect_traces()
            if spans:
                self.emit(TracesCollected(task_id=tid, rank=self.rank, traces=[
                    TraceEventData(name=s.name, start_us=s.start_us, duration_us=s.duration_us, rank=s.rank,
                                   category=s.category) for s in spans]))
        self._done(task, status)

    def _fail_active(self, message: str) -> None:
        for tid, task in list(self.active.items()):
            if self.rank == 0:
                self.emit(ChunkGenerated(command_id=task.command_id, chunk=ErrorChunk(
                    model=task.task_params.model, error_message=message)))
            self._done(task, TaskStatus.Failed)
        self.active.clear()

    def _pump(self) -> None:
        assert self.engine is not None
        for tid, item in self.engine.step():
            task = self.active.get(tid)
            if task is None:
                continue
            if isinstance(item, Finished):
                self._finish_generation(tid, TaskStatus.Complete)
            elif isinstance(item, Cancelled):
                self._finish_generation(tid, TaskStatus.Cancelled)
            elif self.rank == 0:
                self.emit(ChunkGenerated(command_id=task.command_id, chunk=item))
        if not self.active and isinstance(self.status, RunnerRunning):
            self.set_status(RunnerReady(prefill_server_port=getattr(self.engine, "prefill_server_port", None)))

    # ---- main loop ----
    def _handle(self, task: Task) -> bool:
        """Returns False when the runner should stop."""
        self.emit(TaskAcknowledged(task_id=task.task_id))
        if isinstance(task, Shutdown):
            self.set_status(RunnerShuttingDown())
            self._fail_active("runner shut down")
            self._done(task)
            return False
        if isinstance(task, ConnectToGroup):
            self._connect(task)
        elif isinstance(task, LoadModel):
            if self.single and isinstance(self.status, RunnerIdle):
                self.builder.connect()
            self._load(task)
        elif isinstance(task, StartWarmup):
            self._warmup(task)
        elif isinstance(task, GENERATION):
            self._start_generation(task)
        return True

    def run(self) -> None:
        sh = self.bound.bound_shard
        self.set_status(RunnerIdle())
        if sh.immediate_exception:
            raise RuntimeError("Fake exception - runner failed to spin up (immediate_exception)")
        try:
            while True:
                busy = self.engine is not None and self.engine.has_work
                try:
                    task = self.tasks.receive_nowait() if busy else self.tasks.receive(timeout=self.idle_poll)
                except (TimeoutError, Exception) as e:  # noqa: BLE001 - WouldBlock / timeout: nothing to take
                    if isinstance(e, ChannelClosed):
                        break
                    task = None
                if task is not None and not self._handle(task):
                    break
                for tid in self.cancels.collect():
                    if self.engine is not None:
                        self.engine.cancel(tid)
                if self.engine is not None and self.engine.has_work:
                    self._pump()
        finally:
            try:
                if self.engine is not None:
                    self.engine.close()
                self.builder.close()
            finally:
                self.set_status(RunnerShutdown())
