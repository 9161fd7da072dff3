"""Parent side of a runner: spawn the child, relay its events, notice its death.

The runner owns a GPU context, so it lives in its own process: a CUDA fault or an OOM kills only
that process and the supervisor turns the death into ``RunnerFailed`` plus one ``ErrorChunk`` per
in-flight request (reference ``src/exo/worker/runner/supervisor.py:202-440``: three multiprocessing
channels — events up, tasks down, cancels down —, ``start_task`` returns once the child has
acknowledged, liveness poll every 5 s, stdout/stderr mirrored into the runner logs).
"""
from __future__ import annotations

import os
from collections.abc import Callable

import anyio

from ...shared import constants
from ...shared.base import TaskId
from ...shared.events import (ChunkGenerated, Event, RunnerStatusUpdated, TaskAcknowledged, TaskStatusUpdated)
from ...shared.messages import GenerationTask, ImageEdits, ImageGeneration, Task, TaskStatus, TextGeneration
from ...shared.wire import BoundInstance, ErrorChunk, RunnerFailed, RunnerIdle, RunnerShutdown, RunnerStatus
from ...utils.async_process import AsyncProcess
from ...utils.channels import ChannelClosed, MpReceiver, MpSender, Sender, mp_channel
from .bootstrap import entrypoint
from .diagnostics import DiagnosticCollector, cause_from_exit

GENERATION = (TextGeneration, ImageGeneration, ImageEdits)
LIVENESS_POLL = 5.0


class RunnerSupervisor:
    def __init__(self, bound_instance: BoundInstance, event_sender: Sender[Event], process: AsyncProcess,
                 ev_recv: MpReceiver[Event], task_send: MpSender[Task], cancel_send: MpSender[TaskId]):
        self.bound_instance = bound_instance
        self.status: RunnerStatus = RunnerIdle()
        self.completed: set[TaskId] = set()
        self.in_progress: set[TaskId] = set()
        self.cancelled: set[TaskId] = set()
        self.pending_acks: dict[TaskId, anyio.Event] = {}
        self.tasks: dict[TaskId, Task] = {}
        self._events_out, self._proc = event_sender, process
        self._ev_recv, self._task_send, self._cancel_send = ev_recv, task_send, cancel_send
        self._diag = DiagnosticCollector()
        self._dead = False
        self._follower = bound_instance.bound_shard.device_rank != 0
        self._events_done = anyio.Event()
        self._tg: anyio.abc.TaskGroup | None = None

    @classmethod
    def create(cls, bound_instance: BoundInstance, event_sender: Sender[Event],
               target: Callable[..., None] = entrypoint) -> "RunnerSupervisor":
        ev_s, ev_r = mp_channel()
        task_s, task_r = mp_channel()
        cancel_s, cancel_r = mp_channel()
        proc = AsyncProcess(target, (bound_instance, ev_s, task_r, cancel_r),
                            name=f"runner-{bound_instance.bound_runner_id[:8]}")
        return cls(bound_instance, event_sender, proc, ev_r, task_s, cancel_s)

    # ---- pumps ----
    async def _pump_stream(self, lines, path, is_err: bool) -> None:
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            f = open(path, "a")
        except OSError:
            f = None
        try:
            async for ln in lines:
                if is_err:
                    self._diag.feed(ln)
                if f is not None:
                    f.write(ln + "\n")
                    f.flush()
        finally:
            if f is not None:
                f.close()

    async def _forward_events(self) -> None:
        try:
            await self._forward_events_inner()
        finally:
            self._events_done.set()

    async def _forward_events_inner(self) -> None:
        while True:
            try:
                ev = await self._ev_recv.receive_async()
            except ChannelClosed:
                return
            if isinstance(ev, RunnerStatusUpdated):
                self.status = ev.runner_status
            elif isinstance(ev, TaskAcknowledged):
                self.in_progress.add(ev.task_id)
                w = self.pending_acks.pop(ev.task_id, None)
                if w is not None:
                    w.set()
            elif isinstance(ev, TaskStatusUpdated) and ev.task_status in (TaskStatus.Complete, TaskStatus.Failed,
                                                                          TaskStatus.Cancelled, TaskStatus.TimedOut):
                self.in_progress.discard(ev.task_id)
                self.completed.add(ev.task_id)
            if isinstance(ev, TaskStatusUpdated) and self._follower and ev.task_status != TaskStatus.Failed \
                    and isinstance(self.tasks.get(ev.task_id), GENERATION):
                # rank 0 speaks for the instance: a follower that starts or ends a generation early must not flip
                # the cluster-wide task status under the other ranks' planners
                continue
            await self._events_out.send(ev)

    async def _watch(self) -> None:
        while self._proc.is_alive():
            await anyio.sleep(min(LIVENESS_POLL, 0.25))
        with anyio.move_on_after(1.0):      # what the child said last (its final status) decides clean vs failed
            await self._events_done.wait()
        await self._on_death()

    async def _on_death(self) -> None:
        if self._dead:
            return
        self._dead = True
        code = self._proc.exitcode
        clean = isinstance(self.status, RunnerShutdown) and code == 0
        for w in self.pending_acks.values():
            w.set()
        self.pending_acks.clear()
        if clean:
            return
        await anyio.sleep(0.05)  # let the stderr pump drain the traceback
        diags = self._diag.diagnostics()
        tail = " | ".join(list(self._diag.context)[-2:])
        msg = f"{cause_from_exit(code)}" + (f": {tail}" if tail else "")
        for tid in list(self.in_progress):
            t = self.tasks.get(tid)
            if isinstance(t, GENERATION) and self.bound_instance.bound_shard.device_rank == 0:
                await self._events_out.send(ChunkGenerated(command_id=t.command_id, chunk=ErrorChunk(
                    model=t.task_params.model, error_message=msg, diagnostics=diags)))
            await self._events_out.send(TaskStatusUpdated(task_id=tid, task_status=TaskStatus.Failed))
        self.in_progress.clear()
        self.status = RunnerFailed(error_message=msg, diagnostics=diags)
        await self._events_out.send(RunnerStatusUpdated(runner_id=self.bound_instance.bound_runner_id,
                                                        runner_status=self.status))

    # ---- API used by the worker ----
    async def run(self) -> None:
        self._proc.start()
        async with anyio.create_task_group() as tg:
            self._tg = tg
            tg.start_soon(self._pump_stream, self._proc.stdout_lines(), constants.EXO_RUNNER_STDOUT_LOG, False)
            tg.start_soon(self._pump_stream, self._proc.stderr_lines(), constants.EXO_RUNNER_STDERR_LOG, True)
            tg.start_soon(self._forward_events)
            await self._watch()
            await anyio.sleep(0.1)
            tg.cancel_scope.cancel()

    async def start_task(self, task: Task, ack_timeout: float = 30.0) -> bool:
        """Hand a task to the child; returns once it acknowledged (or died)."""
        if self._dead:
            return False
        self.tasks[task.task_id] = task
        w = anyio.Event()
        self.pending_acks[task.task_id] = w
        await self._task_send.send_async(task)
        with anyio.move_on_after(ack_timeout):
            await w.wait()
        return task.task_id in self.in_progress or task.task_id in self.completed

    async def cancel_task(self, task_id: TaskId) -> None:
        self.cancelled.add(task_id)
        if not self._dead:
            await self._cancel_send.send_async(task_id)

    async def shutdown(self, grace: float = 3.0) -> None:
        with anyio.move_on_after(grace):
            while self._proc.is_alive():
                await anyio.sleep(0.05)
        if self._proc.is_alive():
            await self._proc.stop()
        with anyio.move_on_after(1.0):      # let the child's last events (its final status) through before stopping the pumps
            await self._events_done.wait()
        if self._tg is not None:
            self._tg.cancel_scope.cancel()
