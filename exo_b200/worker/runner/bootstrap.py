"""Entry point of the runner child process.

Chooses the engine builder, runs the ``Runner`` state machine, and converts any exception into a
traceback on stderr plus a non-zero exit so that the supervisor can report ``RunnerFailed``
(reference ``src/exo/worker/runner/bootstrap.py:18-97``).  The child raises its file-descriptor
limit and pins itself to its GPU before any CUDA call.
"""
from __future__ import annotations

import os
import resource
import sys
import traceback

from ...shared.base import TaskId
from ...shared.events import Event
from ...shared.messages import Task
from ...shared.wire import BoundInstance
from ...utils.channels import MpReceiver, MpSender


class RunnerTerminationError(Exception):
    def __init__(self, message: str, tb: str):
        super().__init__(message)
        self.tb = tb


def make_builder(bound: BoundInstance):
    kind = os.environ.get("EXO_ENGINE", "b200")
    if kind == "fake":
        from ..engines.fake import FakeBuilder
        return FakeBuilder(bound)
    if bound.is_image_model:
        from ..engines.image.builder import ImageBuilder
        return ImageBuilder(bound)
    from ..engines.b200.bringup import B200Builder
    return B200Builder(bound)


def entrypoint(bound: BoundInstance, events: MpSender[Event], tasks: MpReceiver[Task], cancels: MpReceiver[TaskId]) -> None:
    try:
        soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
        resource.setrlimit(resource.RLIMIT_NOFILE, (min(max(soft, 65535), hard), hard))
    except (ValueError, OSError):
        pass
    gpu = bound.bound_shard.gpu_index
    if gpu is not None:
        os.environ.setdefault("EXO_GPU_INDEX", str(gpu))
    from .runner import Runner
    try:
        Runner(bound, make_builder(bound), events, tasks, cancels).run()
    except BaseException as e:  # noqa: BLE001 - the process is about to exit: report everything
        tb = traceback.format_exc()
        sys.stderr.write(tb)
        sys.stderr.flush()
        events.close()
        raise SystemExit(1) from RunnerTerminationError(str(e), tb)
    events.close()
