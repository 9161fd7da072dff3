"""A deterministic engine without a model, for control-plane tests and dry runs.

It plays the part the reference's tests give to a monkey-patched MLX (fake group, fake loader,
fake warm-up: ``src/exo/worker/tests/unittests/test_runner/test_event_ordering.py:123-140``) and
implements the reference's host-side fault hooks: the magic prompts ``EXO RUNNER MUST FAIL`` /
``MUST OOM`` / ``MUST TIMEOUT`` (``src/exo/worker/runner/llm_inference/batch_generator.py:67-86``;
the OOM is a simulated allocation failure, never a real device allocation), plus ``MUST LOSE A PEER``: the
exception the GPU executor raises when a collective kernel's bounded wait on a peer ran out.
"""
from __future__ import annotations

import time
from collections.abc import Iterable, Iterator

from ...api.types import CompletionTokensDetails, PromptTokensDetails, Usage
from ...shared.base import TaskId
from ...shared.messages import GenerationTask, TextGeneration
from ...shared.wire import TokenChunk
from .base import Builder, Cancelled, Engine, Finished, LoadProgress, StepItem


class FakeEngine(Engine):
    def __init__(self, model_id: str, rank: int = 0, tokens_per_request: int = 4):
        self.model_id, self.rank, self.n = model_id, rank, tokens_per_request
        self.active: dict[TaskId, int] = {}
        self.cancelled: set[TaskId] = set()

    def warmup(self) -> None:
        pass

    def submit(self, task: GenerationTask) -> None:
        if isinstance(task, TextGeneration):
            text = " ".join(m.content for m in task.task_params.input)
            if "EXO RUNNER MUST FAIL" in text:
                raise RuntimeError("Artificial runner exception (requested by prompt)")
            if "EXO RUNNER MUST OOM" in text:
                raise MemoryError("Simulated allocation failure (requested by prompt)")
            if "EXO RUNNER MUST TIMEOUT" in text:
                time.sleep(3600)
            if "EXO RUNNER MUST LOSE A PEER" in text:
                self.lose_peer = True
        self.active[task.task_id] = 0

    def cancel(self, task_id: TaskId) -> None:
        if task_id in self.active:
            self.cancelled.add(task_id)

    @property
    def has_work(self) -> bool:
        return bool(self.active)

    def step(self) -> Iterable[tuple[TaskId, StepItem]]:
        if getattr(self, "lose_peer", False):
            # what the B200 executor raises after a step whose collective kernel gave up waiting for a peer GPU
            # (host-side stand-in: no device is involved)
            from ...ops.cuda import DeviceWaitTimeout
            raise DeviceWaitTimeout("cuda:0: a collective kernel gave up waiting for a peer GPU (code 4)")
        out: list[tuple[TaskId, StepItem]] = []
        for tid in list(self.active):
            if tid in self.cancelled:
                self.cancelled.discard(tid)
                del self.active[tid]
                out.append((tid, Cancelled()))
                continue
            i = self.active[tid]
            last = i == self.n - 1
            if self.rank == 0:
                usage = Usage(prompt_tokens=1, completion_tokens=i + 1, total_tokens=i + 2,
                              prompt_tokens_details=PromptTokensDetails(), completion_tokens_details=CompletionTokensDetails())
                out.append((tid, TokenChunk(model=self.model_id, text=f"tok{i} ", token_id=i, usage=usage,
                                            finish_reason="stop" if last else None)))
            if last:
                del self.active[tid]
                out.append((tid, Finished()))
            else:
                self.active[tid] = i + 1
        return out


class FakeBuilder(Builder):
    def connect(self) -> None:
        sh = self.bound_instance.bound_shard
        if sh.should_timeout:
            time.sleep(sh.should_timeout)

    def load(self) -> Iterator[LoadProgress]:
        sh = self.bound_instance.bound_shard
        total = sh.end_layer - sh.start_layer
        for i in range(1, total + 1, max(1, total // 4)):
            yield LoadProgress(min(i, total), total)
        yield LoadProgress(total, total)

    def build(self) -> Engine:
        sh = self.bound_instance.bound_shard
        return FakeEngine(str(sh.model_card.model_id), sh.device_rank)
