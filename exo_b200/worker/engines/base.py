"""Engine contract between the runner state machine and an inference backend.

Same two roles as the reference (``src/exo/worker/engines/base.py:16-60``): a ``Builder`` walks the
bring-up steps (connect to the rank group → load the shard, reporting progress → build), an
``Engine`` serves (warm up, submit, step, cancel, close).  ``step()`` yields ``(task_id, item)``
pairs where ``item`` is a chunk to stream, ``Finished`` or ``Cancelled``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from collections.abc import Iterable, Iterator
from dataclasses import dataclass

from ...shared.base import TaskId
from ...shared.messages import GenerationTask
from ...shared.wire import BoundInstance, Chunk


@dataclass(frozen=True)
class LoadProgress:
    layers_loaded: int
    total_layers: int


@dataclass(frozen=True)
class Finished:
    pass


@dataclass(frozen=True)
class Cancelled:
    pass


StepItem = Chunk | Finished | Cancelled


class Engine(ABC):
    @abstractmethod
    def warmup(self) -> None: ...

    @abstractmethod
    def submit(self, task: GenerationTask) -> None: ...

    @abstractmethod
    def step(self) -> Iterable[tuple[TaskId, StepItem]]: ...

    @abstractmethod
    def cancel(self, task_id: TaskId) -> None: ...

    @property
    @abstractmethod
    def has_work(self) -> bool: ...

    def close(self) -> None:
        pass

    def serve_prefill(self, request: object) -> None:  # prefill/decode disaggregation hook
        raise NotImplementedError

    def collect_traces(self) -> list:
        return []


class Builder(ABC):
    def __init__(self, bound_instance: BoundInstance):
        self.bound_instance = bound_instance

    @abstractmethod
    def connect(self) -> None: ...

    @abstractmethod
    def load(self) -> Iterator[LoadProgress]: ...

    @abstractmethod
    def build(self) -> Engine: ...

    def close(self) -> None:
        pass
