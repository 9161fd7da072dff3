"""Request parameters, tasks, commands, events and the global ``State``.

Class and field names follow the reference (``src/exo/shared/types/text_generation.py:102-135``,
``tasks.py:24-106``, ``commands.py:20-132``, ``events.py:22-197``, ``state.py:30-94``): these
objects are the inter-node protocol and the content of the persisted event log.
"""
from __future__ import annotations

from collections.abc import Mapping, Sequence
from datetime import datetime
from enum import Enum
from typing import Any, ClassVar, Literal, cast

from pydantic import BaseModel, ConfigDict, Field, field_serializer, field_validator
from pydantic.alias_generators import to_camel

from ..api.types import ImageEditsTaskParams, ImageGenerationTaskParams, ReasoningEffort
from .base import (CommandId, EventId, FrozenModel, InstanceId, InstanceLinkId, ModelId, NodeId, RunnerId, SessionId,
                   SystemId, TaggedModel, TaskId)
from .cards import Backend, ModelCard, card_cache
from .topology import Connection, Topology, TopologySnapshot
from .wire import (BoundInstance, Chunk, DiskUsage, DownloadProgress, GatheredInfo, InputImageChunk, Instance,
                   InstanceLink, InstanceMeta, MemoryUsage, NodeIdentity, NodeNetworkInfo, NodeNvlinkInfo,
                   NodeRdmaCtlStatus, NodeThunderboltInfo, RunnerStatus, Sharding, ShardMetadata,
                   SystemPerformanceProfile, ThunderboltBridgeStatus)

MessageRole = Literal["user", "assistant", "system", "developer", "tool"]


def resolve_reasoning_params(effort: ReasoningEffort | None, thinking: bool | None):
    """``enable_thinking`` and ``reasoning_effort`` imply each other when only one is given."""
    if effort is None and thinking is not None:
        effort = "medium" if thinking else "none"
    if thinking is None and effort is not None:
        thinking = effort != "none"
    return effort, thinking


class InputMessage(BaseModel, frozen=True):
    role: MessageRole
    content: str


class TextGenerationTaskParams(BaseModel, frozen=True):
    """The one internal request shape every API dialect is converted into."""
    model: ModelId
    input: list[InputMessage]
    instructions: str | None = None
    max_output_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    stream: bool = False
    tools: list[dict[str, Any]] | None = None
    bench: bool = False
    use_prefix_cache: bool = False
    top_k: int | None = None
    stop: str | list[str] | None = None
    seed: int | None = None
    chat_template_messages: list[dict[str, Any]] | None = None
    reasoning_effort: ReasoningEffort | None = None
    enable_thinking: bool | None = None
    logprobs: bool = False
    top_logprobs: int | None = None
    min_p: float | None = None
    repetition_penalty: float | None = None
    repetition_context_size: int | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None
    images: list[str] = Field(default_factory=list)
    image_hashes: dict[int, str] = Field(default_factory=dict)
    prefill_endpoint: str | None = None

    def with_card_sampling_defaults(self) -> "TextGenerationTaskParams":
        """Fill unset sampling knobs from the model card (thinking / non-thinking variants first)."""
        card = card_cache.get(self.model)
        if card is None:
            return self
        d = card.sampling_defaults
        vals = d.thinking if (self.enable_thinking is True and d.thinking) else \
            d.non_thinking if (self.enable_thinking is False and d.non_thinking) else d
        upd = {k: getattr(vals, k) for k in ("temperature", "top_p", "top_k", "min_p", "repetition_penalty",
                                              "presence_penalty", "frequency_penalty")
               if getattr(self, k) is None and getattr(vals, k) is not None}
        return self.model_copy(update=upd) if upd else self


# ------------------------------------------------------------------------------------------------
# tasks
# ------------------------------------------------------------------------------------------------
class TaskStatus(str, Enum):
    Pending = "Pending"
    Running = "Running"
    Complete = "Complete"
    TimedOut = "TimedOut"
    Failed = "Failed"
    Cancelled = "Cancelled"


class BaseTask(TaggedModel):
    task_id: TaskId = Field(default_factory=TaskId)
    task_status: TaskStatus = TaskStatus.Pending
    instance_id: InstanceId


class CreateRunner(BaseTask):
    bound_instance: BoundInstance


class DownloadModel(BaseTask):
    shard_metadata: ShardMetadata


class LoadModel(BaseTask): ...
class ConnectToGroup(BaseTask): ...
class StartWarmup(BaseTask): ...


class TextGeneration(BaseTask):
    command_id: CommandId
    task_params: TextGenerationTaskParams
    error_type: str | None = None
    error_message: str | None = None


class CancelTask(BaseTask):
    cancelled_task_id: TaskId
    runner_id: RunnerId


class ImageGeneration(BaseTask):
    command_id: CommandId
    task_params: ImageGenerationTaskParams
    error_type: str | None = None
    error_message: str | None = None


class ImageEdits(BaseTask):
    command_id: CommandId
    task_params: ImageEditsTaskParams
    error_type: str | None = None
    error_message: str | None = None


class Shutdown(BaseTask):
    runner_id: RunnerId


Task = (CreateRunner | DownloadModel | ConnectToGroup | LoadModel | StartWarmup | TextGeneration | CancelTask
        | ImageGeneration | ImageEdits | Shutdown)
GenerationTask = TextGeneration | ImageGeneration | ImageEdits


# ------------------------------------------------------------------------------------------------
# commands (client → master)
# ------------------------------------------------------------------------------------------------
class BaseCommand(TaggedModel):
    command_id: CommandId = Field(default_factory=CommandId)


class TestCommand(BaseCommand):
    __test__ = False


class TextGenerationCommand(BaseCommand):
    __tag__: ClassVar[str] = "TextGeneration"
    task_params: TextGenerationTaskParams


class ImageGenerationCommand(BaseCommand):
    __tag__: ClassVar[str] = "ImageGeneration"
    task_params: ImageGenerationTaskParams


class ImageEditsCommand(BaseCommand):
    __tag__: ClassVar[str] = "ImageEdits"
    task_params: ImageEditsTaskParams


class PlaceInstance(BaseCommand):
    model_card: ModelCard
    sharding: Sharding
    instance_meta: InstanceMeta
    min_nodes: int


class CreateInstance(BaseCommand):
    instance: Instance


class DeleteInstance(BaseCommand):
    instance_id: InstanceId


class TaskCancelled(BaseCommand):
    cancelled_command_id: CommandId


class TaskFinished(BaseCommand):
    finished_command_id: CommandId


class SendInputChunk(BaseCommand):
    chunk: InputImageChunk


class RequestEventLog(BaseCommand):
    since_idx: int


class StartDownload(BaseCommand):
    target_node_id: NodeId
    shard_metadata: ShardMetadata


class DeleteDownload(BaseCommand):
    target_node_id: NodeId
    model_id: ModelId


class CancelDownload(BaseCommand):
    target_node_id: NodeId
    model_id: ModelId


class AddCustomModelCard(BaseCommand):
    model_card: ModelCard


class DeleteCustomModelCard(BaseCommand):
    model_id: ModelId


class SetInstanceLink(BaseCommand):
    link_id: InstanceLinkId
    prefill_instances: list[InstanceId]
    decode_instances: list[InstanceId]


class DeleteInstanceLink(BaseCommand):
    link_id: InstanceLinkId


DownloadCommand = StartDownload | DeleteDownload | CancelDownload
Command = (TestCommand | RequestEventLog | TextGenerationCommand | ImageGenerationCommand | ImageEditsCommand
           | PlaceInstance | CreateInstance | DeleteInstance | TaskCancelled | TaskFinished | SendInputChunk
           | AddCustomModelCard | DeleteCustomModelCard | SetInstanceLink | DeleteInstanceLink)


class ForwarderCommand(FrozenModel):
    origin: SystemId
    command: Command


class ForwarderDownloadCommand(FrozenModel):
    origin: SystemId
    command: DownloadCommand
