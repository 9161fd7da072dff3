"""The cluster's wire model: shards, runners, instances, downloads, chunks, request parameters,
tasks, commands, events and the global ``State``.

One module instead of the reference's dozen (``src/exo/shared/types/*.py``) but the same class and
field names, because these objects ARE the protocol: they travel between nodes as JSON, are
persisted in the event log and are rendered by the dashboard (`/state`).  A "node" is one GPU.
"""
from __future__ import annotations

from collections.abc import Mapping, Sequence
from datetime import datetime
from enum import Enum
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field, field_serializer, field_validator, model_validator
from pydantic.alias_generators import to_camel

from ..api.types import (FinishReason, GenerationStats, ImageEditsTaskParams, ImageGenerationStats,
                         ImageGenerationTaskParams, ToolCallItem, TopLogprobItem, Usage)
from .base import (CommandId, EventId, FrozenModel, Host, Id, InstanceId, InstanceLinkId, Memory, ModelId, NodeId,
                   RunnerId, SessionId, SystemId, TaggedModel, TaskId)
from .cards import Backend, ModelCard, ModelTask
from .topology import Connection, Topology, TopologySnapshot

# ------------------------------------------------------------------------------------------------
# runner diagnostics (classified stderr evidence attached to failures)
# ------------------------------------------------------------------------------------------------


class KnownRunnerDiagnostic(FrozenModel):
    kind: str
    summary: str
    evidence: list[str] = []


# ------------------------------------------------------------------------------------------------
# node telemetry
# ------------------------------------------------------------------------------------------------
class MemoryUsage(FrozenModel):
    ram_total: Memory
    ram_available: Memory
    swap_total: Memory
    swap_available: Memory

    @classmethod
    def from_bytes(cls, *, ram_total: int, ram_available: int, swap_total: int = 0, swap_available: int = 0):
        return cls(ram_total=Memory.from_bytes(ram_total), ram_available=Memory.from_bytes(ram_available),
                   swap_total=Memory.from_bytes(swap_total), swap_available=Memory.from_bytes(swap_available))


class DiskUsage(FrozenModel):
    total: Memory
    available: Memory


class SystemPerformanceProfile(FrozenModel):
    gpu_usage: float = 0.0
    temp: float = 0.0
    sys_power: float = 0.0
    pcpu_usage: float = 0.0
    ecpu_usage: float = 0.0


class NetworkInterfaceInfo(FrozenModel):
    name: str
    ip_address: str
    interface_type: Literal["wifi", "ethernet", "maybe_ethernet", "thunderbolt", "unknown"] = "unknown"


class NodeIdentity(FrozenModel):
    model_id: str = "Unknown"
    chip_id: str = "Unknown"
    friendly_name: str = "Unknown"
    os_version: str = "Unknown"
    os_build_version: str = "Unknown"


class NodeNetworkInfo(FrozenModel):
    interfaces: Sequence[NetworkInterfaceInfo] = []


class ThunderboltIdentifier(FrozenModel):
    rdma_interface: str
    domain_uuid: str
    link_speed: str = ""


class NodeThunderboltInfo(FrozenModel):
    interfaces: Sequence[ThunderboltIdentifier] = []


class NodeRdmaCtlStatus(FrozenModel):
    enabled: bool


class ThunderboltBridgeStatus(FrozenModel):
    enabled: bool
    exists: bool
    service_name: str | None = None


class NvlinkPeer(FrozenModel):
    peer_gpu: int
    links: int = 0
    gbps: float = 0.0          # one-direction copy bandwidth: measured by the link probe, else links x nominal
    p2p: bool = True
    latency_us: float = 0.0    # small peer copy (0: not measured)
    measured: bool = False


class NodeNvlinkInfo(FrozenModel):
    """What NVML and the peer-copy probe say about one GPU's links."""
    gpu_index: int
    uuid: str = ""
    peers: Sequence[NvlinkPeer] = []
    hbm_gbps: float = 0.0      # measured device-copy bandwidth of this GPU's HBM (0: not measured)


# gathered-info messages (what the telemetry task of a node emits)
class StaticNodeInformation(TaggedModel):
    model: str = "Unknown"
    chip: str = "Unknown"
    os_version: str = "Unknown"
    os_build_version: str = "Unknown"


class NodeNetworkInterfaces(TaggedModel):
    ifaces: Sequence[NetworkInterfaceInfo] = []


class NodeMemory(TaggedModel):
    memory: MemoryUsage


class NodePerformance(TaggedModel):
    profile: SystemPerformanceProfile


class NodeDiskUsage(TaggedModel):
    disk_usage: DiskUsage


class MiscData(TaggedModel):
    friendly_name: str = "Unknown"


class NodeBackends(TaggedModel):
    backends: list[Backend] = []


class NodeNvlink(TaggedModel):
    info: NodeNvlinkInfo


class RdmaCtlStatus(TaggedModel):
    enabled: bool = False


GatheredInfo = (StaticNodeInformation | NodeNetworkInterfaces | NodeMemory | NodePerformance | NodeDiskUsage | MiscData
                | NodeBackends | NodeNvlink | RdmaCtlStatus)


# ------------------------------------------------------------------------------------------------
# shards, runners, instances
# ------------------------------------------------------------------------------------------------
class Sharding(str, Enum):
    Tensor = "Tensor"
    Pipeline = "Pipeline"


class BaseShardMetadata(TaggedModel):
    """A slice of a model bound to a device rank; layers are the half-open range [start, end)."""
    model_card: ModelCard
    device_rank: int
    world_size: int
    immediate_exception: bool = False       # fault-injection hook: runner raises on start
    should_timeout: float | None = None     # fault-injection hook: runner sleeps this long in connect
    start_layer: int = Field(ge=0)
    end_layer: int = Field(ge=0)
    n_layers: int = Field(ge=0)
    # engine placement chosen by the planner (extra to the reference's fields)
    tp_size: int = 1
    tp_rank: int = 0
    pp_size: int = 1
    pp_rank: int = 0
    gpu_index: int | None = None

    @property
    def is_first_layer(self) -> bool:
        return self.start_layer == 0

    @property
    def is_last_layer(self) -> bool:
        return self.end_layer == self.n_layers

    def __hash__(self) -> int:
        return hash((self.model_card.model_id, self.start_layer, self.end_layer, self.n_layers, self.device_rank,
                     self.world_size))


class PipelineShardMetadata(BaseShardMetadata): ...
class TensorShardMetadata(BaseShardMetadata): ...


class CfgShardMetadata(BaseShardMetadata):
    cfg_rank: int
    cfg_world_size: int = 2
    pipeline_rank: int
    pipeline_world_size: int


ShardMetadata = PipelineShardMetadata | CfgShardMetadata | TensorShardMetadata


class RunnerError(Exception):
    pass


class BaseRunnerStatus(TaggedModel):
    def is_running(self) -> bool:
        return isinstance(self, RunnerRunning)


class RunnerIdle(BaseRunnerStatus): ...
class RunnerConnecting(BaseRunnerStatus): ...
class RunnerConnected(BaseRunnerStatus): ...


class RunnerLoading(BaseRunnerStatus):
    layers_loaded: int = 0
    total_layers: int = 0


class RunnerLoaded(BaseRunnerStatus): ...
class RunnerWarmingUp(BaseRunnerStatus): ...


class RunnerReady(BaseRunnerStatus):
    prefill_server_port: int | None = None


class RunnerRunning(BaseRunnerStatus): ...
class RunnerShuttingDown(BaseRunnerStatus): ...
class RunnerShutdown(BaseRunnerStatus): ...


class RunnerFailed(BaseRunnerStatus):
    error_message: str | None = None
    diagnostics: list[KnownRunnerDiagnostic] = []


RunnerStatus = (RunnerIdle | RunnerConnecting | RunnerConnected | RunnerLoading | RunnerLoaded | RunnerWarmingUp
                | RunnerReady | RunnerRunning | RunnerShuttingDown | RunnerShutdown | RunnerFailed)


class ShardAssignments(FrozenModel):
    model_id: ModelId
    runner_to_shard: Mapping[RunnerId, ShardMetadata]
    node_to_runner: Mapping[NodeId, RunnerId]

    @model_validator(mode="after")
    def _runners_exist(self) -> "ShardAssignments":
        for r in self.node_to_runner.values():
            if r not in self.runner_to_shard:
                raise ValueError(f"Runner {r} in node_to_runner does not exist in runner_to_shard")
        return self


class InstanceMeta(str, Enum):
    MlxRing = "MlxRing"     # accepted for request compatibility; both map onto the NVLink backend
    MlxJaccl = "MlxJaccl"
    Nvlink = "Nvlink"


class BaseInstance(TaggedModel):
    instance_id: InstanceId
    shard_assignments: ShardAssignments

    def shard(self, runner_id: RunnerId) -> ShardMetadata | None:
        return self.shard_assignments.runner_to_shard.get(runner_id)


class MlxRingInstance(BaseInstance):
    hosts_by_node: dict[NodeId, list[Host]]
    ephemeral_port: int


class MlxJacclInstance(BaseInstance):
    jaccl_devices: list[list[str | None]]
    jaccl_coordinators: dict[NodeId, str]


class NvlinkInstance(BaseInstance):
    """One model placed on GPUs of this box: ranks rendezvous on 127.0.0.1:``rendezvous_port``."""
    rendezvous_port: int
    gpu_by_node: dict[NodeId, int]
    parallelism: str = "tp1"      # e.g. "tp8", "pp2xtp4", "tp8+ep8"


Instance = MlxRingInstance | MlxJacclInstance | NvlinkInstance


class BoundInstance(FrozenModel):
    instance: Instance
    bound_runner_id: RunnerId
    bound_node_id: NodeId

    @property
    def bound_shard(self) -> ShardMetadata:
        s = self.instance.shard(self.bound_runner_id)
        assert s is not None
        return s

    @property
    def is_image_model(self) -> bool:
        t = self.bound_shard.model_card.tasks
        return ModelTask.TextToImage in t or ModelTask.ImageToImage in t

    @model_validator(mode="after")
    def _bound(self) -> "BoundInstance":
        assert self.bound_runner_id in self.instance.shard_assignments.runner_to_shard, \
            "Bound Instance must be constructed with a runner_id that is in the instances assigned shards"
        return self


class InstanceLink(FrozenModel):
    link_id: InstanceLinkId
    prefill_instances: list[InstanceId]
    decode_instances: list[InstanceId]


# ------------------------------------------------------------------------------------------------
# downloads
# ------------------------------------------------------------------------------------------------
class DownloadProgressData(FrozenModel):
    total: Memory
    downloaded: Memory
    downloaded_this_session: Memory
    completed_files: int
    total_files: int
    speed: float
    eta_ms: int
    files: dict[str, "DownloadProgressData"]


class BaseDownloadProgress(TaggedModel):
    node_id: NodeId
    shard_metadata: ShardMetadata
    model_directory: str = ""


class DownloadPending(BaseDownloadProgress):
    downloaded: Memory = Memory()
    total: Memory = Memory()


class DownloadCompleted(BaseDownloadProgress):
    total: Memory
    read_only: bool = False


class DownloadFailed(BaseDownloadProgress):
    error_message: str


class DownloadOngoing(BaseDownloadProgress):
    download_progress: DownloadProgressData


DownloadProgress = DownloadPending | DownloadCompleted | DownloadFailed | DownloadOngoing


# ------------------------------------------------------------------------------------------------
# chunks (what a runner streams back for a command)
# ------------------------------------------------------------------------------------------------
class BaseChunk(TaggedModel):
    model: ModelId


class TokenChunk(BaseChunk):
    text: str
    token_id: int
    usage: Usage | None
    finish_reason: Literal["stop", "length", "content_filter"] | None = None
    stats: GenerationStats | None = None
    logprob: float | None = None
    top_logprobs: list[TopLogprobItem] | None = None
    is_thinking: bool = False


class ErrorChunk(BaseChunk):
    error_message: str
    finish_reason: Literal["error"] = "error"
    diagnostics: list[KnownRunnerDiagnostic] = []


class ToolCallChunk(BaseChunk):
    tool_calls: list[ToolCallItem]
    usage: Usage | None
    finish_reason: Literal["tool_calls"] = "tool_calls"
    stats: GenerationStats | None = None


class ImageChunk(BaseChunk):
    data: str
    chunk_index: int
    total_chunks: int
    image_index: int
    is_partial: bool = False
    partial_index: int | None = None
    total_partials: int | None = None
    stats: ImageGenerationStats | None = None
    format: Literal["png", "jpeg", "webp"] | None = None
    finish_reason: FinishReason | None = None
    error_message: str | None = None


class InputImageChunk(BaseChunk):
    command_id: CommandId
    data: str
    chunk_index: int
    total_chunks: int
    image_index: int = 0


class PrefillProgressChunk(BaseChunk):
    processed_tokens: int
    total_tokens: int


GenerationChunk = TokenChunk | ImageChunk | ToolCallChunk | ErrorChunk
Chunk = PrefillProgressChunk | GenerationChunk
