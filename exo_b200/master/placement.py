"""Placement planner: which GPUs run a model, and as what kind of shards.

The reference plans over Macs linked by Thunderbolt: candidates are simple cycles of the
topology graph, filtered by memory, tensor-divisibility, backend and RDMA capability, smallest
cycle first, ties broken by download progress and free memory (``src/exo/master/placement.py:
106-311``; layer split by free-memory fraction ``placement_utils.py:47-122``).  Here a node is a
B200 behind NVSwitch, every pair is one hop, so a candidate is simply "the n GPUs with the most
free HBM that are all NVLink peers", and the interesting decision is the *shape*: pure TP-n, or
PP2 × TP-n/2, chosen with a small cost model fed by the measured NVLink bandwidth and the HBM
each GPU has free.  The filter order and the error strings the API shows in placement previews
follow the reference.
"""
from __future__ import annotations

import random
from collections.abc import Mapping, Sequence
from copy import deepcopy

from ..shared.base import InstanceId, Memory, ModelId, NodeId, RunnerId, TaskId
from ..shared.cards import Backend, ModelCard
from ..shared.events import Event, InstanceCreated, InstanceDeleted, TaskStatusUpdated
from ..shared.messages import (DeleteInstance, GenerationTask, PlaceInstance, Task, TaskStatus, TextGeneration,
                               ImageGeneration, ImageEdits)
from ..shared.topology import Topology
from ..shared.wire import (CfgShardMetadata, DownloadCompleted, DownloadOngoing, DownloadProgress, Instance,
                           InstanceMeta, MemoryUsage, NvlinkInstance, PipelineShardMetadata, ShardAssignments, Sharding,
                           ShardMetadata, TensorShardMetadata)

# Fallbacks of the cost model, used until the nodes' link probes have reported (``utils.link_probe``: device-copy
# bandwidth of each GPU's HBM, copy bandwidth and small-copy latency to each peer):
HBM_GBS = 6500.0              # per-GPU streaming bandwidth
AR_LATENCY_US = 6.0           # one small fused all-reduce over NVSwitch
P2P_HOP_US = 12.0             # one pipeline activation hop
MEMORY_HEADROOM = 0.92        # fraction of free HBM a shard may claim (KV pool comes out of the rest)
KV_RESERVE_FRACTION = 0.10    # at least this share of a GPU stays free for KV blocks


def random_ephemeral_port() -> int:
    return random.randint(49152, 65535)


def allocate_layers_proportionally(total_layers: int, fractions: Sequence[float]) -> list[int]:
    """Largest-remainder split of ``total_layers`` by weight, at least one layer each."""
    n = len(fractions)
    if n == 0 or total_layers < n:
        raise ValueError(f"Cannot assign {total_layers} layers to {n} stages")
    s = sum(fractions) or 1.0
    raw = [f / s * total_layers for f in fractions]
    base = [max(1, int(x)) for x in raw]
    while sum(base) > total_layers:
        i = max(range(n), key=lambda k: base[k] - raw[k] if base[k] > 1 else -1e9)
        base[i] -= 1
    order = sorted(range(n), key=lambda k: raw[k] - int(raw[k]), reverse=True)
    k = 0
    while sum(base) < total_layers:
        base[order[k % n]] += 1
        k += 1
    return base


def estimate_decode_step_us(card: ModelCard, tp: int, pp: int, nvlink_gbps: float, batch: int = 1,
                            hbm_gbps: float = 0.0, link_latency_us: float = 0.0) -> float:
    """Rough decode-step latency of a (tp, pp) shape: weight streaming + collectives + stage hops.  ``hbm_gbps`` and
    ``link_latency_us`` are the measured figures of the chosen GPUs (0: use the fallbacks above)."""
    bytes_per_gpu = card.storage_size.in_bytes / (tp * pp)
    stream_us = bytes_per_gpu / ((hbm_gbps or HBM_GBS) * 1e3)             # GB/s → bytes/us
    per_stage = stream_us
    ar_bytes = 2 * batch * card.hidden_size
    link = max(nvlink_gbps, 1.0) * 1e3
    # a small collective is one one-way trip of the pushed words (plus the consumer's poll): the measured small-copy
    # latency stands in for it when the probe has run
    ar_fixed = link_latency_us or AR_LATENCY_US
    ar_us = 0.0 if tp == 1 else ar_fixed + ar_bytes * (tp - 1) / link
    layers_per_stage = card.n_layers / pp
    per_stage += 2 * layers_per_stage * ar_us
    # decode walks the stages one after the other
    return pp * per_stage + (pp - 1) * max(P2P_HOP_US, 2 * link_latency_us)


def is_moe_card(card: ModelCard) -> bool:
    """Mixture-of-experts models name their active parameter count in the model id (``-A22B``, ``-A3B``) or are of a
    family that has no dense members; their experts are spread over the tensor-parallel ranks."""
    import re
    name = f"{card.model_id} {card.base_model}"
    return (bool(re.search(r"-A\d+(\.\d+)?B\b", name, re.IGNORECASE)) or card.family in ("deepseek", "kimi", "minimax", "glm", "step")
            or "MoE" in name or "Coder-Next" in name or "gpt-oss" in name.lower())


def _tensor_ok(card: ModelCard, n: int) -> bool:
    kv = card.num_key_value_heads
    # KV heads are replicated when there are fewer of them than ranks, so n may exceed kv if it divides evenly
    return card.hidden_size % n == 0 and (kv is None or kv % n == 0 or n % kv == 0)


def _download_score(nodes: Sequence[NodeId], model_id: ModelId,
                    downloads: Mapping[NodeId, Sequence[DownloadProgress]]) -> float:
    score = 0.0
    for n in nodes:
        for dp in downloads.get(n, ()):
            if dp.shard_metadata.model_card.model_id != model_id:
                continue
            if isinstance(dp, DownloadCompleted):
                score += 1.0
            elif isinstance(dp, DownloadOngoing) and dp.download_progress.total.in_bytes:
                score += dp.download_progress.downloaded.in_bytes / dp.download_progress.total.in_bytes
    return score


def _fits(card: ModelCard, nodes: Sequence[NodeId], node_memory: Mapping[NodeId, MemoryUsage]) -> bool:
    share = card.storage_size.in_bytes / len(nodes)
    for n in nodes:
        mem = node_memory.get(n)
        if mem is None:
            return False
        if share > mem.ram_available.in_bytes * MEMORY_HEADROOM - mem.ram_total.in_bytes * KV_RESERVE_FRACTION:
            return False
    return True


def candidate_groups(topology: Topology, node_memory: Mapping[NodeId, MemoryUsage], min_nodes: int,
                     required_nodes: set[NodeId] | None = None) -> list[list[NodeId]]:
    """For every group size, the GPUs with the most free memory that are mutual NVLink peers."""
    nodes = [n for n in topology.list_nodes() if n in node_memory]
    nodes.sort(key=lambda n: node_memory[n].ram_available.in_bytes, reverse=True)
    out: list[list[NodeId]] = []
    for size in range(max(1, min_nodes), len(nodes) + 1):
        if size > 1 and size not in (2, 4, 8, 16):
            continue
        group: list[NodeId] = list(required_nodes or ())
        for n in nodes:
            if len(group) == size:
                break
            if n in group:
                continue
            if all(topology.get_all_connections_between(n, g) and topology.get_all_connections_between(g, n) for g in group):
                group.append(n)
        if len(group) == size:
            out.append(group)
    return out


def get_shard_assignments(card: ModelCard, nodes: Sequence[NodeId], sharding: Sharding, tp: int, pp: int,
                          node_memory: Mapping[NodeId, MemoryUsage], gpu_index: Mapping[NodeId, int]) -> ShardAssignments:
    world = len(nodes)
    assert tp * pp == world
    r2s: dict[RunnerId, ShardMetadata] = {}
    n2r: dict[NodeId, RunnerId] = {}
    stage_mem = [sum(node_memory[nodes[s * tp + t]].ram_available.in_bytes for t in range(tp)) for s in range(pp)]
    layers = allocate_layers_proportionally(card.n_layers, [float(m) for m in stage_mem])
    start = 0
    for s in range(pp):
        for t in range(tp):
            rank = s * tp + t
            node = nodes[rank]
            cls = TensorShardMetadata if pp == 1 else PipelineShardMetadata
            if card.uses_cfg and card.is_image and world % 2 == 0 and pp == world:
                half = world // 2
                sm: ShardMetadata = CfgShardMetadata(
                    model_card=card, device_rank=rank, world_size=world, start_layer=start, end_layer=start + layers[s],
                    n_layers=card.n_layers, cfg_rank=rank // half, pipeline_rank=rank % half, pipeline_world_size=half,
                    tp_size=tp, tp_rank=t, pp_size=pp, pp_rank=s, gpu_index=gpu_index.get(node))
            else:
                sm = cls(model_card=card, device_rank=rank, world_size=world, start_layer=start,
                         end_layer=start + layers[s], n_layers=card.n_layers, tp_size=tp, tp_rank=t, pp_size=pp,
                         pp_rank=s, gpu_index=gpu_index.get(node))
            rid = RunnerId()
            r2s[rid] = sm
            n2r[node] = rid
        start += layers[s]
    return ShardAssignments(model_id=card.model_id, runner_to_shard=r2s, node_to_runner=n2r)


def choose_shape(card: ModelCard, n: int, sharding: Sharding, nvlink_gbps: float, hbm_gbps: float = 0.0,
                 link_latency_us: float = 0.0) -> tuple[int, int]:
    """(tp, pp) for ``n`` GPUs.  Tensor requests may fall back to PP2 x TP-n/2 when the cost model
    says the halved all-reduce fan-in wins; Pipeline requests keep pure layer stages."""
    if n == 1:
        return 1, 1
    if sharding == Sharding.Pipeline:
        return 1, n
    shapes = [(n, 1)]
    if n >= 4 and n % 2 == 0 and _tensor_ok(card, n // 2):
        shapes.append((n // 2, 2))
    shapes = [s for s in shapes if _tensor_ok(card, s[0])]
    if not shapes:
        raise ValueError("no tensor-parallel shape divides this model")
    return min(shapes, key=lambda s: estimate_decode_step_us(card, s[0], s[1], nvlink_gbps, 1, hbm_gbps, link_latency_us))


def place_instance(command: PlaceInstance, topology: Topology, current_instances: Mapping[InstanceId, Instance],
                   node_memory: Mapping[NodeId, MemoryUsage], node_backends: Mapping[NodeId, list[Backend]],
                   required_nodes: set[NodeId] | None = None,
                   download_status: Mapping[NodeId, Sequence[DownloadProgress]] | None = None,
                   gpu_index: Mapping[NodeId, int] | None = None,
                   node_nvlink: Mapping[NodeId, object] | None = None) -> dict[InstanceId, Instance]:
    """``node_nvlink`` (``State.node_nvlink``) carries each GPU's link-probe figures for the cost model."""
    card = command.model_card
    groups = candidate_groups(topology, node_memory, command.min_nodes, required_nodes)
    groups = [g for g in groups if _fits(card, g, node_memory)]
    if not groups:
        raise ValueError("No cycles found with sufficient memory")
    if command.sharding == Sharding.Tensor:
        if not card.supports_tensor:
            raise ValueError(f"Requested Tensor sharding but this model does not support tensor parallelism: {card.model_id}")
        groups = [g for g in groups if _tensor_ok(card, len(g))]
        if not groups:
            kv = card.num_key_value_heads
            raise ValueError(f"No tensor sharding found for model with hidden_size={card.hidden_size}"
                             f"{f', num_key_value_heads={kv}' if kv is not None else ''} across candidate cycles")
    else:
        groups = [g for g in groups if len(g) <= card.n_layers]
    if Backend.B200 not in card.backends and Backend.MlxCuda not in card.backends:
        raise ValueError(f"Model {card.model_id} backends {sorted(b.value for b in card.backends)} cannot satisfy engine "
                         f"{command.instance_meta.value} which requires ['B200']")
    groups = [g for g in groups if all(Backend.B200 in node_backends.get(n, []) for n in g)]
    if not groups:
        raise ValueError(f"No cycle where every node supports a backend in ['B200'] for {card.model_id}")
    smallest = min(len(g) for g in groups)
    groups = [g for g in groups if len(g) == smallest]
    dl = download_status or {}
    chosen = max(groups, key=lambda g: (_download_score(g, card.model_id, dl),
                                        sum(node_memory[n].ram_available.in_bytes for n in g)))
    sharding = command.sharding if len(chosen) > 1 else Sharding.Pipeline
    infos = [node_nvlink[n] for n in chosen if node_nvlink and n in node_nvlink]
    hbm = min((i.hbm_gbps for i in infos if getattr(i, "hbm_gbps", 0.0)), default=0.0)
    lat = max((p.latency_us for i in infos for p in getattr(i, "peers", []) if getattr(p, "measured", False)), default=0.0)
    tp, pp = choose_shape(card, len(chosen), sharding, topology.min_nvlink_gbps(chosen) if len(chosen) > 1 else 0.0, hbm, lat)
    gidx = dict(gpu_index or {})
    assignments = get_shard_assignments(card, chosen, sharding, tp, pp, node_memory, gidx)
    iid = InstanceId()
    target = dict(deepcopy(dict(current_instances)))
    shape = f"tp{tp}" if pp == 1 else (f"pp{pp}" if tp == 1 else f"pp{pp}xtp{tp}")
    if is_moe_card(card) and tp > 1:
        shape += f"+ep{tp}"
    target[iid] = NvlinkInstance(instance_id=iid, shard_assignments=assignments, rendezvous_port=random_ephemeral_port(),
                                 gpu_by_node={n: gidx.get(n, i) for i, n in enumerate(chosen)}, parallelism=shape)
    return target


def delete_instance(command: DeleteInstance, current_instances: Mapping[InstanceId, Instance]) -> dict[InstanceId, Instance]:
    target = dict(deepcopy(dict(current_instances)))
    if command.instance_id not in target:
        raise ValueError(f"Instance {command.instance_id} not found")
    del target[command.instance_id]
    return target


def get_transition_events(current: Mapping[InstanceId, Instance], target: Mapping[InstanceId, Instance],
                          tasks: Mapping[TaskId, Task] | None = None) -> list[Event]:
    """Events that turn ``current`` into ``target``; in-flight generation tasks of deleted instances
    are cancelled first so that their clients are released."""
    evs: list[Event] = []
    for iid, inst in target.items():
        if iid not in current:
            evs.append(InstanceCreated(instance=inst))
    for iid in current:
        if iid not in target:
            for t in (tasks or {}).values():
                if t.instance_id == iid and isinstance(t, (TextGeneration, ImageGeneration, ImageEdits)) \
                        and t.task_status in (TaskStatus.Pending, TaskStatus.Running):
                    evs.append(TaskStatusUpdated(task_id=t.task_id, task_status=TaskStatus.Cancelled))
            evs.append(InstanceDeleted(instance_id=iid))
    return evs


def memory_delta_by_node(instance: Instance) -> dict[str, int]:
    """Bytes a placement would add on each node (shown by placement previews)."""
    out: dict[str, int] = {}
    sa = instance.shard_assignments
    for node, rid in sa.node_to_runner.items():
        sm = sa.runner_to_shard[rid]
        frac = (sm.end_layer - sm.start_layer) / max(1, sm.n_layers) / max(1, sm.tp_size)
        out[str(node)] = int(sm.model_card.storage_size.in_bytes * frac)
    return out
