"""Placement planner and master command/event processing with in-memory channels."""
import anyio
import pytest

from exo_b200.master.main import Master
from exo_b200.master.placement import (allocate_layers_proportionally, choose_shape, get_transition_events,
                                        memory_delta_by_node, place_instance)
from exo_b200.shared.base import Memory, ModelId, NodeId, SessionId, SystemId
from exo_b200.shared.cards import Backend, ModelCard
from exo_b200.shared.events import (InstanceCreated, LocalForwarderEvent, NodeGatheredInfo, RunnerStatusUpdated, State,
                                    TaskCreated, TaskDeleted)
from exo_b200.shared.messages import (DeleteInstance, ForwarderCommand, InputMessage, PlaceInstance, RequestEventLog,
                                      TaskFinished, TextGenerationCommand, TextGenerationTaskParams)
from exo_b200.shared.topology import Connection, NvlinkConnection, Topology
from exo_b200.shared.wire import (InstanceMeta, MemoryUsage, NodeBackends, NodeMemory, NodeNvlink, NodeNvlinkInfo,
                                  NvlinkPeer, PipelineShardMetadata, RunnerReady, Sharding, TensorShardMetadata)
from exo_b200.utils.channels import channel

GB = 1024 ** 3


def card(size_gb, layers=32, hidden=4096, kv=8, tensor=True):
    return ModelCard(model_id=ModelId("org/m"), storage_size=Memory.from_gb(size_gb), n_layers=layers, hidden_size=hidden,
                     supports_tensor=tensor, num_key_value_heads=kv, tasks=["TextGeneration"], backends=[Backend.B200])


def box(n, free_gb=170):
    topo, mem, be = Topology(), {}, {}
    ids = [NodeId(f"gpu{i}") for i in range(n)]
    for i, a in enumerate(ids):
        topo.add_node(a)
        mem[a] = MemoryUsage.from_bytes(ram_total=180 * GB, ram_available=(free_gb[i] if isinstance(free_gb, list) else free_gb) * GB)
        be[a] = [Backend.B200]
        for j, b in enumerate(ids):
            if i != j:
                topo.add_connection(Connection(source=a, sink=b, edge=NvlinkConnection(source_gpu=i, sink_gpu=j, gbps=750, links=18)))
    return ids, topo, mem, be


def place(c, n_gpus, sharding=Sharding.Tensor, min_nodes=1, **kw):
    ids, topo, mem, be = box(n_gpus, **kw)
    cmd = PlaceInstance(model_card=c, sharding=sharding, instance_meta=InstanceMeta.MlxRing, min_nodes=min_nodes)
    out = place_instance(cmd, topo, {}, mem, be, gpu_index={n: i for i, n in enumerate(ids)})
    return next(iter(out.values()))


def test_small_model_goes_to_one_gpu_with_most_free_memory():
    inst = place(card(16), 8, free_gb=[100, 100, 170, 100, 100, 100, 100, 100])
    assert list(inst.gpu_by_node.values()) == [2] and inst.parallelism == "tp1"


def test_model_larger_than_one_gpu_is_tensor_sharded_over_smallest_group():
    inst = place(card(240, layers=94, kv=4), 8)
    shards = list(inst.shard_assignments.runner_to_shard.values())
    assert len(shards) == 2 and all(isinstance(s, TensorShardMetadata) for s in shards)
    assert sorted(s.tp_rank for s in shards) == [0, 1]


def test_min_nodes_and_kv_head_replication_allow_tp8_on_4_kv_heads():
    inst = place(card(240, layers=94, kv=4), 8, min_nodes=8)
    assert len(inst.shard_assignments.runner_to_shard) == 8 and inst.parallelism.startswith(("tp8", "pp2xtp4"))


def test_pipeline_request_splits_layers_by_memory():
    inst = place(card(300, layers=80), 4, sharding=Sharding.Pipeline, min_nodes=4, free_gb=[170, 170, 120, 120])
    shards = sorted(inst.shard_assignments.runner_to_shard.values(), key=lambda s: s.device_rank)
    assert all(isinstance(s, PipelineShardMetadata) for s in shards)
    assert shards[0].start_layer == 0 and shards[-1].end_layer == 80
    assert all(a.end_layer == b.start_layer for a, b in zip(shards, shards[1:]))
    sizes = [s.end_layer - s.start_layer for s in shards]
    assert sizes[0] > sizes[-1]
    assert sum(memory_delta_by_node(inst).values()) == pytest.approx(300 * GB, rel=1e-3)


def test_errors_match_reference_wording():
    with pytest.raises(ValueError, match="No cycles found with sufficient memory"):
        place(card(2000), 8)
    with pytest.raises(ValueError, match="does not support tensor parallelism"):
        place(card(240, tensor=False), 8)
    with pytest.raises(ValueError, match="No tensor sharding found"):
        place(card(240, hidden=4100, kv=3), 8, min_nodes=8)


def test_layer_allocation_and_shape_choice():
    assert allocate_layers_proportionally(10, [1, 1, 1]) in ([4, 3, 3], [3, 4, 3], [3, 3, 4])
    assert sum(allocate_layers_proportionally(61, [5, 3, 2, 1])) == 61
    with pytest.raises(ValueError):
        allocate_layers_proportionally(2, [1, 1, 1])
    # with healthy NVLink pure TP-8 wins; with a crippled link the planner halves the all-reduce fan-in
    assert choose_shape(card(140, layers=80, hidden=8192), 8, Sharding.Tensor, 750.0) == (8, 1)
    assert choose_shape(card(140, layers=80, hidden=8192), 8, Sharding.Tensor, 0.001) == (4, 2)


def test_master_places_routes_and_replays(tmp_path):
    async def main():
        ids, topo, mem, be = box(2)
        cmd_s, cmd_r = channel()
        loc_s, loc_r = channel()
        glob_s, glob_r = channel()
        sess = SessionId(master_node_id=ids[0], election_clock=0)
        m = Master(ids[0], sess, command_receiver=cmd_r, local_event_receiver=loc_r, global_event_sender=glob_s,
                   log_dir=tmp_path)
        origin = SystemId("sys")
        async with anyio.create_task_group() as tg:
            tg.start_soon(m.run)
            k = 0
            for i, n in enumerate(ids):
                for info in (NodeMemory(memory=mem[n]), NodeBackends(backends=[Backend.B200]),
                             NodeNvlink(info=NodeNvlinkInfo(gpu_index=i, peers=[NvlinkPeer(peer_gpu=1 - i, links=18, gbps=750)]))):
                    await loc_s.send(LocalForwarderEvent(origin_idx=k, origin=origin, session=sess,
                                                         event=NodeGatheredInfo(node_id=n, when="", info=info)))
                    k += 1
            await anyio.sleep(0.1)
            assert m.state.topology.min_nvlink_gbps(ids) == 750
            await cmd_s.send(ForwarderCommand(origin=origin, command=PlaceInstance(
                model_card=card(16), sharding=Sharding.Tensor, instance_meta=InstanceMeta.MlxRing, min_nodes=2)))
            await anyio.sleep(0.1)
            assert len(m.state.instances) == 1
            inst = next(iter(m.state.instances.values()))
            # request before runners are ready -> error chunk; after -> task on that instance
            tp = TextGenerationTaskParams(model="org/m", input=[InputMessage(role="user", content="hi")])
            c1 = TextGenerationCommand(task_params=tp)
            await cmd_s.send(ForwarderCommand(origin=origin, command=c1))
            await anyio.sleep(0.05)
            assert not m.state.tasks
            for r in inst.shard_assignments.runner_to_shard:
                await loc_s.send(LocalForwarderEvent(origin_idx=k, origin=origin, session=sess,
                                                     event=RunnerStatusUpdated(runner_id=r, runner_status=RunnerReady())))
                k += 1
            await anyio.sleep(0.05)
            c2 = TextGenerationCommand(task_params=tp)
            await cmd_s.send(ForwarderCommand(origin=origin, command=c2))
            await anyio.sleep(0.05)
            assert len(m.state.tasks) == 1 and next(iter(m.state.tasks.values())).instance_id == inst.instance_id
            await cmd_s.send(ForwarderCommand(origin=origin, command=TaskFinished(finished_command_id=c2.command_id)))
            await anyio.sleep(0.05)
            assert not m.state.tasks
            seen = glob_r.collect()
            assert [e.origin_idx for e in seen] == list(range(len(seen)))
            await cmd_s.send(ForwarderCommand(origin=origin, command=RequestEventLog(since_idx=2)))
            await anyio.sleep(0.05)
            replay = glob_r.collect()
            assert [e.origin_idx for e in replay] == list(range(2, len(seen)))
            assert replay[0].event == seen[2].event
            await cmd_s.send(ForwarderCommand(origin=origin, command=DeleteInstance(instance_id=inst.instance_id)))
            await anyio.sleep(0.05)
            assert not m.state.instances
            tg.cancel_scope.cancel()
    anyio.run(main)
