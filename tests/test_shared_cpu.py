"""Wire model, apply(), topology, buffers, disk log, channels, election — pure CPU."""
import anyio
import pytest
from pydantic import TypeAdapter

from exo_b200.shared.base import InstanceId, Memory, ModelId, NodeId, RunnerId, SessionId, TaskId
from exo_b200.shared.cards import ModelCard, card_cache
from exo_b200.shared.events import (IndexedEvent, InstanceCreated, InstanceDeleted, NodeGatheredInfo, NodeTimedOut,
                                    RunnerStatusUpdated, State, TaskCreated, TaskFailed, TaskStatusUpdated, apply)
from exo_b200.shared.messages import (Command, InputMessage, LoadModel, TaskStatus, TextGeneration,
                                      TextGenerationCommand, TextGenerationTaskParams)
from exo_b200.shared.topology import Connection, NvlinkConnection, Topology
from exo_b200.shared.wire import (MemoryUsage, NodeMemory, NodeNvlink, NodeNvlinkInfo, NvlinkInstance, NvlinkPeer,
                                  RunnerReady, RunnerShutdown, ShardAssignments, TensorShardMetadata)
from exo_b200.utils.buffers import DiskEventLog, KeyedBackoff, MultiSourceBuffer, OrderedBuffer
from exo_b200.utils.channels import ChannelClosed, channel, mp_channel


def _card():
    return ModelCard(model_id=ModelId("org/m"), storage_size=Memory.from_gb(16), n_layers=32, hidden_size=4096,
                     supports_tensor=True, num_key_value_heads=8, tasks=["TextGeneration"])


def _instance(nodes):
    card = _card()
    r2s, n2r, gpus = {}, {}, {}
    for i, n in enumerate(nodes):
        r = RunnerId()
        r2s[r] = TensorShardMetadata(model_card=card, device_rank=i, world_size=len(nodes), start_layer=0, end_layer=32,
                                     n_layers=32, tp_size=len(nodes), tp_rank=i, gpu_index=i)
        n2r[n] = r
        gpus[n] = i
    return NvlinkInstance(instance_id=InstanceId(), shard_assignments=ShardAssignments(
        model_id=card.model_id, runner_to_shard=r2s, node_to_runner=n2r), rendezvous_port=4000, gpu_by_node=gpus,
        parallelism=f"tp{len(nodes)}")


def test_tagged_union_roundtrip_and_command_tag():
    cmd = TextGenerationCommand(task_params=TextGenerationTaskParams(model="m", input=[InputMessage(role="user", content="x")]))
    js = cmd.model_dump_json()
    assert js.startswith('{"TextGeneration":')
    back = TypeAdapter(Command).validate_json(js)
    assert isinstance(back, TextGenerationCommand) and back.command_id == cmd.command_id


def test_apply_fold_and_state_json_roundtrip():
    a, b = NodeId("a"), NodeId("b")
    inst = _instance([a, b])
    r0 = next(iter(inst.shard_assignments.runner_to_shard))
    task = LoadModel(instance_id=inst.instance_id)
    tg = TextGeneration(instance_id=inst.instance_id, command_id="c1", task_params=TextGenerationTaskParams(
        model="org/m", input=[InputMessage(role="user", content="hi")]))
    evs = [InstanceCreated(instance=inst), RunnerStatusUpdated(runner_id=r0, runner_status=RunnerReady(prefill_server_port=9)),
           TaskCreated(task_id=task.task_id, task=task), TaskCreated(task_id=tg.task_id, task=tg),
           TaskFailed(task_id=tg.task_id, error_type="E", error_message="boom"),
           TaskStatusUpdated(task_id=tg.task_id, task_status=TaskStatus.Failed),
           NodeGatheredInfo(node_id=a, when="2025-01-01T00:00:00+00:00", info=NodeMemory(
               memory=MemoryUsage.from_bytes(ram_total=100, ram_available=60)))]
    st = State()
    for i, e in enumerate(evs):
        st = apply(st, IndexedEvent.model_validate_json(IndexedEvent(idx=i, event=e).model_dump_json()))
    assert st.prefill_server_ports[r0] == 9 and st.tasks[tg.task_id].error_message == "boom"
    assert st.tasks[tg.task_id].task_status == TaskStatus.Failed and st.node_memory[a].ram_available.in_bytes == 60
    assert State.model_validate_json(st.model_dump_json()) == st
    assert '"lastEventAppliedIdx"' in st.model_dump_json()
    with pytest.raises(AssertionError):
        apply(st, IndexedEvent(idx=99, event=InstanceDeleted(instance_id=inst.instance_id)))
    st = apply(st, IndexedEvent(idx=len(evs), event=RunnerStatusUpdated(runner_id=r0, runner_status=RunnerShutdown())))
    assert r0 not in st.runners and r0 not in st.prefill_server_ports
    st = apply(st, IndexedEvent(idx=len(evs) + 1, event=NodeTimedOut(node_id=a)))
    assert a not in st.node_memory and not st.topology.contains_node(a)


def test_nvlink_reports_become_topology_edges():
    st = State()
    ids = [NodeId(f"gpu{i}") for i in range(3)]
    for i, n in enumerate(ids):
        peers = [NvlinkPeer(peer_gpu=j, links=18, gbps=750.0) for j in range(3) if j != i]
        st = apply(st, IndexedEvent(idx=i, event=NodeGatheredInfo(node_id=n, when="x", info=NodeNvlink(
            info=NodeNvlinkInfo(gpu_index=i, peers=peers)))))
    assert st.topology.min_nvlink_gbps(ids) == 750.0
    cycles = [c for c in st.topology.get_cycles() if len(c) == 3]
    assert cycles and st.topology.is_rdma_cycle(cycles[0])


def test_topology_cycles_and_snapshot():
    t = Topology()
    a, b, c = NodeId("a"), NodeId("b"), NodeId("c")
    for s, k in ((a, b), (b, a), (b, c), (c, a)):
        t.add_connection(Connection(source=s, sink=k, edge=NvlinkConnection(source_gpu=0, sink_gpu=1, gbps=1.0)))
    sizes = sorted(len(x) for x in t.get_cycles())
    assert sizes == [1, 1, 1, 2, 3]
    assert Topology.from_snapshot(t.to_snapshot()) == t
    t.remove_node(b)
    assert sorted(len(x) for x in t.get_cycles()) == [1, 1]


def test_buffers_backoff_and_disk_log(tmp_path):
    ob = OrderedBuffer()
    ob.ingest(1, "b"); assert ob.drain() == [] and ob.has_gap
    ob.ingest(0, "a"); assert ob.drain() == ["a", "b"]
    ms = MultiSourceBuffer()
    ms.ingest(0, "x", "s1"); ms.ingest(1, "z", "s2"); ms.ingest(0, "y", "s2")
    assert sorted(ms.drain()) == ["x", "y", "z"]
    kb = KeyedBackoff(base=10.0)
    assert kb.should_proceed("k"); kb.record_attempt("k"); assert not kb.should_proceed("k"); kb.reset("k"); assert kb.should_proceed("k")
    log = DiskEventLog(tmp_path)
    for i in range(600):
        log.append({"i": i})
    assert [r["i"] for r in log.read_range(250, 260)] == list(range(250, 260)) and len(log) == 600
    log.close()
    log2 = DiskEventLog(tmp_path)   # previous log rotated into an archive, new one starts empty
    assert len(log2) == 0 and len(list(tmp_path.glob("*.bin.gz"))) == 1
    log2.close()


def test_channels_inproc_and_mp():
    async def main():
        s, r = channel()
        s2 = s.clone()
        await s.send(1); await s2.send(2)
        assert r.collect() == [1, 2]
        s.close(); s2.close()
        with pytest.raises(ChannelClosed):
            await r.receive()
    anyio.run(main)
    ms, mr = mp_channel()
    ms.send("a"); ms.close()
    assert mr.receive(timeout=5) == "a"
    with pytest.raises(ChannelClosed):
        mr.receive(timeout=5)


def test_election_three_nodes_agree_and_force_master_wins():
    from exo_b200.shared.election import Election, FORCE_MASTER_SENIORITY

    async def main():
        ids = [NodeId(x) for x in ("n1", "n2", "n3")]
        inboxes = [channel() for _ in ids]
        results = [channel() for _ in ids]
        conns = [channel() for _ in ids]
        cmds = [channel() for _ in ids]
        bus_s, bus_r = channel()
        els = [Election(n, election_message_receiver=inboxes[i][1], election_message_sender=bus_s.clone(),
                        election_result_sender=results[i][0], connection_message_receiver=conns[i][1],
                        command_receiver=cmds[i][1], seniority=FORCE_MASTER_SENIORITY if i == 1 else 0, timeout=0.3)
               for i, n in enumerate(ids)]

        async def fanout():
            async for m in bus_r:
                for s, _ in inboxes:
                    await s.send(m)

        async with anyio.create_task_group() as tg:
            tg.start_soon(fanout)
            for e in els:
                tg.start_soon(e.run)
            await anyio.sleep(0.1)
            from exo_b200.shared.election import ConnectionMessage
            for s, _ in conns:          # a link change triggers a real (timed) round everywhere
                await s.send(ConnectionMessage(node_id=ids[0], connected=True))
            await anyio.sleep(1.2)
            finals = [r.collect()[-1] for _, r in results]
            assert all(f.session_id.master_node_id == ids[1] for f in finals)
            assert len({f.session_id for f in finals}) == 1
            tg.cancel_scope.cancel()
    anyio.run(main)


def test_builtin_cards_load():
    c = card_cache.get("meta-llama/Llama-3.1-8B-Instruct")
    assert c is not None and c.n_layers == 32 and c.sampling_defaults.temperature == 0.6
    assert len(card_cache.list_all()) >= 30


def test_cards_of_every_served_family_load_and_place():
    """One card per family the engine loads: the sparse ones are recognised as such by the planner, vision shows as a capability."""
    from exo_b200.master.placement import is_moe_card
    cards = {str(c.model_id): c for c in card_cache.list_all()}
    assert len(cards) >= 120
    for mid, moe in (("mlx-community/Step-3.5-Flash-8Bit", True), ("mlx-community/Qwen3-Next-80B-A3B-Instruct-8bit", True),
                     ("mlx-community/Qwen3.5-9B-8bit", False), ("mlx-community/gemma-4-26b-a4b-it-8bit", True),
                     ("mlx-community/gemma-4-31b-it-8bit", False), ("mlx-community/NVIDIA-Nemotron-3-Nano-30B-A3B-MLX-8Bit", True),
                     ("mlx-community/GLM-4.7-8bit-gs32", True), ("mlx-community/MiniMax-M2.5-8bit", True),
                     ("mlx-community/Qwen3-Coder-Next-8bit", True), ("meta-llama/Llama-3.1-8B-Instruct", False)):
        assert mid in cards and is_moe_card(cards[mid]) is moe, mid
    assert "vision" in cards["mlx-community/Qwen3.5-9B-8bit"].capabilities and cards["mlx-community/Step-3.5-Flash-8Bit"].n_layers == 45
    assert all(c.backends and c.storage_size.in_bytes > 0 for c in cards.values())
