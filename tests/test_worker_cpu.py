"""Worker planner rules, runner state machine, supervisor failure path — CPU only, fake engine."""
import os
from dataclasses import dataclass, field

import anyio
import pytest

from exo_b200.shared.base import InstanceId, Memory, ModelId, NodeId, RunnerId, TaskId
from exo_b200.shared.cards import ModelCard
from exo_b200.shared.events import ChunkGenerated, RunnerStatusUpdated, TaskAcknowledged, TaskStatusUpdated
from exo_b200.shared.messages import (CancelTask, ConnectToGroup, CreateRunner, DownloadModel, InputMessage, LoadModel,
                                      Shutdown, StartWarmup, TaskStatus, TextGeneration, TextGenerationTaskParams)
from exo_b200.shared.wire import (BoundInstance, DownloadCompleted, ErrorChunk, NvlinkInstance, RunnerConnected,
                                  RunnerConnecting, RunnerFailed, RunnerIdle, RunnerLoaded, RunnerReady, RunnerRunning,
                                  RunnerShutdown, RunnerWarmingUp, ShardAssignments, TensorShardMetadata, TokenChunk)
from exo_b200.utils.buffers import KeyedBackoff
from exo_b200.utils.channels import channel, mp_channel
from exo_b200.worker.plan import plan


def card():
    return ModelCard(model_id=ModelId("org/m"), storage_size=Memory.from_gb(1), n_layers=8, hidden_size=64,
                     supports_tensor=True, tasks=["TextGeneration"])


def instance(n, **shard_kw):
    nodes = [NodeId(f"n{i}") for i in range(n)]
    rids = [RunnerId(f"r{i}") for i in range(n)]
    r2s = {rids[i]: TensorShardMetadata(model_card=card(), device_rank=i, world_size=n, start_layer=0, end_layer=8,
                                        n_layers=8, tp_size=n, tp_rank=i, **shard_kw) for i in range(n)}
    inst = NvlinkInstance(instance_id=InstanceId("inst"), shard_assignments=ShardAssignments(
        model_id=card().model_id, runner_to_shard=r2s, node_to_runner=dict(zip(nodes, rids))), rendezvous_port=1,
        gpu_by_node={n_: i for i, n_ in enumerate(nodes)})
    return inst, nodes, rids


@dataclass
class FakeSup:
    bound_instance: BoundInstance
    status: object
    completed: set = field(default_factory=set)
    in_progress: set = field(default_factory=set)
    cancelled: set = field(default_factory=set)


def sup(inst, node, rid, status):
    return FakeSup(BoundInstance(instance=inst, bound_runner_id=rid, bound_node_id=node), status)


def done(inst, nodes):
    return {n: [DownloadCompleted(node_id=n, shard_metadata=next(iter(inst.shard_assignments.runner_to_shard.values())),
                                  total=Memory.from_gb(1))] for n in nodes}


def test_lifecycle_rule_order_two_ranks():
    inst, nodes, rids = instance(2)
    insts = {inst.instance_id: inst}
    # nothing local yet -> create
    t = plan(nodes[0], {}, {}, insts, {}, {})
    assert isinstance(t, CreateRunner) and t.bound_instance.bound_runner_id == rids[0]
    r0 = {rids[0]: sup(inst, nodes[0], rids[0], RunnerIdle())}
    allr = {rids[0]: RunnerIdle(), rids[1]: RunnerIdle()}
    assert isinstance(plan(nodes[0], r0, {}, insts, allr, {}), DownloadModel)
    dl = done(inst, nodes)
    # rank 0 (accepting) connects first; the last rank waits until the others are Connecting
    assert isinstance(plan(nodes[0], r0, dl, insts, allr, {}), ConnectToGroup)
    r1 = {rids[1]: sup(inst, nodes[1], rids[1], RunnerIdle())}
    assert plan(nodes[1], r1, dl, insts, allr, {}) is None
    allr = {rids[0]: RunnerConnecting(), rids[1]: RunnerIdle()}
    assert isinstance(plan(nodes[1], r1, dl, insts, allr, {}), ConnectToGroup)
    # load when everyone is connected
    r0[rids[0]].status = RunnerConnected()
    allr = {rids[0]: RunnerConnected(), rids[1]: RunnerConnected()}
    assert isinstance(plan(nodes[0], r0, dl, insts, allr, {}), LoadModel)
    # warm-up: followers first, rank 0 once they are warming up
    r0[rids[0]].status = RunnerLoaded()
    allr = {rids[0]: RunnerLoaded(), rids[1]: RunnerLoaded()}
    assert plan(nodes[0], r0, dl, insts, allr, {}) is None
    r1[rids[1]].status = RunnerLoaded()
    assert isinstance(plan(nodes[1], r1, dl, insts, allr, {}), StartWarmup)
    allr = {rids[0]: RunnerLoaded(), rids[1]: RunnerWarmingUp()}
    assert isinstance(plan(nodes[0], r0, dl, insts, allr, {}), StartWarmup)


def test_forwarding_cancel_and_kill_rules():
    inst, nodes, rids = instance(2)
    insts = {inst.instance_id: inst}
    tg = TextGeneration(instance_id=inst.instance_id, command_id="c", task_params=TextGenerationTaskParams(
        model="org/m", input=[InputMessage(role="user", content="x")]))
    tasks = {tg.task_id: tg}
    r0 = {rids[0]: sup(inst, nodes[0], rids[0], RunnerReady())}
    # peer not ready -> hold the task back
    assert plan(nodes[0], r0, {}, insts, {rids[0]: RunnerReady(), rids[1]: RunnerWarmingUp()}, tasks) is None
    allr = {rids[0]: RunnerReady(), rids[1]: RunnerRunning()}
    assert plan(nodes[0], r0, {}, insts, allr, tasks) == tg
    r0[rids[0]].in_progress.add(tg.task_id)
    assert plan(nodes[0], r0, {}, insts, allr, tasks) is None
    cancelled = {tg.task_id: tg.model_copy(update={"task_status": TaskStatus.Cancelled})}
    t = plan(nodes[0], r0, {}, insts, allr, cancelled)
    assert isinstance(t, CancelTask) and t.cancelled_task_id == tg.task_id
    # a failed peer brings this runner down; a vanished instance too
    assert isinstance(plan(nodes[0], r0, {}, insts, {rids[0]: RunnerReady(), rids[1]: RunnerFailed()}, {}), Shutdown)
    assert isinstance(plan(nodes[0], r0, {}, {}, allr, {}), Shutdown)
    # re-creation respects the back-off and waits for failed peers
    bo = KeyedBackoff(base=100.0)
    bo.record_attempt(inst.instance_id)
    assert plan(nodes[0], {}, {}, insts, {}, {}, instance_backoff=bo) is None
    assert plan(nodes[0], {}, {}, insts, {rids[1]: RunnerFailed()}, {}) is None


def _tg_task(inst, text="hello"):
    return TextGeneration(instance_id=inst.instance_id, command_id="cmd", task_params=TextGenerationTaskParams(
        model="org/m", input=[InputMessage(role="user", content=text)]))


def _run_supervised(inst, nodes, rids, script):
    """Run a real child process (fake engine) under a supervisor and collect its events."""
    os.environ["EXO_ENGINE"] = "fake"
    from exo_b200.worker.runner.supervisor import RunnerSupervisor
    out = []

    async def main():
        ev_s, ev_r = channel()
        s = RunnerSupervisor.create(BoundInstance(instance=inst, bound_runner_id=rids[0], bound_node_id=nodes[0]), ev_s)
        async with anyio.create_task_group() as tg:
            tg.start_soon(s.run)
            await script(s)
            with anyio.move_on_after(45):     # a loaded machine takes seconds to spawn the child and to notice its death
                while not isinstance(s.status, (RunnerShutdown, RunnerFailed)):
                    await anyio.sleep(0.05)
            await anyio.sleep(1.0)
            out.extend(ev_r.collect())
            tg.cancel_scope.cancel()
    anyio.run(main)
    return out


def test_runner_child_lifecycle_event_order():
    inst, nodes, rids = instance(1)

    async def script(s):
        assert await s.start_task(LoadModel(instance_id=inst.instance_id))
        assert await s.start_task(StartWarmup(instance_id=inst.instance_id))
        t = _tg_task(inst)
        assert await s.start_task(t)
        with anyio.move_on_after(10):
            while t.task_id not in s.completed:
                await anyio.sleep(0.02)
        assert await s.start_task(Shutdown(instance_id=inst.instance_id, runner_id=rids[0]))
    evs = _run_supervised(inst, nodes, rids, script)
    statuses = [type(e.runner_status).__name__ for e in evs if isinstance(e, RunnerStatusUpdated)]
    dedup = [s for i, s in enumerate(statuses) if i == 0 or s != statuses[i - 1]]
    assert dedup == ["RunnerIdle", "RunnerLoading", "RunnerLoaded", "RunnerWarmingUp", "RunnerReady", "RunnerRunning",
                     "RunnerReady", "RunnerShuttingDown", "RunnerShutdown"]
    chunks = [e.chunk for e in evs if isinstance(e, ChunkGenerated)]
    assert [c.text for c in chunks] == ["tok0 ", "tok1 ", "tok2 ", "tok3 "] and chunks[-1].finish_reason == "stop"
    assert sum(isinstance(e, TaskAcknowledged) for e in evs) == 4


def test_runner_death_becomes_runner_failed_and_error_chunk():
    inst, nodes, rids = instance(1)

    async def script(s):
        await s.start_task(LoadModel(instance_id=inst.instance_id))
        await s.start_task(StartWarmup(instance_id=inst.instance_id))
        await s.start_task(_tg_task(inst, "EXO RUNNER MUST FAIL"))
    evs = _run_supervised(inst, nodes, rids, script)
    failed = [e for e in evs if isinstance(e, RunnerStatusUpdated) and isinstance(e.runner_status, RunnerFailed)]
    assert failed and "exited with code 1" in failed[-1].runner_status.error_message
    errs = [e.chunk for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, ErrorChunk)]
    assert errs and "Artificial runner exception" in errs[0].error_message
    assert any(isinstance(e, TaskStatusUpdated) and e.task_status == TaskStatus.Failed for e in evs)


def test_a_collective_that_gave_up_on_a_peer_ends_the_runner_with_a_diagnostic():
    """The executor raises after a step whose device-side wait on a peer ran out (it reads the status words every
    step); the runner process dies, the supervisor reports RunnerFailed with the collective-timeout diagnostic and
    an ErrorChunk for the request in flight.  The failure is made on the host: no GPU takes part."""
    inst, nodes, rids = instance(1)

    async def script(s):
        await s.start_task(LoadModel(instance_id=inst.instance_id))
        await s.start_task(StartWarmup(instance_id=inst.instance_id))
        await s.start_task(_tg_task(inst, "EXO RUNNER MUST LOSE A PEER"))
    evs = _run_supervised(inst, nodes, rids, script)
    failed = [e.runner_status for e in evs if isinstance(e, RunnerStatusUpdated) and isinstance(e.runner_status, RunnerFailed)]
    assert failed and any(d.kind == "collective_timeout" for d in failed[-1].diagnostics)
    errs = [e.chunk for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, ErrorChunk)]
    assert errs and "peer GPU" in errs[0].error_message


def test_immediate_exception_hook_and_oom_diagnostic():
    inst, nodes, rids = instance(1, immediate_exception=True)

    async def script(s):
        await anyio.sleep(0.1)
    evs = _run_supervised(inst, nodes, rids, script)
    assert any(isinstance(e, RunnerStatusUpdated) and isinstance(e.runner_status, RunnerFailed) for e in evs)
    inst2, nodes2, rids2 = instance(1)

    async def script2(s):
        await s.start_task(LoadModel(instance_id=inst2.instance_id))
        await s.start_task(StartWarmup(instance_id=inst2.instance_id))
        await s.start_task(_tg_task(inst2, "EXO RUNNER MUST OOM"))
    evs = _run_supervised(inst2, nodes2, rids2, script2)
    failed = [e.runner_status for e in evs if isinstance(e, RunnerStatusUpdated) and isinstance(e.runner_status, RunnerFailed)]
    assert failed and any(d.kind == "host_oom" for d in failed[-1].diagnostics)
