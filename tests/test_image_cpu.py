"""Image engine on CPU: sampler determinism, chunked PNG output, CFG-parallel and pipeline schedules on gloo ranks."""
import base64
import io
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from exo_b200.api.types import AdvancedImageParams, ImageEditsTaskParams, ImageGenerationTaskParams
from exo_b200.shared.base import InstanceId
from exo_b200.shared.messages import ImageEdits, ImageGeneration
from exo_b200.shared.wire import ImageChunk
from exo_b200.worker.engines.base import Cancelled, Finished
from exo_b200.worker.engines.image.builder import ImageEngine, decode_image
from exo_b200.worker.engines.image.dit import Dit, DitConfig
from exo_b200.worker.engines.image.pipeline import DiffusionRunner


def small(uses_cfg=False):
    return DitConfig(hidden=64, n_heads=2, n_joint=1, n_single=3, uses_cfg=uses_cfg)


def final(runner, **kw):
    out = list(runner.generate("a red fox", 128, 128, 4, 7, **kw))
    assert out[-1][0] == "final"
    return out[-1][1], out[:-1]


def test_sampler_is_deterministic_and_seed_and_prompt_matter():
    r = DiffusionRunner(Dit(small()))
    a, _ = final(r)
    b, _ = final(r)
    assert a.shape == (128, 128, 3) and a.dtype == torch.uint8 and torch.equal(a, b)
    c = list(r.generate("a red fox", 128, 128, 4, 8))[-1][1]
    d = list(r.generate("a blue whale", 128, 128, 4, 7))[-1][1]
    assert not torch.equal(a, c) and not torch.equal(a, d)
    _, partials = final(r, partial_images=2)
    assert [p[0] for p in partials] == ["partial", "partial"] and [p[2] for p in partials] == [0, 1]
    # image-to-image: low strength stays close to the input, high strength moves away from it
    src = a
    near = list(r.generate("x", 128, 128, 8, 1, init_image=src, strength=0.2))[-1][1].float()
    far = list(r.generate("x", 128, 128, 8, 1, init_image=src, strength=0.95))[-1][1].float()
    assert (near - src.float()).abs().mean() < (far - src.float()).abs().mean()


def _collect(engine, task):
    engine.submit(task)
    chunks, end = [], None
    while engine.has_work:
        for _tid, item in engine.step():
            if isinstance(item, ImageChunk):
                chunks.append(item)
            else:
                end = item
    return chunks, end


def test_engine_streams_chunked_images_with_partials_stats_edits_and_cancel(monkeypatch):
    from exo_b200.shared import constants
    monkeypatch.setattr(constants, "EXO_MAX_CHUNK_SIZE", 4096)
    eng = ImageEngine(DiffusionRunner(Dit(small())), "org/img", 0, 1)
    p = ImageGenerationTaskParams(prompt="a lighthouse", model="org/img", size="256x256", quality="low", n=2, stream=True,
                                  partial_images=1, bench=True, advanced_params=AdvancedImageParams(seed=3))
    chunks, end = _collect(eng, ImageGeneration(instance_id=InstanceId("i"), command_id="c", task_params=p))
    assert isinstance(end, Finished)
    finals = {}
    for c in chunks:
        if not c.is_partial:
            finals.setdefault(c.image_index, {})[c.chunk_index] = c
    assert sorted(finals) == [0, 1] and all(len(v) == v[0].total_chunks > 1 for v in finals.values())
    png = base64.b64decode("".join(finals[0][i].data for i in range(len(finals[0]))))
    img = decode_image(png)
    assert img.shape == (256, 256, 3)
    assert sum(c.is_partial and c.chunk_index == 0 for c in chunks) == 2            # one preview per image
    last = finals[1][len(finals[1]) - 1]
    assert last.stats is not None and last.stats.num_images == 2 and last.stats.num_inference_steps == 4 and last.finish_reason == "stop"
    assert finals[0][len(finals[0]) - 1].stats is None
    # edit: the uploaded image comes back at its own size when size is auto
    e = ImageEditsTaskParams(image_data=base64.b64encode(png).decode(), prompt="make it night", model="org/img", quality="low",
                             image_strength=0.3, advanced_params=AdvancedImageParams(seed=1))
    chunks, end = _collect(eng, ImageEdits(instance_id=InstanceId("i"), command_id="c2", task_params=e))
    out = decode_image(base64.b64decode("".join(c.data for c in sorted(chunks, key=lambda c: c.chunk_index))))
    assert isinstance(end, Finished) and out.shape == (256, 256, 3)
    # cancel before it starts
    t = ImageGeneration(instance_id=InstanceId("i"), command_id="c3", task_params=p)
    eng.cancel(t.task_id)
    chunks, end = _collect(eng, t)
    assert chunks == [] and isinstance(end, Cancelled)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = small(uses_cfg=mode == "cfg")
        if mode == "cfg":
            groups = [dist.new_group([0]), dist.new_group([1])]
            r = DiffusionRunner(Dit(cfg), rank=rank, world=2, cfg_parallel=True, pipe_groups=groups)
        else:
            groups = [dist.new_group([0, 1])]
            per = cfg.n_blocks // 2
            model = Dit(cfg, blocks=range(rank * per, (rank + 1) * per))
            r = DiffusionRunner(model, rank=rank, world=2, num_sync_steps=99 if mode == "pipe_sync" else 1, pipe_groups=groups)
        img = list(r.generate("a red fox", 128, 128, 4, 7))[-1][1]
        q.put((rank, img, r.n_exchanges, r.n_patch_hops))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["cfg", "pipe_sync", "pipefusion"])
def test_two_rank_schedules_against_single_rank(mode):
    want = list(DiffusionRunner(Dit(small(uses_cfg=mode == "cfg"))).generate("a red fox", 128, 128, 4, 7))[-1][1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict((r, (img, ex, hops)) for r, img, ex, hops in (q.get(timeout=180) for _ in range(2)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert torch.equal(got[0][0], got[1][0])                      # every rank ends with the same image
    diff = (got[0][0].float() - want.float()).abs()
    if mode == "cfg":
        assert got[0][1] == 4 and diff.max() <= 1                # one swap per step; same maths as the local two-pass CFG
    elif mode == "pipe_sync":
        assert got[0][2] == 0 and diff.max() <= 1                # synchronous stages reproduce the single-rank image
    else:
        assert got[0][2] == 3 * 2                                  # 3 asynchronous steps x 2 patches hop to stage 1
        assert diff.mean() < 40                                    # stale K/V of the other patch: close, not equal


def test_image_instance_through_the_runner_process(monkeypatch):
    """Bootstrap picks the image builder for an image card; chunks come back as events from the child process."""
    import anyio
    from exo_b200.shared.base import Memory, ModelId, NodeId, RunnerId
    from exo_b200.shared.cards import ModelCard
    from exo_b200.shared.events import ChunkGenerated
    from exo_b200.shared.messages import LoadModel, Shutdown, StartWarmup
    from exo_b200.shared.wire import (BoundInstance, NvlinkInstance, PipelineShardMetadata, RunnerFailed, RunnerReady,
                                      RunnerShutdown, ShardAssignments)
    from exo_b200.utils.channels import channel
    from exo_b200.worker.runner.supervisor import RunnerSupervisor
    monkeypatch.setenv("EXO_ENGINE", "b200")
    monkeypatch.setenv("EXO_DEVICE", "cpu")
    card = ModelCard(model_id=ModelId("org/tiny-image"), storage_size=Memory.from_mb(1), n_layers=4, hidden_size=64,
                     supports_tensor=False, tasks=["TextToImage", "ImageToImage"], family="flux")
    node, rid = NodeId("n0"), RunnerId("r0")
    inst = NvlinkInstance(instance_id=InstanceId("img"), shard_assignments=ShardAssignments(
        model_id=card.model_id, runner_to_shard={rid: PipelineShardMetadata(model_card=card, device_rank=0, world_size=1, start_layer=0,
                                                                            end_layer=4, n_layers=4)},
        node_to_runner={node: rid}), rendezvous_port=1, gpu_by_node={node: 0})
    task = ImageGeneration(instance_id=inst.instance_id, command_id="cmd", task_params=ImageGenerationTaskParams(
        prompt="a boat", model="org/tiny-image", size="256x256", quality="low", advanced_params=AdvancedImageParams(seed=5)))
    events = []

    async def main():
        ev_s, ev_r = channel()
        sup = RunnerSupervisor.create(BoundInstance(instance=inst, bound_runner_id=rid, bound_node_id=node), ev_s)
        async with anyio.create_task_group() as tg:
            tg.start_soon(sup.run)
            with anyio.fail_after(120):
                await sup.start_task(LoadModel(instance_id=inst.instance_id))
                await sup.start_task(StartWarmup(instance_id=inst.instance_id))
                while not isinstance(sup.status, (RunnerReady, RunnerFailed)):
                    await anyio.sleep(0.05)
                assert isinstance(sup.status, RunnerReady), sup.status
                await sup.start_task(task)
                while task.task_id not in sup.completed:
                    await anyio.sleep(0.05)
                await sup.start_task(Shutdown(instance_id=inst.instance_id, runner_id=rid))
                while not isinstance(sup.status, (RunnerShutdown, RunnerFailed)):
                    await anyio.sleep(0.05)
            await anyio.sleep(0.2)
            events.extend(ev_r.collect())
            tg.cancel_scope.cancel()
    anyio.run(main)
    chunks = [e.chunk for e in events if isinstance(e, ChunkGenerated) and isinstance(e.chunk, ImageChunk)]
    assert chunks and chunks[-1].finish_reason == "stop"
    img = decode_image(base64.b64decode("".join(c.data for c in sorted(chunks, key=lambda c: c.chunk_index))))
    assert img.shape == (256, 256, 3)
