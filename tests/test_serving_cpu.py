"""The serving engine end to end on CPU: checkpoint dir -> builder -> runner -> chunks (1 and 2 ranks)."""
import json
import os
import socket

import anyio
import pytest
import torch

from exo_b200.models.config import preset
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights, write_safetensors
from exo_b200.shared.base import InstanceId, Memory, ModelId, NodeId, RunnerId
from exo_b200.shared.cards import ModelCard
from exo_b200.shared.events import ChunkGenerated, RunnerStatusUpdated
from exo_b200.shared.messages import (ConnectToGroup, InputMessage, LoadModel, Shutdown, StartWarmup, TextGeneration,
                                      TextGenerationTaskParams)
from exo_b200.shared.wire import (BoundInstance, NvlinkInstance, PipelineShardMetadata, RunnerFailed, RunnerReady, RunnerShutdown,
                                  ShardAssignments, TensorShardMetadata, TokenChunk, ToolCallChunk)
from exo_b200.utils.channels import channel


@pytest.fixture(autouse=True)
def _engine_env(monkeypatch):
    monkeypatch.setenv("EXO_ENGINE", "b200")
    monkeypatch.setenv("EXO_DEVICE", "cpu")
    monkeypatch.setenv("EXO_MAX_KV_BLOCKS", "128")


def make_checkpoint(tmp_path):
    """A tiny Llama checkpoint in HF layout (config.json + model.safetensors), byte-level vocab."""
    cfg = preset("tiny-llama")
    cfg.vocab = 512
    d = tmp_path / "org--tiny"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({
        "model_type": "llama", "architectures": ["LlamaForCausalLM"], "hidden_size": cfg.hidden, "num_hidden_layers": cfg.n_layers,
        "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "intermediate_size": cfg.ffn,
        "vocab_size": cfg.vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048, "eos_token_id": 257}))
    src = RandomSource(seed=0)
    names = {"model.embed_tokens.weight": (cfg.vocab, cfg.hidden), "model.norm.weight": (cfg.hidden,), "lm_head.weight": (cfg.vocab, cfg.hidden)}
    D = cfg.head_dim
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        names.update({p + "input_layernorm.weight": (cfg.hidden,), p + "post_attention_layernorm.weight": (cfg.hidden,),
                      p + "self_attn.q_proj.weight": (cfg.n_heads * D, cfg.hidden), p + "self_attn.k_proj.weight": (cfg.n_kv_heads * D, cfg.hidden),
                      p + "self_attn.v_proj.weight": (cfg.n_kv_heads * D, cfg.hidden), p + "self_attn.o_proj.weight": (cfg.hidden, cfg.n_heads * D),
                      p + "mlp.gate_proj.weight": (cfg.ffn, cfg.hidden), p + "mlp.up_proj.weight": (cfg.ffn, cfg.hidden),
                      p + "mlp.down_proj.weight": (cfg.hidden, cfg.ffn)})
    write_safetensors(d / "model.safetensors", {k: src.get(k, v) for k, v in names.items()})
    return d, cfg


def instance(model_dir, n, pp=1):
    card = ModelCard(model_id=ModelId(str(model_dir)), storage_size=Memory.from_mb(10), n_layers=2, hidden_size=256,
                     supports_tensor=True, num_key_value_heads=2, tasks=["TextGeneration"], family="llama")
    nodes = [NodeId(f"n{i}") for i in range(n)]
    rids = [RunnerId(f"r{i}") for i in range(n)]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    if pp > 1:      # one layer per stage, rank = pp_rank * tp + tp_rank
        tp = n // pp
        r2s = {rids[i]: PipelineShardMetadata(model_card=card, device_rank=i, world_size=n, start_layer=i // tp, end_layer=i // tp + 1,
                                              n_layers=2, tp_size=tp, tp_rank=i % tp, pp_size=pp, pp_rank=i // tp) for i in range(n)}
    else:
        r2s = {rids[i]: TensorShardMetadata(model_card=card, device_rank=i, world_size=n, start_layer=0, end_layer=2, n_layers=2,
                                            tp_size=n, tp_rank=i) for i in range(n)}
    return NvlinkInstance(instance_id=InstanceId("i"), shard_assignments=ShardAssignments(
        model_id=card.model_id, runner_to_shard=r2s, node_to_runner=dict(zip(nodes, rids))), rendezvous_port=port,
        gpu_by_node={x: i for i, x in enumerate(nodes)}), nodes, rids


def gen_task(inst, text, **kw):
    return TextGeneration(instance_id=inst.instance_id, command_id="cmd", task_params=TextGenerationTaskParams(
        model=inst.shard_assignments.model_id, input=[InputMessage(role="user", content=text)], temperature=0.0, **kw))


def drive(inst, nodes, rids, tasks_fn, timeout=120):
    from exo_b200.worker.runner.supervisor import RunnerSupervisor
    events = []

    async def main():
        ev_s, ev_r = channel()
        sups = [RunnerSupervisor.create(BoundInstance(instance=inst, bound_runner_id=rids[i], bound_node_id=nodes[i]), ev_s.clone())
                for i in range(len(rids))]
        async with anyio.create_task_group() as tg:
            for s in sups:
                tg.start_soon(s.run)

            async def all_do(mk):
                async with anyio.create_task_group() as g:
                    for s in sups:
                        g.start_soon(s.start_task, mk(s))
            with anyio.fail_after(timeout):
                if len(sups) > 1:
                    await all_do(lambda s: ConnectToGroup(instance_id=inst.instance_id))
                await all_do(lambda s: LoadModel(instance_id=inst.instance_id))
                await all_do(lambda s: StartWarmup(instance_id=inst.instance_id))
                while not all(isinstance(s.status, (RunnerReady, RunnerFailed)) for s in sups):
                    await anyio.sleep(0.05)
                assert all(isinstance(s.status, RunnerReady) for s in sups), [s.status for s in sups]
                for t in tasks_fn():
                    await all_do(lambda s, t=t: t)
                    while not all(t.task_id in s.completed for s in sups):
                        await anyio.sleep(0.05)
                for s in sups:
                    await s.start_task(Shutdown(instance_id=inst.instance_id, runner_id=s.bound_instance.bound_runner_id))
                while not all(isinstance(s.status, (RunnerShutdown, RunnerFailed)) for s in sups):
                    await anyio.sleep(0.05)
            await anyio.sleep(0.2)
            events.extend(ev_r.collect())
            tg.cancel_scope.cancel()
    anyio.run(main)
    return events


def test_single_rank_serving_matches_token_engine_and_reports_stats(tmp_path):
    d, cfg = make_checkpoint(tmp_path)
    inst, nodes, rids = instance(d, 1)
    t = gen_task(inst, "hello world", max_output_tokens=12, bench=True)
    evs = drive(inst, nodes, rids, lambda: [t])
    chunks = [e.chunk for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    assert len(chunks) == 12 and chunks[-1].finish_reason == "length"
    assert chunks[-1].usage.completion_tokens == 12 and chunks[-1].stats.generation_tokens == 12
    # same tokens as the bare token engine on the same prompt
    from exo_b200.engine.engine import Engine
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.models.config import ModelConfig
    from exo_b200.models.weights import SafetensorsSource
    from exo_b200.worker.engines.b200.tokenizer import ByteTokenizer, render_prompt
    c2 = ModelConfig.from_pretrained(d); c2.dtype = "fp32"
    w = build_weights(c2, ShardSpec(), SafetensorsSource(d, dtype=torch.float32))
    ids = ByteTokenizer(512).encode(render_prompt(ByteTokenizer(512), t.task_params)[0], add_special_tokens=True)
    want = Engine(c2, w, n_blocks=64).generate(ids, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert [c.token_id for c in chunks] == want


def test_two_rank_tp_serving_on_gloo_matches_single_rank(tmp_path):
    d, cfg = make_checkpoint(tmp_path)
    inst1, n1, r1 = instance(d, 1)
    t1 = gen_task(inst1, "abc", max_output_tokens=8, bench=True)
    one = [e.chunk.token_id for e in drive(inst1, n1, r1, lambda: [t1]) if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    inst2, n2, r2 = instance(d, 2)
    t2 = gen_task(inst2, "abc", max_output_tokens=8, bench=True)
    evs = drive(inst2, n2, r2, lambda: [t2])
    two = [e.chunk.token_id for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    assert len(two) == 8 and two == one


def test_two_stage_pipeline_serving_on_gloo_matches_single_rank(tmp_path):
    d, cfg = make_checkpoint(tmp_path)
    inst1, n1, r1 = instance(d, 1)
    t1 = gen_task(inst1, "pipeline", max_output_tokens=8, bench=True)
    one = [e.chunk.token_id for e in drive(inst1, n1, r1, lambda: [t1]) if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    inst2, n2, r2 = instance(d, 2, pp=2)
    t2 = gen_task(inst2, "pipeline", max_output_tokens=8, bench=True)
    evs = drive(inst2, n2, r2, lambda: [t2])
    two = [e.chunk.token_id for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    assert len(two) == 8 and two == one


def test_image_inputs_reach_the_engine_as_spliced_features(tmp_path):
    """A request with images: the runner encodes them, the prompt grows by the images' feature rows, different
    images give different continuations, and the same image again hits the prefix cache."""
    import base64
    import io

    import numpy as np
    from PIL import Image

    def png(seed):
        buf = io.BytesIO()
        Image.fromarray((np.random.default_rng(seed).random((56, 84, 3)) * 255).astype("uint8")).save(buf, format="PNG")
        return base64.b64encode(buf.getvalue()).decode()
    d, cfg = make_checkpoint(tmp_path)
    inst, nodes, rids = instance(d, 1)
    plain = gen_task(inst, "describe", max_output_tokens=6)
    a1 = gen_task(inst, "describe", max_output_tokens=6, images=[png(1)])
    b = gen_task(inst, "describe", max_output_tokens=6, images=[png(2)])
    a2 = gen_task(inst, "describe", max_output_tokens=6, images=[png(1)])
    evs = drive(inst, nodes, rids, lambda: [plain, a1, b, a2])
    finals = [c for c in (e.chunk for e in evs if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)) if c.finish_reason]
    assert len(finals) == 4, [c.finish_reason for c in finals]
    n_plain, n_a1, n_b, n_a2 = (c.usage.prompt_tokens for c in finals)
    assert n_a1 == n_b == n_a2 and n_a1 - n_plain == 6          # 84x56 pixels = 3 x 2 cells of 28 pixels
    assert finals[3].usage.prompt_tokens_details.cached_tokens > 0 and finals[1].usage.prompt_tokens_details.cached_tokens == 0


@pytest.mark.parametrize("pp", [1, 2])
def test_image_inputs_on_two_ranks_match_one_rank(tmp_path, pp):
    """Image features are computed on rank 0 and follow the step plans to the other ranks (tensor-parallel ranks all embed
    the prompt; with pipeline stages only the first does): the tokens equal those of a single-rank instance."""
    import base64
    import io

    import numpy as np
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray((np.random.default_rng(4).random((56, 84, 3)) * 255).astype("uint8")).save(buf, format="PNG")
    img = base64.b64encode(buf.getvalue()).decode()
    d, cfg = make_checkpoint(tmp_path)

    def tokens(n, pp_):
        inst, nodes, rids = instance(d, n, pp=pp_)
        t = gen_task(inst, "describe", max_output_tokens=6, images=[img], bench=True)
        return [e.chunk.token_id for e in drive(inst, nodes, rids, lambda: [t]) if isinstance(e, ChunkGenerated) and isinstance(e.chunk, TokenChunk)]
    one, two = tokens(1, 1), tokens(2, pp)
    assert len(one) == 6 and two == one
