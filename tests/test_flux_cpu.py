"""FLUX.1 on CPU: checkpoint-folder loading (whole model and pipeline stages), rotary positions, the VAE's shapes, the
sampler with the model's own schedule, the Kontext reference-image path, and the two-rank schedules on gloo."""
import json
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from exo_b200.worker.engines.image.flux import (FluxConfig, FluxModel, FluxVAE, random_weights, rope_apply, rope_tables,
                                                transformer_shapes, vae_shapes)
from exo_b200.worker.engines.image.pipeline import DiffusionRunner


def tiny(**kw):
    base = dict(n_joint=2, n_single=2, n_heads=2, head_dim=32, text_dim=48, pooled_dim=24, axes_dims=(8, 12, 12), text_len=16,
                vae_channels=(32, 64), vae_groups=8, vae_scale=2)
    base.update(kw)
    return FluxConfig(**base)


def write_folder(root, cfg, seed=0):
    from safetensors.torch import save_file
    (root / "transformer").mkdir(parents=True)
    (root / "vae").mkdir()
    (root / "scheduler").mkdir()
    (root / "transformer" / "config.json").write_text(json.dumps({
        "num_layers": cfg.n_joint, "num_single_layers": cfg.n_single, "num_attention_heads": cfg.n_heads, "attention_head_dim": cfg.head_dim,
        "in_channels": cfg.in_channels, "joint_attention_dim": cfg.text_dim, "pooled_projection_dim": cfg.pooled_dim,
        "guidance_embeds": cfg.guidance_embeds, "axes_dims_rope": list(cfg.axes_dims)}))
    (root / "vae" / "config.json").write_text(json.dumps({
        "latent_channels": cfg.latent_channels, "block_out_channels": list(cfg.vae_channels), "layers_per_block": cfg.vae_layers,
        "norm_num_groups": cfg.vae_groups, "scaling_factor": cfg.scaling_factor, "shift_factor": cfg.shift_factor}))
    (root / "scheduler" / "scheduler_config.json").write_text(json.dumps({"use_dynamic_shifting": cfg.dynamic_shift}))
    w = random_weights(transformer_shapes(cfg), seed)
    names = sorted(w)
    half = len(names) // 2                                       # two shards with an index, as the published folders have
    save_file({n: w[n] for n in names[:half]}, str(root / "transformer" / "diffusion_pytorch_model-00001-of-00002.safetensors"))
    save_file({n: w[n] for n in names[half:]}, str(root / "transformer" / "diffusion_pytorch_model-00002-of-00002.safetensors"))
    (root / "transformer" / "diffusion_pytorch_model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        n: f"diffusion_pytorch_model-0000{1 if i < half else 2}-of-00002.safetensors" for i, n in enumerate(names)}}))
    save_file(random_weights(vae_shapes(cfg), seed + 1), str(root / "vae" / "diffusion_pytorch_model.safetensors"))
    return w


def test_tensor_layout_of_the_published_model():
    """The full-size layout has the published parameter count (11.9 B for dev) and the names of the export."""
    s = transformer_shapes(FluxConfig())
    assert sum(math.prod(v) for v in s.values()) == 11_901_408_320
    assert s["single_transformer_blocks.37.proj_out.weight"] == (3072, 15360) and s["transformer_blocks.18.attn.norm_added_k.weight"] == (128,)
    assert "time_text_embed.guidance_embedder.linear_1.weight" not in transformer_shapes(FluxConfig(guidance_embeds=False))
    v = vae_shapes(FluxConfig())
    assert sum(math.prod(x) for x in v.values()) == 83_819_683
    assert v["decoder.up_blocks.2.resnets.0.conv_shortcut.weight"] == (256, 512, 1, 1) and v["encoder.conv_out.weight"] == (32, 512, 3, 3)


def test_rotary_tables_are_the_complex_rotation():
    ids = torch.tensor([[0, 0, 0], [0, 3, 5], [1, 2, 7]])
    cos, sin = rope_tables(ids, (8, 12, 12), 10000.0)
    assert cos.shape == (3, 32) and torch.allclose(cos[0], torch.ones(32)) and torch.allclose(sin[0], torch.zeros(32))
    x = torch.randn(2, 3, 32)
    got = rope_apply(x, cos, sin)
    ang = torch.cat([ids[:, i:i + 1].double() / (10000.0 ** (torch.arange(0, d, 2).double() / d)) for i, d in enumerate((8, 12, 12))], 1)
    want = torch.view_as_real(torch.view_as_complex(x.double().reshape(2, 3, 16, 2)) * torch.polar(torch.ones_like(ang), ang)).reshape(2, 3, 32)
    assert torch.allclose(got.double(), want, atol=1e-5)
    # relative: the score of two tokens depends on their offset only
    q, k = torch.randn(1, 1, 32), torch.randn(1, 1, 32)
    def score(a, b):
        ca, sa = rope_tables(torch.tensor([a]), (8, 12, 12), 10000.0)
        cb, sb = rope_tables(torch.tensor([b]), (8, 12, 12), 10000.0)
        return float((rope_apply(q, ca, sa) * rope_apply(k, cb, sb)).sum())
    assert abs(score([0, 2, 3], [0, 5, 9]) - score([0, 12, 13], [0, 15, 19])) < 1e-4


def test_schedule_follows_the_token_count():
    m = FluxModel.random(tiny())
    a, b = m.schedule(4, 256), m.schedule(4, 4096)
    assert a[0] == b[0] == 1.0 and a[-1] == b[-1] == 0.0 and all(x > y for x, y in zip(a[:-1], a[1:]))
    assert all(y >= x for x, y in zip(a, b)) and b[2] > a[2]                   # more tokens: more time near the noisy end
    mu = 0.5
    assert abs(a[1] - math.exp(mu) / (math.exp(mu) + (1 / 0.75 - 1))) < 1e-9   # 256 tokens: the base shift
    s = FluxModel.random(tiny(guidance_embeds=False, dynamic_shift=False))
    assert s.schedule(4, 1024) == [1.0, 0.75, 0.5, 0.25, 0.0] and s.default_steps["medium"] == 2 and m.default_steps["medium"] == 25


def test_checkpoint_folder_loads_whole_and_by_stage(tmp_path):
    cfg = tiny()
    w = write_folder(tmp_path / "FLUX.1-dev", cfg)
    m = FluxModel.from_folder(tmp_path / "FLUX.1-dev", device="cpu", dtype=torch.float32, text=False)
    assert m.cfg.n_joint == 2 and m.cfg.guidance_embeds and m.cfg.dynamic_shift and not m.cfg.kontext and m.cfg.vae_scale == 2
    assert m.cfg.text_len == 512                                               # dev's T5 length; schnell's is 256
    ref = FluxModel(m.cfg, w, FluxVAE(cfg, random_weights(vae_shapes(cfg), 1), "cpu"))
    lat = torch.randn(16, 8, 12)
    txt, pooled = m.encode_text("a red fox")
    v = m.velocity(lat, 0.7, txt, pooled)
    assert v.shape == lat.shape and torch.equal(v, ref.velocity(lat, 0.7, *ref.encode_text("a red fox")))
    assert not torch.allclose(v, m.velocity(lat, 0.3, txt, pooled)) and not torch.allclose(v, m.velocity(lat, 0.7, *m.encode_text("a whale")))
    m.guidance_value = 1.0
    assert not torch.allclose(v, m.velocity(lat, 0.7, txt, pooled))            # the guidance scale is an input
    m.guidance_value = cfg.guidance
    # two stages hold disjoint blocks and chain to the same prediction
    s0 = FluxModel.from_folder(tmp_path / "FLUX.1-dev", blocks=range(0, 3), device="cpu", dtype=torch.float32, text=False)
    s1 = FluxModel.from_folder(tmp_path / "FLUX.1-dev", blocks=range(3, 4), device="cpu", dtype=torch.float32, text=False)
    assert not any(n.startswith("single_transformer_blocks.1.") for n in s0.w) and not any(n.startswith("transformer_blocks.") for n in s1.w)
    vec = s0.time_vec(0.7, pooled)
    t1, i1 = s0.run_blocks(txt, s0.embed_tokens(lat, 4, 6), vec, grid=(4, 6))
    _, i2 = s1.run_blocks(t1, i1, vec, grid=(4, 6))
    assert torch.allclose(s1.head(i2, 4, 6, vec), v, atol=1e-5)
    img = m.decode(lat)
    assert img.shape == (16, 24, 3) and img.dtype == torch.uint8
    assert m.encode_image(img, 4, 6).shape == (16, 8, 12)
    # a tensor of the wrong shape is refused by name
    from safetensors.torch import load_file, save_file
    f = tmp_path / "FLUX.1-dev" / "transformer" / "diffusion_pytorch_model-00001-of-00002.safetensors"
    d = load_file(str(f))
    k = next(n for n in d if n.endswith("to_q.weight"))
    d[k] = d[k][:, :32].contiguous()
    save_file(d, str(f))
    with pytest.raises(ValueError, match="to_q.weight"):
        FluxModel.from_folder(tmp_path / "FLUX.1-dev", device="cpu", dtype=torch.float32, text=False)


def test_sampler_and_kontext_reference_image():
    r = DiffusionRunner(FluxModel.random(tiny()))
    a = list(r.generate("a red fox", 32, 48, 3, 7))[-1][1]
    assert a.shape == (32, 48, 3) and torch.equal(a, list(r.generate("a red fox", 32, 48, 3, 7))[-1][1])
    assert not torch.equal(a, list(r.generate("a red fox", 32, 48, 3, 8))[-1][1])
    assert not torch.equal(a, list(r.generate("a red fox", 32, 48, 3, 7, guidance=1.5))[-1][1])
    k = DiffusionRunner(FluxModel.random(tiny(kontext=True)))
    ref1, ref2 = torch.zeros(32, 48, 3, dtype=torch.uint8), torch.full((32, 48, 3), 200, dtype=torch.uint8)
    b1 = list(k.generate("make it night", 32, 48, 3, 7, init_image=ref1))[-1][1]
    b2 = list(k.generate("make it night", 32, 48, 3, 7, init_image=ref2))[-1][1]
    assert b1.shape == (32, 48, 3) and not torch.equal(b1, b2)                 # the reference picture conditions the result
    assert k.m.context is not None and k.m.context.shape == (8 * 12, 64)
    c = list(k.generate("make it night", 32, 48, 3, 7))[-1][1]
    assert k.m.context is None and not torch.equal(c, b1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, port, mode, q, world=2):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = tiny(kontext=mode == "kontext")
        per = cfg.n_blocks // world
        model = FluxModel.random(cfg, blocks=range(rank * per, (rank + 1) * per))
        r = DiffusionRunner(model, rank=rank, world=world, num_sync_steps=99 if mode == "pipe_sync" else 1,
                            pipe_groups=[dist.new_group(list(range(world)))])
        r.async_patches = mode != "step_by_step"
        init = torch.full((32, 48, 3), 90, dtype=torch.uint8) if mode == "kontext" else None
        calls = [0]

        def agree() -> bool:                 # what the serving engine does: a host-side collective every time it is asked
            calls[0] += 1
            flag = torch.tensor([1.0 if (mode == "cancelled" and calls[0] == 3) else 0.0])
            dist.all_reduce(flag)
            return bool(flag.item())
        long = mode in ("cancel_checks", "cancelled")
        out = list(r.generate("a red fox", 32, 48, 10 if long else 4, 7, init_image=init, partial_images=1 if mode == "previews" else 0,
                              **({"should_stop": agree} if long else {})))
        if mode == "cancelled":
            q.put((rank, torch.zeros(1), calls[0], out))
            return
        q.put((rank, out[-1][1], r.n_patch_hops, [o[1] for o in out[:-1]]))
    finally:
        dist.destroy_process_group()


def _run_ranks(mode, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, port, mode, q, world)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (img, hops, prev)) for r, img, hops, prev in (q.get(timeout=180) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return got


def test_patches_flowing_across_steps_equal_the_step_by_step_schedule():
    """The continuous patch flow (rows go from the last stage straight back to the first) computes exactly what the
    step-by-step patch schedule computes; four stages keep every pair's messages in order; previews reach every rank."""
    a, b = _run_ranks("pipefusion"), _run_ranks("step_by_step")
    assert torch.equal(a[0][0], a[1][0]) and (a[0][0].float() - b[0][0].float()).abs().max() <= 1 and a[0][1] == b[0][1] == 6
    four = _run_ranks("pipefusion", world=4)
    assert all(torch.equal(four[0][0], four[r][0]) for r in range(4)) and four[0][1] == 3 * 4 and four[3][1] == 0
    # ten steps: cancellation is agreed on at steps 0, 1 (whole-image steps) and then every fourth patch step, without stalling the flow
    cc = _run_ranks("cancel_checks")
    assert torch.equal(cc[0][0], cc[1][0]) and cc[0][1] == 9 * 2
    stopped = _run_ranks("cancelled")
    assert stopped[0][1] == stopped[1][1] == 3 and stopped[0][2] == [] and stopped[1][2] == []      # both ranks left at the same check
    pv = _run_ranks("previews")
    assert len(pv[0][2]) == 1 and torch.equal(pv[0][2][0], pv[1][2][0]) and pv[0][2][0].shape == (32, 48, 3)


@pytest.mark.parametrize("mode", ["pipe_sync", "pipefusion", "kontext"])
def test_two_stage_schedules_against_single_rank(mode):
    init = torch.full((32, 48, 3), 90, dtype=torch.uint8) if mode == "kontext" else None
    want = list(DiffusionRunner(FluxModel.random(tiny(kontext=mode == "kontext"))).generate("a red fox", 32, 48, 4, 7, init_image=init))[-1][1]
    got = _run_ranks(mode)
    assert torch.equal(got[0][0], got[1][0])
    diff = (got[0][0].float() - want.float()).abs()
    if mode == "pipe_sync":
        assert got[0][1] == 0 and diff.max() <= 1
    else:
        assert got[0][1] == 3 * 2 and diff.mean() < 40             # stale keys / values of the other patch: close, not equal


def test_image_builder_serves_a_checkpoint_folder(tmp_path, monkeypatch):
    """A card whose folder is on disk loads as FLUX (this stage's blocks), takes the model's step counts per quality
    level, and streams an image through the engine; an edit request on a Kontext folder uses the reference picture."""
    import base64
    import io
    from PIL import Image
    from exo_b200.api.types import AdvancedImageParams, ImageEditsTaskParams, ImageGenerationTaskParams
    from exo_b200.shared.base import InstanceId, Memory, ModelId, NodeId, RunnerId
    from exo_b200.shared.cards import ModelCard
    from exo_b200.shared.messages import ImageEdits, ImageGeneration
    from exo_b200.shared.wire import BoundInstance, ImageChunk, NvlinkInstance, PipelineShardMetadata, ShardAssignments
    from exo_b200.worker.engines.base import Finished
    from exo_b200.worker.engines.image.builder import ImageBuilder, decode_image
    monkeypatch.setenv("EXO_DEVICE", "cpu")
    root = tmp_path / "FLUX.1-Kontext-dev"
    write_folder(root, tiny(guidance_embeds=False, dynamic_shift=False, vae_channels=(32, 32, 64, 64), vae_scale=8))   # schnell-like: 1 / 2 / 4 steps
    card = ModelCard(model_id=ModelId(str(root)), storage_size=Memory.from_mb(1), n_layers=4, hidden_size=64, supports_tensor=False,
                     tasks=["TextToImage", "ImageToImage"], family="flux")
    node, rid = NodeId("n0"), RunnerId("r0")
    inst = NvlinkInstance(instance_id=InstanceId("img"), shard_assignments=ShardAssignments(
        model_id=card.model_id, runner_to_shard={rid: PipelineShardMetadata(model_card=card, device_rank=0, world_size=1, start_layer=0,
                                                                            end_layer=4, n_layers=4)},
        node_to_runner={node: rid}), rendezvous_port=1, gpu_by_node={node: 0})
    b = ImageBuilder(BoundInstance(instance=inst, bound_runner_id=rid, bound_node_id=node))
    b.connect()
    progress = list(b.load())
    assert isinstance(b.model, FluxModel) and b.model.cfg.kontext and progress[-1].layers_loaded == 4
    eng = b.build()

    def run(task):
        eng.submit(task)
        chunks, end = [], None
        while eng.has_work:
            for _tid, item in eng.step():
                if isinstance(item, ImageChunk):
                    chunks.append(item)
                else:
                    end = item
        assert isinstance(end, Finished)
        return decode_image(base64.b64decode("".join(c.data for c in sorted(chunks, key=lambda c: c.chunk_index)))), chunks
    p = ImageGenerationTaskParams(prompt="a boat", model=str(root), size="256x256", quality="high", bench=True, advanced_params=AdvancedImageParams(seed=5))
    img, chunks = run(ImageGeneration(instance_id=inst.instance_id, command_id="c", task_params=p))
    assert img.shape == (256, 256, 3) and chunks[-1].stats.num_inference_steps == 4
    buf = io.BytesIO()
    Image.fromarray(torch.full((64, 96, 3), 180, dtype=torch.uint8).numpy()).save(buf, format="PNG")
    e = ImageEditsTaskParams(prompt="at night", model=str(root), image_data=base64.b64encode(buf.getvalue()).decode(), quality="low",
                             advanced_params=AdvancedImageParams(seed=5))
    edited, _ = run(ImageEdits(instance_id=inst.instance_id, command_id="c2", task_params=e))
    assert edited.shape == (64, 96, 3) and b.model.context is not None


def test_text_encoders_load_from_the_checkpoint_folder(tmp_path):
    """``text_encoder/`` (CLIP) and ``text_encoder_2/`` (T5) with their tokenizers, as the published folders lay them out: the
    prompt becomes T5 token features (projected to the model width) and CLIP's pooled vector, and conditions the prediction."""
    tf = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models, pre_tokenizers, processors
    cfg = tiny(text_dim=48, pooled_dim=24)
    root = tmp_path / "FLUX.1-schnell"
    write_folder(root, tiny(guidance_embeds=False, dynamic_shift=False))
    vocab = {w: i for i, w in enumerate(["<pad>", "</s>", "<unk>", "a", "red", "fox", "blue", "whale", "on", "the", "hill"])}
    for sub, max_len in (("tokenizer", 12), ("tokenizer_2", 256)):
        t = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
        t.pre_tokenizer = pre_tokenizers.Whitespace()
        t.post_processor = processors.TemplateProcessing(single="$A </s>", special_tokens=[("</s>", 1)])      # CLIP pools at the end token
        (root / sub).mkdir()
        t.save(str(root / sub / "tokenizer.json"))
        (root / sub / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast", "model_max_length": max_len,
                                                                      "pad_token": "<pad>", "eos_token": "</s>", "unk_token": "<unk>"}))
    torch.manual_seed(0)
    tf.CLIPTextModel(tf.CLIPTextConfig(vocab_size=len(vocab), hidden_size=24, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2,
                                       max_position_embeddings=12, eos_token_id=1, pad_token_id=0, bos_token_id=2)).save_pretrained(root / "text_encoder")
    tf.T5EncoderModel(tf.T5Config(vocab_size=len(vocab), d_model=48, d_kv=8, d_ff=64, num_layers=1, num_heads=2, pad_token_id=0,
                                  eos_token_id=1, decoder_start_token_id=0)).save_pretrained(root / "text_encoder_2")
    m = FluxModel.from_folder(root, device="cpu", dtype=torch.float32)
    assert m.text is not None and m.cfg.text_len == 256 and not m.cfg.guidance_embeds
    txt, pooled = m.encode_text("a red fox on the hill")
    assert txt.shape == (256, m.cfg.hidden) and pooled.shape == (24,)
    txt2, pooled2 = m.encode_text("a blue whale")
    assert not torch.allclose(txt[:3], txt2[:3]) and not torch.allclose(pooled, pooled2)
    lat = torch.randn(16, 8, 12)
    v1, v2 = m.velocity(lat, 0.5, txt, pooled), m.velocity(lat, 0.5, txt2, pooled2)
    assert v1.shape == lat.shape and not torch.allclose(v1, v2)
    img = list(DiffusionRunner(m).generate("a red fox", 32, 48, 2, 3))[-1][1]
    assert img.shape == (32, 48, 3)
