"""Family image processors and the Qwen2-VL tower against the ``transformers`` implementations of the same models."""
import numpy as np
import pytest
import torch
from PIL import Image

from exo_b200.worker.engines.b200.vision_families import (GemmaProcessor, KimiVLProcessor, QwenVLProcessor, QwenVLTower,
                                                          QwenVLTowerConfig, family_for, smart_resize)


def picture(h, w, seed=0):
    rng = np.random.default_rng(seed)
    base = rng.integers(0, 255, (h // 8 + 1, w // 8 + 1, 3), dtype=np.uint8)
    return Image.fromarray(base).resize((w, h), Image.BILINEAR)       # smooth content: resampling filters agree closely


@pytest.mark.parametrize("hw", [(300, 500), (64, 48), (2000, 1500), (28, 900)])
def test_qwen_vl_processor_matches_transformers(hw):
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor
    ref = Qwen2VLImageProcessor()
    imgs = [picture(*hw, seed=1), picture(hw[0] // 2 + 30, hw[1] // 2 + 30, seed=2)]
    want = ref(images=imgs, return_tensors="pt")
    patches, grid, tokens = QwenVLProcessor.from_config(ref.to_dict())(imgs)
    assert torch.equal(grid, want["image_grid_thw"])
    assert tokens == [int(t * h * w) // 4 for t, h, w in grid.tolist()]
    assert patches.shape == want["pixel_values"].shape
    # the layouts are identical; values differ by the resize filters' rounding to 8 bits (a few grey levels at most)
    diff = (patches - want["pixel_values"].float()).abs()
    assert diff.max() < 0.08 and diff.mean() < 2e-3, (diff.max(), diff.mean())


def test_smart_resize_bounds():
    assert smart_resize(300, 500, 28, 56 * 56, 28 * 28 * 1280) == (308, 504)
    h, w = smart_resize(4000, 6000, 28, 56 * 56, 28 * 28 * 1280)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 28 * 28 * 1280 and abs(h / w - 4000 / 6000) < 0.02
    h, w = smart_resize(10, 20, 28, 56 * 56, 28 * 28 * 1280)
    assert h * w >= 56 * 56
    with pytest.raises(ValueError):
        smart_resize(10, 4000, 28, 56 * 56, 28 * 28 * 1280)


def test_qwen_vl_tower_matches_transformers():
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
    torch.manual_seed(0)
    vc = Qwen2VLVisionConfig(depth=3, embed_dim=64, hidden_size=96, num_heads=4, mlp_ratio=4, patch_size=14,
                             spatial_merge_size=2, temporal_patch_size=2)
    vc._attn_implementation = "eager"
    hf = Qwen2VisionTransformerPretrainedModel(vc).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05)
    proc = QwenVLProcessor()
    patches, grid, tokens = proc([picture(120, 200, 3), picture(90, 60, 4)])
    with torch.no_grad():
        want = hf(patches, grid_thw=grid)
    want = getattr(want, "pooler_output", want)
    want = want[0] if isinstance(want, tuple) else want
    tower = QwenVLTower(QwenVLTowerConfig.from_config(vc.to_dict()), dict(hf.state_dict()))
    got = tower(patches, grid)
    assert got.shape == (sum(tokens), 96) == tuple(want.shape)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("family", ["qwen3_vl", "qwen3_5"])
def test_qwen3_vl_tower_matches_transformers(family):
    """The Qwen3-VL / Qwen3.5 tower (interpolated position table, tanh-GELU MLP, renamed merger) against the library's."""
    tf = pytest.importorskip("transformers")
    if family == "qwen3_vl":
        from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig as VC
        from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel as VM
        extra = {"deepstack_visual_indexes": []}
    else:
        from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5VisionConfig as VC
        from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5VisionModel as VM
        extra = {}
    torch.manual_seed(0)
    vc = VC(depth=2, hidden_size=64, intermediate_size=160, num_heads=4, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
            out_hidden_size=96, num_position_embeddings=36, **extra)
    vc._attn_implementation = "eager"
    hf = VM(vc).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05)
    proc = family_for({"model_type": family, "vision_config": vc.to_dict()}, {})
    assert proc.patch == 16 and proc.mean == (0.5, 0.5, 0.5)
    patches, grid, tokens = proc([picture(120, 200, 3), picture(90, 70, 4)])
    with torch.no_grad():
        want = hf(patches, grid_thw=grid)
    want = getattr(want, "pooler_output", want)
    want = want[0] if isinstance(want, tuple) else want
    cfg = QwenVLTowerConfig.from_config(vc.to_dict())
    assert cfg.variant == "qwen3" and cfg.mlp_dim == 160 and cfg.n_pos == 36
    got = QwenVLTower(cfg, dict(hf.state_dict()))(patches, grid)
    assert got.shape == (sum(tokens), 96) == tuple(want.shape)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


def test_gemma_processor_matches_transformers():
    from transformers.models.gemma3.image_processing_gemma3 import Gemma3ImageProcessor
    ref = Gemma3ImageProcessor(size={"height": 896, "width": 896})
    imgs = [picture(300, 500, 5), picture(1000, 700, 6)]
    want = ref(images=imgs, return_tensors="pt")["pixel_values"]
    x, grid, tokens = GemmaProcessor.from_config(ref.to_dict(), {"mm_tokens_per_image": 256})(imgs)
    assert grid is None and tokens == [256, 256] and x.shape == want.shape == (2, 3, 896, 896)
    diff = (x - want.float()).abs()
    assert diff.max() < 0.05 and diff.mean() < 2e-3, (diff.max(), diff.mean())
    rows = torch.arange(64 * 64 * 2, dtype=torch.float32).reshape(64 * 64, 2)
    pooled = GemmaProcessor.pool(rows, 256)
    assert pooled.shape == (256, 2)
    torch.testing.assert_close(pooled[0], rows.reshape(64, 64, 2)[:4, :4].reshape(16, 2).mean(0))


def test_kimi_vl_processor_grid_budget_and_padding():
    proc = KimiVLProcessor()
    patches, grid, tokens = proc([picture(100, 150, 7)])
    assert grid.tolist() == [[8, 12]] and patches.shape == (96, 3, 14, 14) and tokens == [24]   # padded 100x150 -> 112x168
    assert torch.all(patches.reshape(8, 12, 3, 14, 14)[7, :, :, 2:, :] == 0)                   # rows past pixel 100 are padding
    big = picture(2000, 3000, 8)
    patches, grid, tokens = proc([big])
    gh, gw = grid[0].tolist()
    assert (gh - 2) * (gw - 2) <= 4096 and gh % 2 == 0 and gw % 2 == 0 and abs(gh / gw - 2 / 3) < 0.05
    assert tokens == [gh * gw // 4]


def test_family_selection_from_config_json():
    assert isinstance(family_for({"model_type": "qwen2_5_vl", "vision_config": {"patch_size": 14}}), QwenVLProcessor)
    q3 = family_for({"model_type": "qwen3_vl", "vision_config": {"patch_size": 16}})
    assert q3.patch == 16 and q3.mean == (0.5, 0.5, 0.5)
    assert isinstance(family_for({"model_type": "kimi_vl"}), KimiVLProcessor)
    g = family_for({"model_type": "gemma3", "mm_tokens_per_image": 256}, {"size": {"height": 896, "width": 896}})
    assert isinstance(g, GemmaProcessor) and g.size == 896
    assert family_for({"model_type": "llama"}) is None


def test_gemma4_processor_and_tower_match_transformers():
    """Gemma-4: the aspect-preserving patch processor against the library's, and the vision encoder + multimodal embedder
    against ``Gemma4VisionModel`` / ``Gemma4MultimodalEmbedder`` on a random tiny configuration."""
    tf = pytest.importorskip("transformers")
    if not hasattr(tf, "Gemma4ForConditionalGeneration"):
        pytest.skip("this transformers build has no Gemma-4")
    from PIL import Image
    from transformers.models.gemma4.image_processing_gemma4 import Gemma4ImageProcessor
    from transformers.models.gemma4.modeling_gemma4 import Gemma4MultimodalEmbedder, Gemma4VisionModel
    from exo_b200.worker.engines.b200.vision_families import Gemma4Processor, Gemma4VisionConfig, Gemma4VisionTower, family_for
    rng = np.random.default_rng(0)
    im = Image.fromarray(rng.integers(0, 255, (150, 260, 3), dtype=np.uint8))
    proc = family_for({"model_type": "gemma4", "vision_config": {"patch_size": 16, "pooling_kernel_size": 3}}, {"max_soft_tokens": 70})
    assert isinstance(proc, Gemma4Processor)
    rows, pos, counts = proc([im])
    ref = Gemma4ImageProcessor(max_soft_tokens=70)(images=[im], return_tensors="pt")
    n = rows[0].shape[0]
    assert counts == list(ref["num_soft_tokens_per_image"]) and n == counts[0] * 9
    assert torch.equal(pos[0], ref["image_position_ids"][0, :n]) and (ref["image_position_ids"][0, n:] == -1).all()
    assert (rows[0] - ref["pixel_values"][0, :n]).abs().max() < 2 / 255
    torch.manual_seed(0)
    vc = tf.Gemma4VisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                               head_dim=16, patch_size=16, pooling_kernel_size=3, position_embedding_size=64)
    import types
    tc = types.SimpleNamespace(hidden_size=96)                  # all the embedder reads of the text configuration
    tower, emb = Gemma4VisionModel(vc).float().eval(), Gemma4MultimodalEmbedder(vc, tc).float().eval()
    with torch.no_grad():
        for m in (tower, emb):
            for name, p in m.named_parameters():
                p.normal_(1.0 if "norm" in name else 0.0, 0.2 if "norm" in name else 0.1)
        want = emb(tower(pixel_values=ref["pixel_values"], pixel_position_ids=ref["image_position_ids"]).last_hidden_state)
    weights = dict(tower.state_dict())
    weights.update({"embed_vision." + k: v for k, v in emb.state_dict().items()})
    mine = Gemma4VisionTower(Gemma4VisionConfig.from_config(vc.to_dict()), weights)
    got = mine(rows[0], pos[0])
    assert got.shape == want.shape == (counts[0], 96)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())


def test_serving_engine_uses_the_checkpoints_own_tower(tmp_path):
    """A checkpoint folder with Gemma-4 tower tensors: the serving engine expands an image to the tower's soft tokens between
    the begin / end markers, and the spliced rows are the tower's output."""
    tf = pytest.importorskip("transformers")
    if not hasattr(tf, "Gemma4ForConditionalGeneration"):
        pytest.skip("this transformers build has no Gemma-4")
    import base64
    import io
    import json
    import types
    from PIL import Image
    from safetensors.torch import save_file
    from transformers.models.gemma4.modeling_gemma4 import Gemma4MultimodalEmbedder, Gemma4VisionModel
    from exo_b200.worker.engines.b200.builder import ServingEngine
    from exo_b200.worker.engines.b200.vision_families import Gemma4Processor
    torch.manual_seed(0)
    vc = tf.Gemma4VisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                               head_dim=16, patch_size=16, pooling_kernel_size=3, position_embedding_size=64)
    tower, emb = Gemma4VisionModel(vc).float().eval(), Gemma4MultimodalEmbedder(vc, types.SimpleNamespace(hidden_size=96)).float().eval()
    sd = {"model.vision_tower." + k: v.contiguous() for k, v in tower.state_dict().items()}
    sd.update({"model.embed_vision." + k: v.contiguous() for k, v in emb.state_dict().items()})
    save_file(sd, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "gemma4", "vision_config": vc.to_dict(), "image_token_id": 7,
                                                      "boi_token_id": 5, "eoi_token_id": 6}))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"max_soft_tokens": 70}))
    eng = object.__new__(ServingEngine)
    eng.model_id, eng.vision, eng.tok = str(tmp_path), None, types.SimpleNamespace(pad_token_id=0)
    eng.cfg = types.SimpleNamespace(hidden=96)
    eng.te = types.SimpleNamespace(exe=types.SimpleNamespace(spec=types.SimpleNamespace(tp_size=1, pp_size=1), device=torch.device("cpu")))
    buf = io.BytesIO()
    Image.fromarray(np.random.default_rng(1).integers(0, 255, (120, 200, 3), dtype=np.uint8)).save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    ids, embeds, media = eng._with_images([2, 11, 7, 12, 7, 13], [b64, b64])
    assert isinstance(eng.vision[0], Gemma4Processor)
    n = embeds[0][1].shape[0]
    assert ids == [2, 11, 5] + [7] * n + [6, 12, 5] + [7] * n + [6, 13]
    assert [p for p, _ in embeds] == [3, 3 + n + 3] and [(a, b) for a, b, _ in media] == [(3, 3 + n), (6 + n, 6 + 2 * n)]
    assert embeds[0][1].shape == (n, 96) and torch.equal(embeds[0][1], embeds[1][1])


def test_kimi_k25_tower_matches_its_parts_in_vllm():
    """The Kimi-K2.5 tower against a model assembled from the pure-PyTorch pieces of the vLLM implementation in this image
    (patch embedding + position table, 2-D rotary tables and their application, the frame-pooling merger) with plain linear
    layers in place of its tensor-parallel ones."""
    kv = pytest.importorskip("vllm.model_executor.models.kimi_k25_vit")
    import torch.nn.functional as F
    from exo_b200.worker.engines.b200.vision_families import KimiTower, KimiTowerConfig
    torch.manual_seed(0)
    cfg = KimiTowerConfig(patch=14, pos_h=6, pos_w=4, pos_t=4, heads=2, layers=2, hidden=32, mlp_dim=48, out_hidden=40)
    E, H = cfg.hidden, cfg.heads
    embed = kv.MoonVision3dPatchEmbed(out_dim=E, patch_size=14, pos_emb_height=6, pos_emb_width=4, pos_emb_time=4).float()
    rope = kv.Rope2DPosEmbRepeated(E // H, 64, 64)
    w = {"patch_embed.proj.weight": embed.proj.weight.detach(), "patch_embed.proj.bias": embed.proj.bias.detach(),
         "patch_embed.pos_emb.weight": embed.pos_emb.weight.detach()}
    lin = lambda o, i: (torch.randn(o, i) * 0.2, torch.randn(o) * 0.1)          # noqa: E731
    for i in range(cfg.layers):
        b = f"encoder.blocks.{i}."
        for n, (o, k) in {"wqkv": (3 * E, E), "wo": (E, E), "mlp.fc0": (cfg.mlp_dim, E), "mlp.fc1": (E, cfg.mlp_dim)}.items():
            w[b + n + ".weight"], w[b + n + ".bias"] = lin(o, k)
        for n in ("norm0", "norm1"):
            w[b + n + ".weight"], w[b + n + ".bias"] = 1 + torch.randn(E) * 0.1, torch.randn(E) * 0.1
    w["encoder.final_layernorm.weight"], w["encoder.final_layernorm.bias"] = 1 + torch.randn(E) * 0.1, torch.randn(E) * 0.1
    w["mm_projector.pre_norm.weight"], w["mm_projector.pre_norm.bias"] = 1 + torch.randn(E) * 0.1, torch.randn(E) * 0.1
    w["mm_projector.linear_1.weight"], w["mm_projector.linear_1.bias"] = lin(4 * E, 4 * E)      # vLLM's names for proj.0 / proj.2
    w["mm_projector.linear_2.weight"], w["mm_projector.linear_2.bias"] = lin(cfg.out_hidden, 4 * E)
    grid = torch.tensor([[1, 6, 4], [2, 6, 4]])                                  # the table's own grid: no resampling on that side
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    patches = torch.randn(n, 3, 14, 14)
    with torch.no_grad():
        x = embed(patches, grid)
        fc = rope.get_freqs_cis(grid, torch.device("cpu"))
        spans = (grid[:, 0] * grid[:, 1] * grid[:, 2]).tolist()
        for i in range(cfg.layers):
            b = f"encoder.blocks.{i}."
            y = F.layer_norm(x, (E,), w[b + "norm0.weight"], w[b + "norm0.bias"])
            q, k, v = F.linear(y, w[b + "wqkv.weight"], w[b + "wqkv.bias"]).view(n, 3, H, E // H).unbind(1)
            q, k = kv.apply_rope(q, k, fc)
            outs, o = [], 0
            for s in spans:
                outs.append(F.scaled_dot_product_attention(*(t[o:o + s].transpose(0, 1)[None] for t in (q, k, v)))[0].transpose(0, 1).reshape(s, E))
                o += s
            x = x + F.linear(torch.cat(outs), w[b + "wo.weight"], w[b + "wo.bias"])
            y = F.layer_norm(x, (E,), w[b + "norm1.weight"], w[b + "norm1.bias"])
            x = x + F.linear(F.gelu(F.linear(y, w[b + "mlp.fc0.weight"], w[b + "mlp.fc0.bias"]), approximate="tanh"), w[b + "mlp.fc1.weight"], w[b + "mlp.fc1.bias"])
        x = F.layer_norm(x, (E,), w["encoder.final_layernorm.weight"], w["encoder.final_layernorm.bias"])
        m = torch.cat(kv.tpool_patch_merger(x, grid, (2, 2)))
        m = F.layer_norm(m, (E,), w["mm_projector.pre_norm.weight"], w["mm_projector.pre_norm.bias"], 1e-5).view(-1, 4 * E)
        want = F.linear(F.gelu(F.linear(m, w["mm_projector.linear_1.weight"], w["mm_projector.linear_1.bias"])),
                        w["mm_projector.linear_2.weight"], w["mm_projector.linear_2.bias"])
    got = KimiTower(cfg, dict(w))(patches, grid)
    assert got.shape == want.shape == (2 * 6 * 4 // 4, cfg.out_hidden)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), float((got - want).abs().max())
    # another grid: the position table is resampled bicubically
    tower = KimiTower(cfg, dict(w))
    e = tower._positions([(1, 8, 6)])
    ref_e = F.interpolate(w["patch_embed.pos_emb.weight"].permute(2, 0, 1)[None], size=(8, 6), mode="bicubic")[0].permute(1, 2, 0).reshape(48, E)
    assert torch.allclose(e, ref_e, atol=1e-6)
    assert tower(torch.randn(48, 3, 14, 14), torch.tensor([[8, 6]])).shape == (12, cfg.out_hidden)


def test_serving_engine_builds_qwen35_and_kimi_towers_from_checkpoint_folders(tmp_path):
    """Checkpoint folders of a Qwen3.5 model (``model.visual.*``) and of a Kimi-K2.5 model (``vision_tower.*`` + ``mm_projector.*``):
    the serving engine picks the matching processor and tower and expands an image at the family's placeholder token."""
    import base64
    import io
    import json
    import types
    from safetensors.torch import save_file
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5VisionConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5VisionModel
    from exo_b200.worker.engines.b200.builder import ServingEngine
    from exo_b200.worker.engines.b200.vision_families import KimiTower, KimiTowerConfig, KimiVLProcessor

    def engine(folder):
        eng = object.__new__(ServingEngine)
        eng.model_id, eng.vision, eng.tok = str(folder), None, types.SimpleNamespace(pad_token_id=0)
        eng.cfg = types.SimpleNamespace(hidden=96)
        eng.te = types.SimpleNamespace(exe=types.SimpleNamespace(spec=types.SimpleNamespace(tp_size=1, pp_size=1), device=torch.device("cpu")))
        return eng
    buf = io.BytesIO()
    picture(120, 200, 1).save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    # Qwen3.5
    torch.manual_seed(0)
    vc = Qwen3_5VisionConfig(depth=1, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
                             out_hidden_size=96, num_position_embeddings=36)
    q = tmp_path / "qwen"
    q.mkdir()
    save_file({"model.visual." + k: v.contiguous() for k, v in Qwen3_5VisionModel(vc).float().state_dict().items()}, str(q / "model.safetensors"))
    (q / "config.json").write_text(json.dumps({"model_type": "qwen3_5", "vision_config": vc.to_dict(), "image_token_id": 9}))
    eng = engine(q)
    ids, embeds, media = eng._with_images([1, 9, 2], [b64])
    proc, tower, ph, wrap = eng.vision
    assert isinstance(proc, QwenVLProcessor) and isinstance(tower, QwenVLTower) and tower.cfg.variant == "qwen3" and ph == 9 and wrap is None
    n = embeds[0][1].shape[0]
    assert ids == [1] + [9] * n + [2] and embeds[0][1].shape == (n, 96) and media[0][:2] == (1, 1 + n)
    # Kimi-K2.5
    cfg = KimiTowerConfig(patch=14, pos_h=8, pos_w=8, heads=2, layers=1, hidden=32, mlp_dim=48, out_hidden=96)
    E = cfg.hidden
    w = {"vision_tower.patch_embed.proj.weight": torch.randn(E, 3, 14, 14) * 0.05, "vision_tower.patch_embed.proj.bias": torch.zeros(E),
         "vision_tower.patch_embed.pos_emb.weight": torch.randn(8, 8, E) * 0.1}
    for name, (o, i) in {"wqkv": (3 * E, E), "wo": (E, E), "mlp.fc0": (48, E), "mlp.fc1": (E, 48)}.items():
        w[f"vision_tower.encoder.blocks.0.{name}.weight"], w[f"vision_tower.encoder.blocks.0.{name}.bias"] = torch.randn(o, i) * 0.1, torch.zeros(o)
    for name in ("encoder.blocks.0.norm0", "encoder.blocks.0.norm1", "encoder.final_layernorm"):
        w[f"vision_tower.{name}.weight"], w[f"vision_tower.{name}.bias"] = torch.ones(E), torch.zeros(E)
    w["mm_projector.pre_norm.weight"], w["mm_projector.pre_norm.bias"] = torch.ones(E), torch.zeros(E)
    w["mm_projector.proj.0.weight"], w["mm_projector.proj.0.bias"] = torch.randn(4 * E, 4 * E) * 0.1, torch.zeros(4 * E)
    w["mm_projector.proj.2.weight"], w["mm_projector.proj.2.bias"] = torch.randn(96, 4 * E) * 0.1, torch.zeros(96)
    k = tmp_path / "kimi"
    k.mkdir()
    save_file({n_: t.contiguous() for n_, t in w.items()}, str(k / "model.safetensors"))
    (k / "config.json").write_text(json.dumps({"model_type": "kimi_k25", "media_placeholder_token_id": 77, "vision_config": {
        "patch_size": 14, "init_pos_emb_height": 8, "init_pos_emb_width": 8, "num_attention_heads": 2, "num_hidden_layers": 1,
        "hidden_size": E, "intermediate_size": 48, "mm_hidden_size": 96}}))
    (k / "preprocessor_config.json").write_text(json.dumps({"in_token_limit": 64}))
    eng = engine(k)
    ids, embeds, _ = eng._with_images([1, 77, 2], [b64])
    proc, tower, ph, _wrap = eng.vision
    assert isinstance(proc, KimiVLProcessor) and isinstance(tower, KimiTower) and ph == 77
    n = embeds[0][1].shape[0]
    assert 0 < n <= 32 and ids == [1] + [77] * n + [2] and embeds[0][1].shape == (n, 96)
