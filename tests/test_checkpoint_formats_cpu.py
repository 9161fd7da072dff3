"""Pre-quantised checkpoints on disk (FP8 block-scaled, FP8 with a weight scale, MLX affine 4/8-bit) load to the
values of their dequantised twins, and a model built from them matches a model built from the twin."""
import json

import pytest
import torch

from exo_b200.models.weights import SafetensorsSource, write_safetensors


def _mlx_pack(w: torch.Tensor, bits: int, group: int):
    """Affine group quantisation in the MLX layout: uint32 words of 32/bits values (low bits first), per-group
    scale and bias over ``group`` input features."""
    n, k = w.shape
    g = w.float().reshape(n, k // group, group)
    lo, hi = g.min(-1).values, g.max(-1).values
    scale = ((hi - lo) / ((1 << bits) - 1)).clamp_min(1e-8)
    q = ((g - lo[..., None]) / scale[..., None]).round().clamp(0, (1 << bits) - 1).to(torch.int64).reshape(n, k)
    per = 32 // bits
    words = (q.reshape(n, k // per, per) << (torch.arange(per) * bits)).sum(-1)
    packed = (words & 0xFFFFFFFF).to(torch.int64)
    packed = torch.where(packed >= (1 << 31), packed - (1 << 32), packed).to(torch.int32).view(torch.uint32)
    deq = (q.reshape(n, k // group, group).float() * scale[..., None] + lo[..., None]).reshape(n, k)
    return packed, scale.to(torch.float16), lo.to(torch.float16), deq


@pytest.mark.parametrize("bits,group", [(4, 64), (8, 32)])
def test_mlx_affine_groups_dequantise_exactly(tmp_path, bits, group):
    g = torch.Generator().manual_seed(bits)
    w = torch.randn(24, 128, generator=g) * 0.1
    packed, scales, biases, _ = _mlx_pack(w, bits, group)
    (tmp_path / "config.json").write_text(json.dumps({"quantization": {"group_size": group, "bits": bits}}))
    write_safetensors(tmp_path / "model.safetensors", {"m.weight": packed, "m.scales": scales, "m.biases": biases,
                                                       "n.weight": w.bfloat16()})
    src = SafetensorsSource(tmp_path, dtype=torch.float32)
    assert src.stored_format("m.weight") == "mlx_affine" and src.stored_format("n.weight") == "plain"
    got = src.get("m.weight", (24, 128))
    per = 32 // bits
    q = ((packed.view(torch.int32).to(torch.int64) & 0xFFFFFFFF).unsqueeze(-1) >> (torch.arange(per) * bits)) & ((1 << bits) - 1)
    want = q.reshape(24, 128).float() * scales.float().repeat_interleave(group, -1) + biases.float().repeat_interleave(group, -1)
    assert torch.equal(got, want)
    assert (got - w).abs().max() < (0.05 if bits == 4 else 0.004)


def test_per_module_mlx_override_and_unsupported_width(tmp_path):
    w = torch.randn(8, 64) * 0.1
    packed8, s8, b8, _ = _mlx_pack(w, 8, 32)
    (tmp_path / "config.json").write_text(json.dumps({"quantization": {"group_size": 64, "bits": 4, "m": {"group_size": 32, "bits": 8}}}))
    write_safetensors(tmp_path / "model.safetensors", {"m.weight": packed8, "m.scales": s8, "m.biases": b8})
    got = SafetensorsSource(tmp_path, dtype=torch.float32).get("m.weight")
    assert got.shape == (8, 64) and (got - w).abs().max() < 0.004
    (tmp_path / "config.json").write_text(json.dumps({"quantization": {"group_size": 64, "bits": 7}}))
    with pytest.raises(ValueError, match="7-bit"):
        SafetensorsSource(tmp_path, dtype=torch.float32).get("m.weight")


def _bitstream_pack(q: torch.Tensor, bits: int) -> torch.Tensor:
    """Codes ``[n, k]`` as a little-endian bit stream per row (lowest bits first), returned as uint32 words."""
    n, k = q.shape
    b = ((q.to(torch.int64).unsqueeze(-1) >> torch.arange(bits)) & 1).reshape(n, k * bits)           # the bits in stream order
    by = (b.reshape(n, -1, 8) << torch.arange(8)).sum(-1).to(torch.uint8)
    return by.contiguous().view(torch.int32).view(torch.uint32)


@pytest.mark.parametrize("bits", [3, 5, 6])
def test_mlx_odd_bit_widths_run_across_byte_boundaries(tmp_path, bits):
    """3-, 5- and 6-bit repositories: fields run on across bytes (8 values in 3 or 5 bytes, 4 values in 3 bytes); a stacked
    expert tensor (three axes) unpacks along its last axis."""
    g = torch.Generator().manual_seed(bits)
    group, n, k = 64, 12, 128
    q = torch.randint(0, 1 << bits, (n, k), generator=g)
    scales, biases = (torch.rand(n, k // group, generator=g) * 0.01 + 0.001).half(), (torch.randn(n, k // group, generator=g) * 0.05).half()
    want = q.float() * scales.float().repeat_interleave(group, -1) + biases.float().repeat_interleave(group, -1)
    packed = _bitstream_pack(q, bits)
    assert packed.shape == (n, k * bits // 32)
    # spot-check the layout against the byte arithmetic of the format: the third 3-bit value straddles bytes 0 and 1, the second
    # 6-bit value bytes 0 and 1, the second 5-bit value bytes 0 and 1
    by = packed.view(torch.uint8)[0].to(torch.int64)
    if bits == 3:
        assert int(q[0, 2]) == int(((by[0] & 0xC0) >> 6) + ((by[1] & 0x1) << 2))
    if bits == 6:
        assert int(q[0, 1]) == int(((by[0] >> 6) & 0x03) + ((by[1] & 0x0F) << 2))
    if bits == 5:
        assert int(q[0, 1]) == int(((by[0] >> 5) & 0x07) + ((by[1] & 0x03) << 3))
    (tmp_path / "config.json").write_text(json.dumps({"quantization": {"group_size": group, "bits": bits}}))
    write_safetensors(tmp_path / "model.safetensors", {
        "m.weight": packed, "m.scales": scales, "m.biases": biases,
        "e.weight": packed.view(3, 4, -1).contiguous(), "e.scales": scales.view(3, 4, -1).contiguous(), "e.biases": biases.view(3, 4, -1).contiguous()})
    src = SafetensorsSource(tmp_path, dtype=torch.float32)
    assert torch.equal(src.get("m.weight", (n, k)), want)
    assert torch.equal(src.get("e.weight", (3, 4, k)), want.view(3, 4, k))


@pytest.mark.parametrize("mode", ["mxfp4", "nvfp4", "mxfp8"])
def test_mlx_microscaling_modes(tmp_path, mode):
    """Codes without biases: e2m1 (or e4m3) values times one scale per group — a power of two per 32 values, or an e4m3 number per
    16 values."""
    g = torch.Generator().manual_seed(1)
    n, k = 6, 64
    bits, group = (8, 32) if mode == "mxfp8" else (4, 16 if mode == "nvfp4" else 32)
    q = torch.randint(0, 1 << bits, (n, k), generator=g)
    if bits == 8:
        q = q.clamp(max=0x7E)                                   # keep away from the NaN code
        vals = q.to(torch.uint8).view(torch.float8_e4m3fn).float()
    else:
        vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])[q]
    if mode == "nvfp4":
        sc8 = torch.randint(0x20, 0x50, (n, k // group), generator=g).to(torch.uint8)
        sc = sc8.view(torch.float8_e4m3fn).float()
    else:
        sc8 = torch.randint(120, 132, (n, k // group), generator=g).to(torch.uint8)
        sc = torch.exp2(sc8.float() - 127)
    want = vals * sc.repeat_interleave(group, -1)
    per = 32 // bits
    words = (q.reshape(n, k // per, per).to(torch.int64) << (torch.arange(per) * bits)).sum(-1)
    packed = torch.where(words >= (1 << 31), words - (1 << 32), words).to(torch.int32).view(torch.uint32)
    (tmp_path / "config.json").write_text(json.dumps({"quantization": {"group_size": group, "bits": bits, "mode": mode}}))
    write_safetensors(tmp_path / "model.safetensors", {"m.weight": packed, "m.scales": sc8})
    got = SafetensorsSource(tmp_path, dtype=torch.float32).get("m.weight", (n, k))
    assert torch.equal(got, want)


def test_fp8_block_scaled_and_scaled_weights(tmp_path):
    g = torch.Generator().manual_seed(1)
    w = torch.randn(200, 300, generator=g)
    # DeepSeek layout: 128 x 128 blocks, weight_scale_inv multiplies the stored value
    nb, kb = 2, 3
    amax = torch.zeros(nb, kb)
    for i in range(nb):
        for j in range(kb):
            amax[i, j] = w[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128].abs().max()
    scale_inv = amax / 448.0
    full = scale_inv.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]
    w8 = (w / full).to(torch.float8_e4m3fn)
    # compressed-tensors layout: one scale per output channel
    ch = w.abs().amax(1, keepdim=True) / 448.0
    w8c = (w / ch).to(torch.float8_e4m3fn)
    write_safetensors(tmp_path / "model.safetensors", {"a.weight": w8, "a.weight_scale_inv": scale_inv,
                                                       "b.weight": w8c, "b.weight_scale": ch,
                                                       "c.weight": w8c, "c.weight_scale": torch.tensor(0.5)})
    src = SafetensorsSource(tmp_path, dtype=torch.float32)
    assert src.stored_format("a.weight") == "fp8_block" and src.stored_format("b.weight") == "fp8_scale"
    a = src.get("a.weight", (200, 300))
    assert torch.equal(a, w8.float() * full) and (a - w).abs().max() < 0.07 * w.abs().max()
    b = src.get("b.weight")
    assert torch.equal(b, w8c.float() * ch) and (b - w).abs().max() < 0.07 * w.abs().max()
    assert torch.equal(src.get("c.weight"), w8c.float() * 0.5)


def test_model_from_an_fp8_checkpoint_matches_the_model_from_its_dequantised_twin(tmp_path):
    """End to end through ``build_weights``: a tiny Llama stored block-scaled fp8 and the same values stored plain."""
    from exo_b200.engine.engine import Engine
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.models.config import preset
    from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
    cfg = preset("tiny-llama")
    cfg.vocab = 512
    src = RandomSource(seed=0)
    D = cfg.head_dim
    names = {"model.embed_tokens.weight": (cfg.vocab, cfg.hidden), "model.norm.weight": (cfg.hidden,), "lm_head.weight": (cfg.vocab, cfg.hidden)}
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        names.update({p + "input_layernorm.weight": (cfg.hidden,), p + "post_attention_layernorm.weight": (cfg.hidden,),
                      p + "self_attn.q_proj.weight": (cfg.n_heads * D, cfg.hidden), p + "self_attn.k_proj.weight": (cfg.n_kv_heads * D, cfg.hidden),
                      p + "self_attn.v_proj.weight": (cfg.n_kv_heads * D, cfg.hidden), p + "self_attn.o_proj.weight": (cfg.hidden, cfg.n_heads * D),
                      p + "mlp.gate_proj.weight": (cfg.ffn, cfg.hidden), p + "mlp.up_proj.weight": (cfg.ffn, cfg.hidden),
                      p + "mlp.down_proj.weight": (cfg.hidden, cfg.ffn)})
    q_dir, twin_dir = tmp_path / "fp8", tmp_path / "twin"
    q_dir.mkdir(); twin_dir.mkdir()
    stored, twin = {}, {}
    for k, shp in names.items():
        w = src.get(k, shp).float()
        if "proj" in k:
            nb, kb = -(-shp[0] // 128), -(-shp[1] // 128)
            si = torch.zeros(nb, kb)
            for i in range(nb):
                for j in range(kb):
                    si[i, j] = w[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128].abs().max() / 448.0
            full = si.repeat_interleave(128, 0)[:shp[0]].repeat_interleave(128, 1)[:, :shp[1]]
            w8 = (w / full).to(torch.float8_e4m3fn)
            stored[k], stored[k[:-len(".weight")] + ".weight_scale_inv"] = w8, si
            twin[k] = (w8.float() * full)
        else:
            stored[k], twin[k] = w, w
    write_safetensors(q_dir / "model.safetensors", stored)
    write_safetensors(twin_dir / "model.safetensors", twin)
    prompt = list(range(3, 40))
    outs = []
    for d in (q_dir, twin_dir):
        w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32))
        outs.append(Engine(cfg, w, n_blocks=32).generate(prompt, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)))
    assert outs[0] == outs[1] and len(outs[0]) == 8
