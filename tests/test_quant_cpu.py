"""Block-scaled fp8 weight packers and their use by the model on the CPU oracle path."""
import pytest
import torch

from exo_b200.ops import quant
from exo_b200.ops import reference as ref


@pytest.mark.parametrize("kind", ["mxfp8", "dsfp8"])
def test_roundtrip_error_and_shapes(kind):
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(200, 384, generator=g) * 0.02).bfloat16()
    q = quant.quantize(w, kind)
    assert q.q.dtype == torch.float8_e4m3fn and q.shape == w.shape
    if kind == "mxfp8":
        assert q.scale.dtype == torch.uint8 and q.scale.shape == (200, 384 // 32)
    else:
        assert q.scale.dtype == torch.float32 and q.scale.shape == (2, 3)
    d = q.dequantize().float()
    # e4m3 keeps 3 mantissa bits: relative error per weight <= 2^-4 of the block maximum's octave
    err = (d - w.float()).abs()
    blockmax = w.float().abs().max()
    assert err.max() <= blockmax * 2 ** -4
    assert err.mean() < w.float().abs().mean() * 0.04
    assert q.nbytes() < w.numel() * 1.1


def test_mxfp8_scales_are_powers_of_two_and_zero_block_is_safe():
    w = torch.zeros(4, 64)
    w[1, :32] = torch.linspace(-3, 3, 32)
    w[2, 32:] = 1e-6
    q = quant.quantize_mxfp8(w.bfloat16())
    d = q.dequantize().float()
    assert torch.isfinite(d).all()
    assert d[0].abs().sum() == 0 and d[3].abs().sum() == 0
    assert torch.allclose(d[1, :32], w[1, :32].bfloat16().float(), rtol=2 ** -4, atol=1e-3)
    assert torch.allclose(d[2, 32:], w[2, 32:].bfloat16().float(), rtol=2 ** -4)


def test_stacked_experts_and_linear():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(3, 64, 128, generator=g).bfloat16()
    q = quant.quantize(w, "mxfp8")
    assert q.scale.shape == (3, 64, 4)
    x = torch.randn(5, 128, generator=g)
    y = ref.linear(x, q[1])
    assert torch.allclose(y, x @ q[1].dequantize().float().t(), atol=1e-4)
    assert torch.allclose(y, x @ w[1].float().t(), atol=0.6, rtol=0.1)


def test_quantized_model_runs_and_tracks_the_bf16_model():
    from dataclasses import replace

    from exo_b200.models.config import preset
    from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
    cfg = replace(preset("tiny-llama"), dtype="bf16")
    qcfg = replace(cfg, quant="mxfp8")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0))
    wq = build_weights(qcfg, ShardSpec(), RandomSource(seed=0))
    lw, lq = w.layers[0], wq.layers[0]
    assert isinstance(lq.wqkv, quant.Fp8Weight) and isinstance(lq.w_gate_up, quant.Fp8Weight)
    assert isinstance(lq.w_down, torch.Tensor)      # K = 688 is not a whole number of 32-blocks: left in bf16
    assert isinstance(lq.attn_norm, torch.Tensor)
    assert torch.allclose(lq.wqkv.dequantize().float(), lw.wqkv.float(), atol=0.02 * 2 ** -3 * 4)
    assert wq.nbytes() < w.nbytes()


def test_quantized_engine_decodes_like_its_dequantised_twin():
    """The engine on fp8 weights gives the tokens of the same engine on the dequantised bf16 weights."""
    from dataclasses import replace

    from exo_b200.engine.engine import Engine
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.models.config import preset
    from exo_b200.models.weights import QUANTIZED_FIELDS, RandomSource, ShardSpec, build_weights
    cfg = replace(preset("tiny-moe"), dtype="bf16")
    qcfg = replace(cfg, quant="mxfp8")
    wq = build_weights(qcfg, ShardSpec(), RandomSource(seed=0, std=0.05))
    wd = build_weights(qcfg, ShardSpec(), RandomSource(seed=0, std=0.05))
    for lw in wd.layers.values():
        for name in QUANTIZED_FIELDS:
            v = getattr(lw, name, None)
            if isinstance(v, quant.Fp8Weight):
                setattr(lw, name, v.dequantize())
    outs = []
    for cfg_i, w in ((qcfg, wq), (cfg, wd)):
        eng = Engine(cfg_i, w, n_blocks=64, block_size=16, device="cpu")
        outs.append(eng.generate(list(range(3, 40)), SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)))
    assert outs[0] == outs[1] and len(outs[0]) == 8
