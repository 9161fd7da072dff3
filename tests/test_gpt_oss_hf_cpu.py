"""GPT-OSS against the ``transformers`` implementation.

A tiny randomly initialised ``GptOssForCausalLM`` is exported under the hub's tensor names (interleaved gate / up columns,
biases on router and experts, attention sinks, sliding and full layers, YaRN without rounding); the engine loads it and must
reproduce the library's logits over a prompt taken in chunks and single-token steps, its greedy continuation, the same under
expert parallelism's weight split, and the 4-bit block form of the published checkpoints.
"""
import json

import pytest
import torch

from exo_b200.engine.engine import Engine
from exo_b200.engine.kv import SamplingParams
from exo_b200.models.config import ModelConfig
from exo_b200.models.transformer import StepInputs, make_decoder, make_kv_pool
from exo_b200.models.weights import SafetensorsSource, ShardSpec, build_weights, write_safetensors

tf = pytest.importorskip("transformers")
if not hasattr(tf, "GptOssForCausalLM"):
    pytest.skip("this transformers build has no GPT-OSS", allow_module_level=True)


@pytest.fixture(scope="module")
def exported(tmp_path_factory):
    torch.manual_seed(0)
    hc = tf.GptOssConfig(vocab_size=256, hidden_size=64, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=32, sliding_window=16, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=512,
                         layer_types=["sliding_attention", "full_attention"] * 2, rms_norm_eps=1e-5, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "yarn", "rope_theta": 150000.0, "factor": 4.0, "original_max_position_embeddings": 64,
                                          "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False})
    hc._attn_implementation = "eager"
    model = tf.GptOssForCausalLM(hc).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.normal_(1.0, 0.2)
            elif n.endswith("sinks"):
                p.normal_(0.0, 1.0)
            elif "bias" in n:
                p.normal_(0.0, 0.3)
            else:
                p.normal_(0, 0.15)
    d = tmp_path_factory.mktemp("gptoss")
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    write_safetensors(d / "model.safetensors", {k: v.clone().contiguous() for k, v in model.state_dict().items()})
    cfg = ModelConfig.from_pretrained(d)
    cfg.dtype = "fp32"
    return model, cfg, d


def _step(dec, kv, toks, start):
    T = len(toks)
    n = start + T
    bt = torch.arange(1, 1 + (n + 15) // 16, dtype=torch.int32)[None]
    pos = torch.arange(start, n, dtype=torch.int32)
    inp = StepInputs(tokens=torch.tensor(toks, dtype=torch.int32), positions=pos, slots=(16 + pos).int(),
                     cu_q=torch.tensor([0, T], dtype=torch.int32), seq_lens=torch.tensor([n], dtype=torch.int32),
                     block_tables=bt, logit_rows=torch.arange(T), max_q_len=T)
    return dec.logits(inp, kv)


def test_config_and_logits_match_library(exported):
    model, cfg, d = exported
    assert cfg.family == "gpt_oss" and cfg.layer_types == ("sliding", "full") * 2 and cfg.attn_sinks and cfg.attn_bias
    assert cfg.n_experts == 4 and cfg.n_experts_per_tok == 2 and cfg.act == "swiglu_oai" and cfg.expert_bias and cfg.router_linear_bias
    assert cfg.rope.kind == "yarn" and cfg.rope.truncate is False and [cfg.window_of(i) for i in range(4)] == [16, 0, 16, 0]
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    assert w.layers[0].e_gate_up.shape == (4, 128, 64) and w.layers[0].e_down.shape == (4, 64, 64) and w.layers[0].e_gate_up_b.shape == (4, 128)
    dec = make_decoder(cfg, w)
    kv = make_kv_pool(cfg, ShardSpec(), n_blocks=16, device="cpu", max_seqs=2)
    toks = torch.randint(0, cfg.vocab, (1, 60), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = model(toks).logits[0]
    got = torch.cat((_step(dec, kv, toks[0, :37].tolist(), 0), _step(dec, kv, toks[0, 37:58].tolist(), 37),     # past the window
                     _step(dec, kv, toks[0, 58:59].tolist(), 58), _step(dec, kv, toks[0, 59:60].tolist(), 59)), 0)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())


def test_engine_greedy_matches_library_and_the_expert_split_sums_to_it(exported):
    model, cfg, d = exported
    src = SafetensorsSource(d, dtype=torch.float32)
    w = build_weights(cfg, ShardSpec(), src, device="cpu")
    prompt = torch.randint(0, cfg.vocab, (1, 23), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want = model.generate(prompt, max_new_tokens=8, do_sample=False)[0, 23:].tolist()
    eng = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=16)
    assert eng.generate(prompt[0].tolist(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)) == want
    # two ranks each hold half of the experts (and half of the heads)
    halves = [build_weights(cfg, ShardSpec(tp_rank=r, tp_size=2), src, device="cpu") for r in range(2)]
    assert halves[0].layers[1].e_gate_up.shape[0] == 2 and torch.equal(halves[1].layers[1].e_down, w.layers[1].e_down[2:])
    assert torch.equal(halves[1].layers[1].e_gate_up_b, w.layers[1].e_gate_up_b[2:]) and halves[0].layers[1].router_b.shape == (4,)


def test_four_bit_block_checkpoints_load_to_their_dequantised_values(exported, tmp_path):
    """The published repositories keep the experts as ``*_blocks`` (two e2m1 codes per byte, 32 values per block, rows first)
    and ``*_scales`` (a power of two per block)."""
    from exo_b200.models.weights import _FP4_E2M1
    _, cfg, d = exported
    src = SafetensorsSource(d, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    tensors = {n: src.get(n, None) for n in src.names() if not n.endswith(("experts.gate_up_proj", "experts.down_proj"))}
    want = {}
    for i in range(cfg.n_layers):
        for part, rows, k in (("gate_up_proj", 2 * cfg.moe_ffn, cfg.hidden), ("down_proj", cfg.hidden, cfg.moe_ffn)):
            codes = torch.randint(0, 16, (cfg.n_experts, rows, k), generator=g)
            sc = torch.randint(118, 124, (cfg.n_experts, rows, k // 32), generator=g).to(torch.uint8)
            blocks = (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8).reshape(cfg.n_experts, rows, k // 32, 16)
            tensors[f"model.layers.{i}.mlp.experts.{part}_blocks"], tensors[f"model.layers.{i}.mlp.experts.{part}_scales"] = blocks, sc
            want[(i, part)] = _FP4_E2M1[codes] * torch.exp2(sc.float() - 127).repeat_interleave(32, -1)
    q = tmp_path / "blocks"
    q.mkdir()
    (q / "config.json").write_text((d / "config.json").read_text())
    write_safetensors(q / "model.safetensors", {k: v.contiguous() for k, v in tensors.items()})
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(q, dtype=torch.float32), device="cpu")
    gu = want[(2, "gate_up_proj")]
    assert torch.equal(w.layers[2].e_gate_up, torch.cat((gu[:, 0::2], gu[:, 1::2]), 1)) and torch.equal(w.layers[2].e_down, want[(2, "down_proj")])
    eng = Engine(cfg, w, n_blocks=32, device="cpu")
    assert len(eng.generate(list(range(1, 20)), SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))) == 4
