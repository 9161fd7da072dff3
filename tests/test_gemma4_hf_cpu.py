"""Gemma-4 text model against the ``transformers`` implementation.

Tiny randomly initialised ``Gemma4ForCausalLM`` models are exported under the hub's tensor names; the engine loads the
checkpoint and must reproduce the library's logits over a prompt taken in two chunks and single-token steps, and its
greedy continuation.  Variants: plain sliding / full layers; per-layer inputs + ``v = k`` on full layers with their own KV
head count + shared-KV last layers with the double-wide MLP; the expert block beside the MLP.
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
if not hasattr(tf, "Gemma4ForCausalLM"):
    pytest.skip("this transformers build has no Gemma-4", allow_module_level=True)

BASE = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
            head_dim=32, global_head_dim=64, sliding_window=16, rms_norm_eps=1e-6, max_position_embeddings=512,
            layer_types=["sliding_attention", "full_attention"] * 3, hidden_size_per_layer_input=0, vocab_size_per_layer_input=512,
            final_logit_softcapping=30.0, tie_word_embeddings=True)
VARIANTS = {
    "plain": {},
    "per-layer-inputs, v = k, shared kv": dict(hidden_size_per_layer_input=16, attention_k_eq_v=True, num_global_key_value_heads=1,
                                               num_kv_shared_layers=2, use_double_wide_mlp=True),
    "expert block": dict(enable_moe_block=True, num_experts=8, top_k_experts=2, moe_intermediate_size=64),
}


@pytest.fixture(scope="module", params=sorted(VARIANTS))
def exported(request, tmp_path_factory):
    torch.manual_seed(0)
    hc = tf.Gemma4TextConfig(**{**BASE, **VARIANTS[request.param]})
    model = tf.Gemma4ForCausalLM(hc).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n or n.endswith("scale"):
                p.normal_(1.0, 0.2)
            else:
                p.normal_(0, 0.08)
        for n, b in model.named_buffers():
            if n.endswith("layer_scalar"):
                b.fill_(0.9)
    d = tmp_path_factory.mktemp("gemma4")
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    write_safetensors(d / "model.safetensors", {k: v.clone() for k, v in model.state_dict().items() if k != "lm_head.weight"})
    cfg = ModelConfig.from_pretrained(d)
    cfg.dtype = "fp32"
    return request.param, model, cfg, d


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
    name, model, cfg, d = exported
    assert cfg.family == "gemma4" and cfg.layer_types == ("sliding", "full") * 3 and cfg.act == "gelu_tanh"
    assert cfg.attn_dims(0) == (2, 32) and cfg.attn_dims(1)[1] == 64 and cfg.logit_softcap == 30.0
    if "shared" in name:
        assert cfg.attn_dims(1) == (1, 64) and cfg.kv_source_layer(4) == 2 and cfg.kv_source_layer(5) == 3 and cfg.ple_dim == 16
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    dec = make_decoder(cfg, w)
    kv = make_kv_pool(cfg, ShardSpec(), n_blocks=16, device="cpu", max_seqs=2)
    toks = torch.randint(0, cfg.vocab, (1, 60), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = model(toks).logits[0]
    got = torch.cat((_step(dec, kv, toks[0, :37].tolist(), 0), _step(dec, kv, toks[0, 37:58].tolist(), 37),     # past the window
                     _step(dec, kv, toks[0, 58:59].tolist(), 58), _step(dec, kv, toks[0, 59:60].tolist(), 59)), 0)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())


def test_engine_greedy_matches_library(exported):
    _, model, cfg, d = exported
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    prompt = torch.randint(0, cfg.vocab, (1, 23), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want = model.generate(prompt, max_new_tokens=8, do_sample=False)[0, 23:].tolist()
    eng = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=16)
    got = eng.generate(prompt[0].tolist(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert got == want
