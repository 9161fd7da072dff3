"""Nemotron-H (Mamba-2 + position-free attention + relu^2 experts with a shared expert) against ``transformers``.

A tiny randomly initialised ``NemotronHForCausalLM`` is exported; the engine loads the checkpoint and must reproduce the
library's logits over a prompt taken in chunks and single-token steps (the Mamba-2 state and convolution history cross
chunk borders) and its greedy continuation.  The library's fallback path clamps the time step at ``time_step_min``,
which neither the ``mamba_ssm`` kernels nor the reference's MLX model do: the oracle's clamp is switched off.  The
fallback path's chunked scan also disagrees with the library's own token-by-token recurrence once a sequence spans more
than one chunk (0.03 on these logits at chunk 16, 1e-6 at a chunk longer than the prompt), so the oracle runs with one
chunk.
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
if not hasattr(tf, "NemotronHForCausalLM"):
    pytest.skip("this transformers build has no Nemotron-H", allow_module_level=True)


@pytest.fixture(scope="module", params=["plain", "latent experts"])
def exported(request, tmp_path_factory):
    torch.manual_seed(0)
    hc = tf.NemotronHConfig(
        vocab_size=512, hidden_size=128, layers_block_type=["mamba", "moe", "attention", "moe", "mamba", "moe"],
        num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, ssm_state_size=32, mamba_num_heads=8,
        mamba_head_dim=16, n_groups=2, conv_kernel=4, chunk_size=128, n_routed_experts=8, num_experts_per_tok=2,
        moe_intermediate_size=64, moe_shared_expert_intermediate_size=96, n_group=2, topk_group=1, routed_scaling_factor=1.5,
        moe_latent_size=48 if request.param == "latent experts" else None, max_position_embeddings=512, tie_word_embeddings=False)
    model = tf.NemotronHForCausalLM(hc).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("norm.weight") or n.endswith("norm_f.weight") or n.endswith(".D"):
                p.normal_(1.0, 0.2)
            elif n.endswith("A_log"):
                p.uniform_(-1.0, 1.0)
            elif n.endswith("dt_bias") or n.endswith("conv1d.bias"):
                p.normal_(0, 0.5)
            else:
                p.normal_(0, 0.08)
        for n, b in model.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.normal_(0, 0.1)
    for mod in model.modules():
        if hasattr(mod, "time_step_min"):
            mod.time_step_min = 0.0
    d = tmp_path_factory.mktemp("nemotron_h")
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    write_safetensors(d / "model.safetensors", {k: v.clone() for k, v in model.state_dict().items()})
    cfg = ModelConfig.from_pretrained(d)
    cfg.dtype = "fp32"
    return model, cfg, d


def _step(dec, kv, toks, start, seat=1):
    T = len(toks)
    n = start + T
    bt = torch.arange(1, 1 + (n + 15) // 16, dtype=torch.int32)[None]
    pos = torch.arange(start, n, dtype=torch.int32)
    inp = StepInputs(tokens=torch.tensor(toks, dtype=torch.int32), positions=pos, slots=(16 + pos).int(),
                     cu_q=torch.tensor([0, T], dtype=torch.int32), seq_lens=torch.tensor([n], dtype=torch.int32),
                     block_tables=bt, logit_rows=torch.arange(T), max_q_len=T, state_slots=torch.tensor([seat], dtype=torch.int32))
    return dec.logits(inp, kv)


def test_config_and_logits_match_library(exported):
    model, cfg, d = exported
    assert cfg.family == "nemotron_h" and cfg.block_types == ("mamba", "moe", "attention", "moe", "mamba", "moe")
    assert cfg.layer_types[0] == "linear" and cfg.layer_is_moe(1) and not cfg.layer_is_moe(2) and cfg.router == "sigmoid"
    assert (cfg.lin_k_heads, cfg.lin_k_dim, cfg.lin_v_heads, cfg.lin_v_dim) == (2, 32, 8, 16) and cfg.has_linear_layers
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    dec = make_decoder(cfg, w)
    kv = make_kv_pool(cfg, ShardSpec(), n_blocks=16, device="cpu", max_seqs=2)
    assert kv.layers[1] == (None, None) and kv.layers[0][1].shape == (3, 8, 32, 16)
    toks = torch.randint(0, cfg.vocab, (1, 60), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = model(toks).logits[0]
    got = torch.cat((_step(dec, kv, toks[0, :37].tolist(), 0), _step(dec, kv, toks[0, 37:58].tolist(), 37),
                     _step(dec, kv, toks[0, 58:59].tolist(), 58), _step(dec, kv, toks[0, 59:60].tolist(), 59)), 0)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())


def test_engine_greedy_matches_library(exported):
    model, cfg, d = exported
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    prompt = torch.randint(0, cfg.vocab, (1, 23), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want = model.generate(prompt, max_new_tokens=8, do_sample=False)[0, 23:].tolist()
    eng = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=16)
    got = eng.generate(prompt[0].tolist(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert got == want
