"""Checkpoint families against the ``transformers`` implementations.

For each family a tiny randomly initialised library model is exported under the hub's tensor names; the engine reads its
``config.json`` and tensors and must reproduce the library's logits over a prompt taken in two chunks and one single-token
step.  (The hybrid Qwen models, Gemma-4, Nemotron-H and GPT-OSS have files of their own.)
"""
import json

import pytest
import torch

from exo_b200.models.config import ModelConfig
from exo_b200.models.transformer import StepInputs, make_decoder, make_kv_pool
from exo_b200.models.weights import SafetensorsSource, ShardSpec, build_weights, write_safetensors

tf = pytest.importorskip("transformers")

BASE = dict(vocab_size=256, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
            max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False)
MOE = dict(n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1, first_k_dense_replace=1, n_group=2,
           topk_group=1, norm_topk_prob=True, routed_scaling_factor=2.5)
CASES = {
    "llama3-scaled": ("LlamaForCausalLM", "LlamaConfig", dict(head_dim=16, rope_parameters={
        "rope_type": "llama3", "rope_theta": 500000.0, "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 32})),
    "mistral": ("MistralForCausalLM", "MistralConfig", dict(head_dim=16, sliding_window=None)),
    "qwen2": ("Qwen2ForCausalLM", "Qwen2Config", dict(tie_word_embeddings=True)),
    "qwen3": ("Qwen3ForCausalLM", "Qwen3Config", dict(head_dim=32)),
    "qwen3-moe": ("Qwen3MoeForCausalLM", "Qwen3MoeConfig", dict(head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                                                                 norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])),
    "mixtral": ("MixtralForCausalLM", "MixtralConfig", dict(head_dim=16, num_local_experts=4, num_experts_per_tok=2, sliding_window=None)),
    "glm4-moe": ("Glm4MoeForCausalLM", "Glm4MoeConfig", dict(head_dim=16, partial_rotary_factor=0.5, use_qk_norm=True, attention_bias=True, **MOE)),
    "deepseek-v3": ("DeepseekV3ForCausalLM", "DeepseekV3Config", dict(q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                                                                      v_head_dim=16, num_key_value_heads=4, **MOE,
                                                                      rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0,
                                                                                       "original_max_position_embeddings": 32, "beta_fast": 32,
                                                                                       "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0})),
    "glm4-moe-lite": ("Glm4MoeLiteForCausalLM", "Glm4MoeLiteConfig", dict(q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                                                                          v_head_dim=16, num_key_value_heads=4, **MOE)),
    "ministral3": ("Ministral3ForCausalLM", "Ministral3Config", dict(head_dim=16, sliding_window=None)),
    "glm5": ("GlmMoeDsaForCausalLM", "GlmMoeDsaConfig", dict(q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                                                             num_key_value_heads=4, index_topk=2048, index_head_dim=16, index_n_heads=2,
                                                             mlp_layer_types=["dense", "sparse", "sparse"], **MOE)),
    "deepseek-v2-lite": ("DeepseekV2ForCausalLM", "DeepseekV2Config", dict(q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                                                                           v_head_dim=16, num_key_value_heads=4, n_routed_experts=8, num_experts_per_tok=2,
                                                                           moe_intermediate_size=32, n_shared_experts=1, first_k_dense_replace=1,
                                                                           n_group=1, topk_group=1, norm_topk_prob=False, routed_scaling_factor=1.0,
                                                                           topk_method="greedy", scoring_func="softmax")),
    "minimax-m2": ("MiniMaxM2ForCausalLM", "MiniMaxM2Config", dict(head_dim=16, num_local_experts=4, num_experts_per_tok=2, use_qk_norm=True,
                                                                   rotary_dim=8, intermediate_size=32,
                                                                   rope_parameters={"rope_type": "default", "rope_theta": 5000000.0,
                                                                                    "partial_rotary_factor": 0.5})),
}


def _step(dec, kv, toks, start):
    T = len(toks)
    n = start + T
    bt = torch.arange(1, 1 + (n + 15) // 16, dtype=torch.int32)[None]
    pos = torch.arange(start, n, dtype=torch.int32)
    inp = StepInputs(tokens=torch.tensor(toks, dtype=torch.int32), positions=pos, slots=(16 + pos).int(),
                     cu_q=torch.tensor([0, T], dtype=torch.int32), seq_lens=torch.tensor([n], dtype=torch.int32),
                     block_tables=bt, logit_rows=torch.arange(T), max_q_len=T)
    return dec.logits(inp, kv)


@pytest.mark.parametrize("name", sorted(CASES))
def test_logits_match_the_library(name, tmp_path):
    cls, cfg_cls, extra = CASES[name]
    if not hasattr(tf, cls):
        pytest.skip(f"this transformers build has no {cls}")
    torch.manual_seed(0)
    hc = getattr(tf, cfg_cls)(**{**BASE, **extra})
    hc._attn_implementation = "eager"
    model = getattr(tf, cls)(hc).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.normal_(1.0, 0.2)
            elif n.endswith("e_score_correction_bias"):
                p.uniform_(0.0, 0.5)
            elif "bias" in n:
                p.normal_(0.0, 0.2)
            else:
                p.normal_(0, 0.12)
        for n, b in model.named_buffers():
            if n.endswith("e_score_correction_bias"):
                # non-negative: the library zeroes the excluded groups' candidates where this engine removes them, which differs
                # only for a token whose candidates inside the chosen groups are all negative after the bias
                b.uniform_(0.0, 0.5)
    sd = {k: v.clone().contiguous() for k, v in model.state_dict().items()}
    if hc.tie_word_embeddings:
        sd.pop("lm_head.weight", None)
    (tmp_path / "config.json").write_text(json.dumps(hc.to_dict()))
    write_safetensors(tmp_path / "model.safetensors", sd)
    cfg = ModelConfig.from_pretrained(tmp_path)
    cfg.dtype = "fp32"
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(tmp_path, dtype=torch.float32), device="cpu")
    dec = make_decoder(cfg, w)
    kv = make_kv_pool(cfg, ShardSpec(), n_blocks=16, device="cpu", max_seqs=2)
    toks = torch.randint(0, cfg.vocab, (1, 50), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = model(toks).logits[0]
    got = torch.cat((_step(dec, kv, toks[0, :31].tolist(), 0), _step(dec, kv, toks[0, 31:49].tolist(), 31), _step(dec, kv, toks[0, 49:50].tolist(), 49)), 0)
    assert torch.allclose(got, want, atol=3e-3, rtol=3e-3), float((got - want).abs().max())
