"""Checkpoint families: ``config.json`` → engine config, and checkpoint tensor names → sharded weights.

Each case writes a tiny ``config.json`` in the published layout of one family, checks the fields the engine derives
from it, writes a random checkpoint under that family's tensor names and compares the engine's greedy tokens with the
fp32 oracle that reads the same names independently.
"""
import json

import pytest
import torch

from exo_b200.engine.engine import Engine
from exo_b200.engine.kv import SamplingParams
from exo_b200.models.config import ModelConfig
from exo_b200.models.oracle import OracleModel
from exo_b200.models.weights import RandomSource, SafetensorsSource, ShardSpec, build_weights, write_safetensors

BASE = {"hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 32,
        "intermediate_size": 256, "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "max_position_embeddings": 512}

CASES = {
    "ministral": ({"model_type": "ministral3", "architectures": ["Ministral3ForCausalLM"]},
                  dict(family="llama", is_moe=False)),
    "mistral3-nested": ({"model_type": "mistral3", "text_config": {**BASE, "model_type": "ministral3"}},
                        dict(family="llama", is_moe=False)),
    "mixtral": ({"model_type": "mixtral", "num_local_experts": 4, "num_experts_per_tok": 2},
                dict(family="mixtral", is_moe=True, n_experts=4, router="softmax", first_dense_layers=0)),
    "glm4-moe": ({"model_type": "glm4_moe", "n_routed_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64,
                  "n_shared_experts": 1, "first_k_dense_replace": 1, "attention_bias": True, "use_qk_norm": True,
                  "partial_rotary_factor": 0.5, "norm_topk_prob": True, "routed_scaling_factor": 1.5, "n_group": 1,
                  "topk_group": 1},
                 dict(family="glm4_moe", is_moe=True, router="sigmoid", router_bias=True, qk_norm=True, attn_bias=True,
                      first_dense_layers=1, routed_scaling=1.5)),
    "glm4-moe-lite": ({"model_type": "glm4_moe_lite", "n_routed_experts": 8, "num_experts_per_tok": 2,
                       "moe_intermediate_size": 64, "n_shared_experts": 1, "first_k_dense_replace": 1, "q_lora_rank": 64,
                       "kv_lora_rank": 32, "qk_nope_head_dim": 16, "qk_rope_head_dim": 16, "v_head_dim": 16,
                       "norm_topk_prob": True, "routed_scaling_factor": 1.0, "n_group": 1, "topk_group": 1},
                      dict(family="deepseek_v3", mla=True, is_moe=True, router="sigmoid")),
    "glm5": ({"model_type": "glm_moe_dsa", "n_routed_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64,
              "n_shared_experts": 1, "mlp_layer_types": ["dense", "sparse"], "q_lora_rank": 64, "kv_lora_rank": 32,
              "qk_nope_head_dim": 24, "qk_rope_head_dim": 16, "v_head_dim": 32, "norm_topk_prob": True,
              "routed_scaling_factor": 2.5, "n_group": 1, "topk_group": 1, "index_topk": 2048, "index_head_dim": 128,
              "index_n_heads": 32},
             dict(family="deepseek_v3", mla=True, is_moe=True, router="sigmoid", first_dense_layers=1, v_head_dim=32)),
    "minimax": ({"model_type": "minimax_m2", "num_local_experts": 8, "num_experts_per_tok": 2, "use_qk_norm": True,
                 "rotary_dim": 16},
                dict(family="minimax", is_moe=True, router="sigmoid", router_bias=True, qk_norm_full=True, moe_ffn=256)),
    "qwen3-next": ({"model_type": "qwen3_next", "num_hidden_layers": 4, "linear_num_key_heads": 2, "linear_num_value_heads": 4,
                    "linear_key_head_dim": 32, "linear_value_head_dim": 32, "linear_conv_kernel_dim": 4, "num_experts": 8,
                    "num_experts_per_tok": 2, "moe_intermediate_size": 64, "shared_expert_intermediate_size": 64,
                    "decoder_sparse_step": 1, "mlp_only_layers": [1], "norm_topk_prob": True, "rms_norm_eps": 1e-6},
                   dict(family="qwen3_next", is_moe=True, router="softmax", qk_norm=True, attn_gate=True, norm_one_plus=True,
                        layer_types=("linear", "linear", "linear", "full"), lin_split_proj=False, shared_expert_gate=True,
                        mlp_only_layers=(1,))),
    "qwen3.5": ({"model_type": "qwen3_5", "text_config": {**BASE, "model_type": "qwen3_5_text", "num_hidden_layers": 3,
                                                          "layer_types": ["linear_attention", "full_attention", "linear_attention"],
                                                          "linear_num_key_heads": 2, "linear_num_value_heads": 2,
                                                          "linear_key_head_dim": 32, "linear_value_head_dim": 64,
                                                          "rope_parameters": {"rope_theta": 50000.0, "rope_type": "default",
                                                                              "partial_rotary_factor": 0.5}}},
                dict(family="qwen3_next", is_moe=False, lin_split_proj=True, weight_prefix="model.language_model.",
                     layer_types=("linear", "full", "linear"), attn_gate=True)),
    "gemma4-multimodal": ({"model_type": "gemma4", "text_config": {**BASE, "model_type": "gemma4_text", "num_hidden_layers": 6,
                                                                    "head_dim": 32, "global_head_dim": 64, "sliding_window": 16,
                                                                    "hidden_size_per_layer_input": 8, "attention_k_eq_v": True,
                                                                    "num_global_key_value_heads": 1, "num_kv_shared_layers": 2,
                                                                    "final_logit_softcapping": 30.0}},
                          dict(family="gemma4", weight_prefix="model.language_model.", k_eq_v=True, global_kv_heads=1, ple_dim=8,
                               kv_shared_layers=2, act="gelu_tanh", logit_softcap=30.0, sliding_window=16,
                               layer_types=("sliding",) * 5 + ("full",))),
    "nemotron-h-pattern": ({"model_type": "nemotron_h", "hybrid_override_pattern": "M-M*ME", "ssm_state_size": 64, "mamba_num_heads": 8,
                            "mamba_head_dim": 32, "n_groups": 2, "conv_kernel": 4, "n_routed_experts": 8, "num_experts_per_tok": 2,
                            "moe_intermediate_size": 64, "moe_shared_expert_intermediate_size": 96, "layer_norm_epsilon": 1e-5},
                           dict(family="nemotron_h", n_layers=6, block_types=("mamba", "mlp", "mamba", "attention", "mamba", "moe"),
                                layer_types=("linear", "full", "linear", "full", "linear", "full"), act="relu2", router="sigmoid",
                                lin_k_heads=2, lin_k_dim=64, lin_v_heads=8, lin_v_dim=32, shared_expert_ffn=96,
                                weight_prefix="backbone.")),
    "step3.5": ({"model_type": "step3p5", "architectures": ["Step3p5ForCausalLM"], "num_hidden_layers": 4, "num_attention_groups": 2,
                 "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention", "full_attention"],
                 "sliding_window": 8, "attention_other_setting": {"attention_type": "sliding_attention", "num_attention_heads": 8,
                                                                  "num_attention_groups": 2, "head_dim": 32},
                 "use_head_wise_attn_gate": True, "rope_theta": [500000.0, 10000.0, 10000.0, 500000.0, 500000.0],
                 "partial_rotary_factors": [0.5, 1.0, 1.0, 0.5, 0.5], "yarn_only_types": ["full_attention"],
                 "rope_scaling": {"rope_type": "llama3", "factor": 2.0, "original_max_position_embeddings": 64, "low_freq_factor": 1.0,
                                  "high_freq_factor": 4.0},
                 "moe_num_experts": 8, "moe_top_k": 2, "moe_intermediate_size": 64, "share_expert_dim": 96, "moe_layers_enum": "1,2,3",
                 "norm_expert_weight": True, "moe_router_activation": "sigmoid", "moe_router_scaling_factor": 3.0,
                 "use_moe_router_bias": True, "need_fp32_gate": True, "swiglu_limits": [0, 0, 0.08, 0.08, 0],
                 "swiglu_limits_shared": [0.05, 0, 0, 0.06, 0], "num_nextn_predict_layers": 1, "att_impl_type": "GQA"},
                dict(family="step3p5", is_moe=True, router="sigmoid", router_bias=True, routed_scaling=3.0, norm_topk_prob=True,
                     qk_norm=True, norm_one_plus=True, head_gate=True, n_kv_heads=2, layer_n_heads=(4, 8, 8, 4), sliding_window=8,
                     layer_types=("full", "sliding", "sliding", "full"), mlp_only_layers=(0,), shared_expert_ffn=96, moe_ffn=64,
                     swiglu_limits=(0.0, 0.0, 0.08, 0.08, 0.0))),
    "qwen2": ({"model_type": "qwen2", "tie_word_embeddings": True}, dict(family="llama", attn_bias=True, tie_embeddings=True)),
}


def write_config(d, extra):
    d.mkdir(parents=True, exist_ok=True)
    cfg = extra if "text_config" in extra else {**BASE, **extra}
    (d / "config.json").write_text(json.dumps(cfg))
    return ModelConfig.from_pretrained(d)


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_json_of_each_family_maps_to_engine_fields(name, tmp_path):
    extra, want = CASES[name]
    cfg = write_config(tmp_path / name, extra)
    for k, v in want.items():
        assert getattr(cfg, k) == v, (name, k, getattr(cfg, k), v)
    if name == "glm4-moe":
        assert cfg.rope.partial_rotary_factor == 0.5
    if name == "qwen3-next":
        assert cfg.rope.partial_rotary_factor == 0.25 and [cfg.layer_is_moe(i) for i in range(4)] == [True, False, True, True]
    if name == "qwen3.5":
        assert cfg.rope.partial_rotary_factor == 0.5 and cfg.rope.theta == 50000.0
    if name == "step3.5":
        assert [cfg.window_of(i) for i in range(4)] == [0, 8, 8, 0] and [cfg.layer_is_moe(i) for i in range(4)] == [False, True, True, True]
        assert [(r.theta, r.partial_rotary_factor, r.kind) for r in cfg.layer_rope] == [
            (500000.0, 0.5, "llama3"), (10000.0, 1.0, "default"), (10000.0, 1.0, "default"), (500000.0, 0.5, "llama3")]
        assert cfg.swiglu_limit(0, shared=True) == 0.05 and cfg.swiglu_limit(2) == 0.08 and cfg.swiglu_limit(9) == 0.0


class Recorder(RandomSource):
    """A random source that remembers every tensor it was asked for, to write them out as a checkpoint."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.seen: dict[str, torch.Tensor] = {}

    def get(self, name, shape=None):
        if name in self.seen:
            return self.seen[name]
        t = super().get(name, shape)
        if name.endswith("e_score_correction_bias"):         # non-zero, so the selection bias matters to the tokens
            t = torch.empty(shape).normal_(0.0, 0.1, generator=self._gen(name))
        self.seen[name] = t
        return t


@pytest.mark.parametrize("name", ["mixtral", "glm4-moe", "glm4-moe-lite", "glm5", "ministral", "minimax", "qwen3-next", "qwen3.5"])
def test_checkpoint_under_family_names_loads_and_matches_oracle(name, tmp_path):
    extra, _ = CASES[name]
    d = tmp_path / name
    cfg = write_config(d, extra)
    cfg.dtype = "fp32"
    rec = Recorder(seed=3, std=0.05)
    oracle = OracleModel(cfg, rec)
    prompt_t = torch.randint(0, cfg.vocab, (17,), generator=torch.Generator().manual_seed(1))
    prompt = [int(t) for t in prompt_t]
    want = oracle.greedy(prompt_t, 6)
    build_weights(cfg, ShardSpec(), rec, device="cpu")        # touch every tensor the engine reads (unrouted experts too)
    names = set(rec.seen)
    if name == "mixtral":
        assert any(".block_sparse_moe.experts.0.w1.weight" in n for n in names) and not any(".mlp." in n for n in names)
    if name == "minimax":
        assert any(n.endswith("block_sparse_moe.e_score_correction_bias") for n in names)
        assert rec.seen["model.layers.0.self_attn.q_norm.weight"].shape == (4 * 32,) and cfg.rope.partial_rotary_factor == 0.5
    if name == "qwen3-next":
        assert rec.seen["model.layers.0.linear_attn.in_proj_qkvz.weight"].shape == (2 * 64 + 2 * 128, 128)
        assert rec.seen["model.layers.3.self_attn.q_proj.weight"].shape == (4 * 2 * 32, 128)
        assert "model.layers.0.mlp.shared_expert_gate.weight" in names and "model.layers.1.mlp.gate_proj.weight" in names
    if name == "qwen3.5":
        assert "model.language_model.layers.0.linear_attn.in_proj_qkv.weight" in names
    if name.startswith("glm4-moe"):
        assert any(n.endswith("mlp.gate.e_score_correction_bias") for n in names)
        assert any(n.endswith("layers.0.mlp.gate_proj.weight") for n in names)       # the leading dense layer
        assert any(n.endswith("mlp.shared_experts.gate_proj.weight") for n in names)
    write_safetensors(d / "model.safetensors", {k: v.contiguous() for k, v in rec.seen.items()})
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    eng = Engine(cfg, w, n_blocks=16, device="cpu")
    got = eng.generate(prompt, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert got == want


def test_step35_hub_and_mlx_layouts_load_to_the_same_tokens(tmp_path):
    """Step-3.5 under the hub export's names (stacked experts under ``moe.``, ``share_expert`` beside it, zero-centred norms, a
    next-token-prediction layer past the decoder's depth) and under an MLX conversion's (``mlp.switch_mlp`` / ``mlp.gate`` /
    ``mlp.share_expert``, norm weights with the 1 added): both give the oracle's tokens."""
    extra, _ = CASES["step3.5"]
    d = tmp_path / "hub"
    cfg = write_config(d, extra)
    cfg.dtype = "fp32"
    rec = Recorder(seed=5, std=0.05)
    prompt_t = torch.randint(0, cfg.vocab, (21,), generator=torch.Generator().manual_seed(2))
    prompt = [int(t) for t in prompt_t]
    want = OracleModel(cfg, rec).greedy(prompt_t, 6)
    build_weights(cfg, ShardSpec(), rec, device="cpu")
    names = set(rec.seen)
    assert rec.seen["model.layers.1.self_attn.q_proj.weight"].shape == (8 * 32, 128) and rec.seen["model.layers.0.self_attn.g_proj.weight"].shape == (4, 128)
    assert rec.seen["model.layers.1.moe.gate_proj.weight"].shape == (8, 64, 128) and "model.layers.1.share_expert.down_proj.weight" in names
    assert "model.layers.0.mlp.gate_proj.weight" in names and "model.layers.1.moe.router_bias" in names
    hub = {k: v.contiguous() for k, v in rec.seen.items()}
    hub["model.layers.4.self_attn.q_proj.weight"] = torch.zeros(4, 4)            # a prediction head's layer: never read
    write_safetensors(d / "model.safetensors", hub)
    run = lambda folder: Engine(cfg, build_weights(cfg, ShardSpec(), SafetensorsSource(folder, dtype=torch.float32), device="cpu"),   # noqa: E731
                                n_blocks=16, device="cpu").generate(prompt, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert run(d) == want
    mlx = {}
    for k, v in rec.seen.items():
        k2 = (k.replace(".moe.gate.weight", ".mlp.gate.gate.weight").replace(".moe.router_bias", ".mlp.gate.router_bias")
              .replace(".moe.", ".mlp.switch_mlp.").replace(".share_expert.", ".mlp.share_expert."))
        mlx[k2] = (v + 1.0 if "norm" in k else v).contiguous()
    d2 = tmp_path / "mlx"
    write_config(d2, extra)
    write_safetensors(d2 / "model.safetensors", mlx)
    assert run(d2) == want


@pytest.mark.parametrize("wrapper,prefix", [("qwen3_vl", "model.language_model."), ("kimi_vl", "language_model.model.")])
def test_text_model_inside_a_multimodal_checkpoint_is_found(wrapper, prefix, tmp_path):
    """Multimodal repositories keep the decoder under a wrapper prefix (and other tensors beside it): the loader finds the
    text model whichever of the known layouts the repository uses."""
    inner = {**BASE, "model_type": "qwen3_vl_text"} if wrapper == "qwen3_vl" else \
        {**BASE, "model_type": "deepseek_v3", "n_routed_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64,
         "n_shared_experts": 1, "first_k_dense_replace": 1, "q_lora_rank": 64, "kv_lora_rank": 32, "qk_nope_head_dim": 16,
         "qk_rope_head_dim": 16, "v_head_dim": 16, "norm_topk_prob": True, "routed_scaling_factor": 1.0, "n_group": 1, "topk_group": 1}
    d = tmp_path / wrapper
    cfg = write_config(d, {"model_type": wrapper, "text_config": inner})
    cfg.dtype = "fp32"
    assert cfg.family == ("qwen3" if wrapper == "qwen3_vl" else "deepseek_v3")
    rec = Recorder(seed=4, std=0.05)
    flat = ModelConfig(**{**cfg.to_dict(), "rope": cfg.rope, "weight_prefix": "model."})
    oracle = OracleModel(flat, rec)
    prompt_t = torch.randint(0, cfg.vocab, (15,), generator=torch.Generator().manual_seed(2))
    want = oracle.greedy(prompt_t, 5)
    build_weights(flat, ShardSpec(), rec, device="cpu")
    tensors = {(prefix + k[len("model."):] if k.startswith("model.") else ("language_model." + k if prefix.startswith("language") else k)): v.contiguous()
               for k, v in rec.seen.items()}
    tensors["vision_tower.patch_embed.weight"] = torch.zeros(4, 4)
    write_safetensors(d / "model.safetensors", tensors)
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    eng = Engine(cfg, w, n_blocks=16, device="cpu")
    assert eng.generate([int(t) for t in prompt_t], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)) == want
