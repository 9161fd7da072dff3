"""Model architecture description shared by every engine component.

One flat dataclass covers the decoder families the framework serves: dense
Llama-style (Llama, Mistral, Qwen2/3 dense), softmax-routed MoE (Qwen3-MoE),
and DeepSeek-V3-style MLA + sigmoid-routed MoE.  It is built either from a
HuggingFace ``config.json`` (the checkpoint format the reference consumes, see
``src/exo/shared/models/model_cards.py:265-339`` in the reference for the alias
handling this mirrors) or from one of the named presets used by the benchmarks.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict, replace
from pathlib import Path
from typing import Any


@dataclass
class RopeConfig:
    theta: float = 10000.0
    kind: str = "default"  # default | linear | llama3 | yarn | proportional (zero frequencies beyond the rotary share)
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    truncate: bool = True       # YaRN: round the correction range to whole dimensions (GPT-OSS does not)
    partial_rotary_factor: float = 1.0


@dataclass
class ModelConfig:
    name: str = "model"
    family: str = "llama"  # llama | qwen3 | qwen3_moe | qwen3_next | deepseek_v3 | gpt_oss | glm4_moe | mixtral | minimax
    n_layers: int = 2
    hidden: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 688
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope: RopeConfig = field(default_factory=RopeConfig)
    tie_embeddings: bool = False
    qk_norm: bool = False  # per-head RMSNorm on q and k (Qwen3)
    qk_norm_full: bool = False  # RMSNorm over the whole q and the whole k projection, all heads together (MiniMax)
    attn_bias: bool = False
    max_position: int = 131072
    dtype: str = "bf16"  # bf16 | fp32
    # weight storage format of the linear layers
    quant: str = "none"  # none | mxfp8 (1x32 e8m0) | dsfp8 (128x128 blocks)
    # ---- MoE ----
    n_experts: int = 0
    n_experts_per_tok: int = 0
    moe_ffn: int = 0
    n_shared_experts: int = 0
    first_dense_layers: int = 0  # leading layers that keep a dense FFN
    router: str = "softmax"  # softmax | sigmoid
    norm_topk_prob: bool = True
    routed_scaling: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    router_bias: bool = False
    # ---- MLA ----
    mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_dim: int = 0
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    # ---- sliding window / sinks (GPT-OSS class) ----
    sliding_window: int = 0
    attn_sinks: bool = False
    eos_token_ids: tuple[int, ...] = ()
    # hybrid models (Qwen3-Next, Qwen3.5 / 3.6): per layer "full" (softmax attention over the paged cache) or "linear"
    # (gated delta rule over a fixed-size recurrent state); empty = every layer "full"
    layer_types: tuple[str, ...] = ()
    lin_k_heads: int = 0
    lin_v_heads: int = 0
    lin_k_dim: int = 0
    lin_v_dim: int = 0
    lin_conv: int = 4           # taps of the causal depthwise convolution in front of the delta rule
    lin_split_proj: bool = False  # checkpoint keeps in_proj_qkv / z / b / a apart (Qwen3.5) instead of qkvz / ba grouped per key head
    attn_gate: bool = False     # q_proj carries a second, per-head gate: attention output * sigmoid(gate)
    norm_one_plus: bool = False  # RMSNorm weights stored as (w - 1); folded to w when the checkpoint is read
    shared_expert_ffn: int = 0  # one shared expert of this width beside the routed ones ...
    shared_expert_gate: bool = False  # ... scaled per token by sigmoid(x . w_gate)
    moe_every: int = 1          # layer i is sparse when (i + 1) % moe_every == 0 ...
    mlp_only_layers: tuple[int, ...] = ()  # ... and i is not listed here
    weight_prefix: str = "model."  # "model.language_model." in checkpoints that wrap the text model
    # Gemma-4: "sliding" layers (local window, head_dim) alternate with "full" layers (global_head_dim, own KV head count,
    # optionally v = k), norms before AND after attention / MLP, GeGLU, optional per-layer input embeddings, optional
    # expert block beside the dense MLP, the last layers optionally re-using the KV of earlier ones
    global_head_dim: int = 0
    global_kv_heads: int = 0
    k_eq_v: bool = False
    kv_shared_layers: int = 0
    ple_dim: int = 0            # width of the per-layer input embeddings (0: none)
    ple_vocab: int = 0
    moe_beside_mlp: bool = False
    double_wide_mlp: bool = False
    logit_softcap: float = 0.0
    act: str = "silu"           # silu | gelu_tanh
    embed_scale: float = 1.0
    rope_global: RopeConfig | None = None   # RoPE of the "full" layers when it differs from `rope`
    # Nemotron-H: every layer is ONE mixer behind one norm: "mamba" (Mamba-2; its state uses the lin_* fields: groups as key
    # heads, state size as key dim, SSM heads and head dim as value heads and dim), "attention" (no position encoding),
    # "mlp" or "moe" (non-gated relu^2, sigmoid router, shared expert, optional latent projection around the experts)
    block_types: tuple[str, ...] = ()
    moe_latent: int = 0
    # Step-3.5: per-layer query-head counts, RoPE (base, rotary share, scaling only on some layer types), a sigmoid gate per
    # head on the attention output, SwiGLU outputs clamped on some layers (0 = not clamped)
    # GPT-OSS experts: a bias on the router and on both expert projections, gate / up interleaved in the checkpoint,
    # (up + 1) * gate * sigmoid(1.702 gate) with the gate capped and the up projection clamped at `oai_limit`
    mla_rope_neox: bool = False  # MLA rotary dims turn as (i, i + d/2) pairs (GLM-5) instead of adjacent pairs (DeepSeek)
    router_linear_bias: bool = False
    expert_bias: bool = False
    oai_limit: float = 7.0
    layer_n_heads: tuple[int, ...] = ()
    layer_rope: tuple[RopeConfig, ...] = ()
    head_gate: bool = False
    swiglu_limits: tuple[float, ...] = ()
    swiglu_limits_shared: tuple[float, ...] = ()

    # -------- derived --------
    @property
    def q_dim(self) -> int:
        return self.n_heads * (self.head_dim if not self.mla else self.qk_nope_dim + self.qk_rope_dim)

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        if self.block_types:
            return self.block_types[i] == "moe"
        return (self.is_moe and i >= self.first_dense_layers and (i + 1) % self.moe_every == 0
                and i not in self.mlp_only_layers)

    def layer_is_sliding(self, i: int) -> bool:
        return bool(self.layer_types) and self.layer_types[i] == "sliding"

    def q_heads(self, i: int) -> int:
        """Query heads of layer ``i`` (Step-3.5's sliding-window layers have more than its full-attention layers)."""
        return self.layer_n_heads[i] if self.layer_n_heads else self.n_heads

    def rope_of(self, i: int) -> RopeConfig:
        return self.layer_rope[i] if self.layer_rope else self.rope

    def window_of(self, i: int) -> int:
        """Sliding window of layer ``i`` (0 = every earlier key): per layer type where the model names layer types."""
        if self.family == "step3p5" or (self.family == "gpt_oss" and self.layer_types):
            return self.sliding_window if self.layer_is_sliding(i) else 0
        return self.sliding_window

    def swiglu_limit(self, i: int, shared: bool = False) -> float:
        t = self.swiglu_limits_shared if shared else self.swiglu_limits
        return float(t[i] or 0.0) if i < len(t) else 0.0

    def attn_dims(self, i: int) -> tuple[int, int]:
        """``(KV heads, head_dim)`` of layer ``i`` (Gemma-4's full-attention layers have their own)."""
        if self.family == "gemma4" and not self.layer_is_sliding(i):
            kvh = self.global_kv_heads if (self.k_eq_v and self.global_kv_heads) else self.n_kv_heads
            return kvh, self.global_head_dim or self.head_dim
        return self.n_kv_heads, self.head_dim

    def kv_source_layer(self, i: int) -> int:
        """The layer whose KV cache layer ``i`` reads: itself, or (Gemma-4, last `kv_shared_layers` layers) the last
        layer of the same type before the sharing starts."""
        first = self.n_layers - self.kv_shared_layers
        if not self.kv_shared_layers or i < first:
            return i
        for j in range(first - 1, -1, -1):
            if self.layer_types[j] == self.layer_types[i]:
                return j
        return i

    def layer_is_linear(self, i: int) -> bool:
        return bool(self.layer_types) and self.layer_types[i] == "linear"

    @property
    def has_linear_layers(self) -> bool:
        return "linear" in self.layer_types

    @property
    def lin_key_dim(self) -> int:
        return self.lin_k_heads * self.lin_k_dim

    @property
    def lin_value_dim(self) -> int:
        return self.lin_v_heads * self.lin_v_dim

    @property
    def kv_bytes_per_token_per_layer(self) -> int:
        el = 2 if self.dtype == "bf16" else 4
        if self.mla:
            return (self.kv_lora_rank + self.qk_rope_dim) * el
        return 2 * self.n_kv_heads * self.head_dim * el

    def param_count(self) -> int:
        h = self.hidden
        attn = h * self.q_dim + 2 * h * self.kv_dim + self.n_heads * self.head_dim * h
        if self.mla:
            qk = self.qk_nope_dim + self.qk_rope_dim
            attn = (h * self.q_lora_rank + self.q_lora_rank * self.n_heads * qk
                    + h * (self.kv_lora_rank + self.qk_rope_dim)
                    + self.kv_lora_rank * self.n_heads * (self.qk_nope_dim + self.v_head_dim)
                    + self.n_heads * self.v_head_dim * h)
        if self.attn_gate:
            attn += h * self.q_dim
        lin = (h * (2 * self.lin_key_dim + 2 * self.lin_value_dim + 2 * self.lin_v_heads)
               + self.lin_conv * (2 * self.lin_key_dim + self.lin_value_dim) + self.lin_value_dim * h)
        total = 0
        for i in range(self.n_layers):
            total += (lin if self.layer_is_linear(i) else attn) + 2 * h
            if self.layer_is_moe(i):
                total += self.n_experts * 3 * h * self.moe_ffn + h * self.n_experts
                total += self.n_shared_experts * 3 * h * self.moe_ffn + 3 * h * self.shared_expert_ffn
            else:
                total += 3 * h * self.ffn
        total += self.vocab * h * (1 if self.tie_embeddings else 2) + h
        return total

    def weight_bytes(self) -> int:
        per = {"none": 2.0 if self.dtype == "bf16" else 4.0, "mxfp8": 1.0 + 1 / 32, "dsfp8": 1.0 + 4 / (128 * 128)}[self.quant]
        return int(self.param_count() * per)

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    # -------- constructors --------
    @staticmethod
    def from_hf(cfg: dict[str, Any], name: str = "model") -> "ModelConfig":
        """Build from a HuggingFace ``config.json`` dict (text_config is unwrapped)."""
        wrapped = "text_config" in cfg and isinstance(cfg["text_config"], dict)      # a multimodal checkpoint around a text model
        if wrapped:
            inner = dict(cfg["text_config"])
            inner.setdefault("model_type", cfg.get("model_type", "llama"))
            cfg = inner
        mt = cfg.get("model_type", "llama")

        def g(*names: str, default: Any = None) -> Any:
            for n in names:
                if n in cfg and cfg[n] is not None:
                    return cfg[n]
            return default

        hidden = g("hidden_size", "n_embd", "d_model")
        n_heads = g("num_attention_heads", "n_head")
        n_kv = g("num_key_value_heads", default=n_heads)
        head_dim = g("head_dim", default=hidden // n_heads)
        rope_scaling = g("rope_scaling", "rope_parameters", default=None) or {}
        for key in ("rope_theta", "partial_rotary_factor"):               # newer configs keep every RoPE field in one table
            if key in rope_scaling and (key not in cfg or cfg.get("rope_parameters")):
                cfg = {**cfg, key: rope_scaling[key]}
        kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
        theta0 = g("rope_theta", default=10000.0)
        rope = RopeConfig(
            theta=float(theta0[0] if isinstance(theta0, (list, tuple)) else theta0),      # a list: one base per layer (Step-3.5)
            kind=kind if kind in ("default", "linear", "llama3", "yarn") else "default",
            factor=float(rope_scaling.get("factor", 1.0)),
            low_freq_factor=float(rope_scaling.get("low_freq_factor", 1.0)),
            high_freq_factor=float(rope_scaling.get("high_freq_factor", 4.0)),
            original_max_position=int(rope_scaling.get("original_max_position_embeddings", 8192)),
            beta_fast=float(rope_scaling.get("beta_fast", 32.0)),
            beta_slow=float(rope_scaling.get("beta_slow", 1.0)),
            mscale=float(rope_scaling.get("mscale", 1.0)),
            mscale_all_dim=float(rope_scaling.get("mscale_all_dim", 0.0)),
            truncate=bool(rope_scaling.get("truncate", True)),
            partial_rotary_factor=float(g("partial_rotary_factor", default=1.0)),
        )
        eos = g("eos_token_id", default=())
        if isinstance(eos, int):
            eos = (eos,)
        # one entry per checkpoint family the engine can shard (the reference keeps one sharding strategy per family,
        # ``src/exo/worker/engines/mlx/auto_parallel.py:500-599``); architectures that share a block structure share
        # an entry: Ministral / Mistral-3 text models are Llama blocks, GLM-4.x-MoE-Lite and Kimi are DeepSeek-V3
        # blocks (MLA + sigmoid-routed experts); GLM-5 is the DeepSeek-V3.2 block, whose sparse-attention indexer is not
        # used (every key is attended, which is what the indexer selects from)
        family = {"llama": "llama", "mistral": "llama", "ministral": "llama", "ministral3": "llama", "mistral3": "llama",
                  "qwen2": "llama", "qwen3": "qwen3", "qwen2_vl": "llama", "qwen2_vl_text": "llama", "qwen2_5_vl": "llama",
                  "qwen2_5_vl_text": "llama", "qwen3_vl": "qwen3", "qwen3_vl_text": "qwen3", "qwen3_vl_moe": "qwen3_moe",
                  "qwen3_vl_moe_text": "qwen3_moe", "kimi_vl": "deepseek_v3", "kimi_k25": "deepseek_v3",
                  "qwen3_moe": "qwen3_moe", "deepseek_v3": "deepseek_v3", "deepseek_v32": "deepseek_v3",
                  "deepseek_v2": "deepseek_v3", "kimi_k2": "deepseek_v3", "glm4_moe_lite": "deepseek_v3",
                  "glm_moe_dsa": "deepseek_v3",
                  "glm4_moe": "glm4_moe", "mixtral": "mixtral", "minimax": "minimax", "minimax_m2": "minimax",
                  "qwen3_next": "qwen3_next", "qwen3_5": "qwen3_next", "qwen3_5_text": "qwen3_next",
                  "qwen3_5_moe": "qwen3_next", "qwen3_5_moe_text": "qwen3_next",
                  "gemma4": "gemma4", "gemma4_text": "gemma4", "nemotron_h": "nemotron_h",
                  "gpt_oss": "gpt_oss", "step3p5": "step3p5"}.get(mt, "llama")
        blocks = None
        if family == "nemotron_h":
            blocks = g("layers_block_type", default=None)
            if blocks is None:
                pat = g("hybrid_override_pattern", default="M-M*")
                blocks = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[c] for c in pat]
            cfg = {**cfg, "num_hidden_layers": len(blocks)}
        mc = ModelConfig(
            name=name, family=family,
            n_layers=g("num_hidden_layers", "n_layer"), hidden=hidden, n_heads=n_heads,
            n_kv_heads=n_kv, head_dim=head_dim,
            ffn=g("intermediate_size", default=4 * hidden), vocab=g("vocab_size"),
            rms_eps=float(g("rms_norm_eps", default=1e-5)), rope=rope,
            tie_embeddings=bool(g("tie_word_embeddings", default=False)),
            qk_norm=family in ("qwen3", "qwen3_moe", "qwen3_next") or (family == "glm4_moe" and bool(g("use_qk_norm", default=False))),
            attn_bias=bool(g("attention_bias", default=mt in ("qwen2", "qwen2_vl", "qwen2_vl_text", "qwen2_5_vl", "qwen2_5_vl_text"))),
            max_position=int(g("max_position_embeddings", default=131072)),
            eos_token_ids=tuple(eos),
            sliding_window=int(g("sliding_window", default=0) or 0) if mt == "gpt_oss" else 0,
            attn_sinks=mt == "gpt_oss",
        )
        if family == "qwen3_moe":
            mc.n_experts = g("num_experts", "num_local_experts")
            mc.n_experts_per_tok = g("num_experts_per_tok")
            mc.moe_ffn = g("moe_intermediate_size")
            mc.norm_topk_prob = bool(g("norm_topk_prob", default=True))
            mc.router = "softmax"
        if family == "qwen3_next":
            # Qwen3-Next / Qwen3.5 / 3.6: three gated-delta-rule layers to one gated softmax-attention layer, RMSNorm
            # weights stored zero-centred, quarter-rotary RoPE, softmax-routed experts plus one sigmoid-gated shared expert
            n_l = mc.n_layers
            every = int(g("full_attention_interval", default=4))
            types = g("layer_types", default=None) or ["linear_attention" if (i + 1) % every else "full_attention" for i in range(n_l)]
            mc.layer_types = tuple("linear" if t == "linear_attention" else "full" for t in types)
            mc.lin_k_heads = g("linear_num_key_heads", default=16)
            mc.lin_v_heads = g("linear_num_value_heads", default=32)
            mc.lin_k_dim = g("linear_key_head_dim", default=128)
            mc.lin_v_dim = g("linear_value_head_dim", default=128)
            mc.lin_conv = g("linear_conv_kernel_dim", default=4)
            mc.lin_split_proj = mt != "qwen3_next"
            mc.attn_gate = True
            mc.norm_one_plus = True
            if "partial_rotary_factor" not in cfg:
                mc.rope.partial_rotary_factor = 0.25
            mc.n_experts = g("num_experts", "num_local_experts", default=0) or 0
            if mc.n_experts:
                mc.n_experts_per_tok = g("num_experts_per_tok")
                mc.moe_ffn = g("moe_intermediate_size")
                mc.norm_topk_prob = bool(g("norm_topk_prob", default=True))
                mc.router = "softmax"
                mc.shared_expert_ffn = g("shared_expert_intermediate_size", default=0) or 0
                mc.shared_expert_gate = mc.shared_expert_ffn > 0
                mc.moe_every = int(g("decoder_sparse_step", default=1))
                mc.mlp_only_layers = tuple(g("mlp_only_layers", default=()) or ())
            if mt != "qwen3_next":
                mc.weight_prefix = "model.language_model."
        if family == "nemotron_h":
            mc.block_types = tuple(blocks)
            mc.layer_types = tuple("linear" if b == "mamba" else "full" for b in blocks)
            mc.lin_k_heads = g("n_groups", default=8)
            mc.lin_k_dim = g("ssm_state_size", default=128)
            mc.lin_v_heads = g("mamba_num_heads", default=128)
            mc.lin_v_dim = g("mamba_head_dim", default=64)
            mc.lin_conv = g("conv_kernel", default=4)
            mc.rms_eps = float(g("layer_norm_epsilon", "rms_norm_eps", default=1e-5))
            mc.act = "relu2"
            mc.rope = RopeConfig(partial_rotary_factor=0.0)             # attention layers carry no position encoding
            mc.n_experts = g("n_routed_experts", default=0) if "moe" in blocks else 0
            if mc.n_experts:
                mc.n_experts_per_tok = g("num_experts_per_tok", default=2)
                mc.moe_ffn = g("moe_intermediate_size")
                mc.shared_expert_ffn = g("moe_shared_expert_intermediate_size", default=0) or 0
                mc.router, mc.router_bias = "sigmoid", True
                mc.norm_topk_prob = bool(g("norm_topk_prob", default=True))
                mc.routed_scaling = float(g("routed_scaling_factor", default=1.0))
                mc.n_group, mc.topk_group = g("n_group", default=1) or 1, g("topk_group", default=1) or 1
                mc.moe_latent = g("moe_latent_size", default=0) or 0
            mc.weight_prefix = "backbone."
        if family == "gemma4":
            n_l = mc.n_layers
            types = g("layer_types", default=None) or ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(n_l)]
            types = list(types)
            types[-1] = "full_attention"
            mc.layer_types = tuple("sliding" if t == "sliding_attention" else "full" for t in types)
            mc.sliding_window = int(g("sliding_window", default=512))
            mc.head_dim = g("head_dim", default=256)
            mc.global_head_dim = g("global_head_dim", default=512) or mc.head_dim
            mc.k_eq_v = bool(g("attention_k_eq_v", default=False))
            mc.global_kv_heads = g("num_global_key_value_heads", default=0) or 0
            mc.kv_shared_layers = g("num_kv_shared_layers", default=0) or 0
            mc.ple_dim = g("hidden_size_per_layer_input", default=256) or 0
            mc.ple_vocab = g("vocab_size_per_layer_input", default=mc.vocab) or mc.vocab
            mc.moe_beside_mlp = bool(g("enable_moe_block", default=False))
            mc.double_wide_mlp = bool(g("use_double_wide_mlp", default=False))
            mc.logit_softcap = float(g("final_logit_softcapping", default=0.0) or 0.0)
            mc.act = "gelu_tanh"
            mc.embed_scale = float(mc.hidden) ** 0.5
            mc.qk_norm = True
            mc.tie_embeddings = bool(g("tie_word_embeddings", default=True))
            rp = g("rope_parameters", default=None) or {}
            loc = rp.get("sliding_attention") or {"rope_type": "default", "rope_theta": 10000.0}
            glo = rp.get("full_attention") or {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000.0}
            mc.rope = RopeConfig(theta=float(loc.get("rope_theta", 10000.0)))
            mc.rope_global = RopeConfig(theta=float(glo.get("rope_theta", 1000000.0)),
                                        kind="proportional" if glo.get("rope_type") == "proportional" else "default",
                                        partial_rotary_factor=float(glo.get("partial_rotary_factor", 1.0)))
            if mc.moe_beside_mlp:
                mc.n_experts = g("num_experts", "num_local_experts")
                mc.n_experts_per_tok = g("top_k_experts")
                mc.moe_ffn = g("moe_intermediate_size")
                mc.router = "softmax"
                mc.norm_topk_prob = True
            if wrapped or mt != "gemma4_text":
                mc.weight_prefix = "model.language_model."
        if family == "step3p5":
            # Step-3.5: one full-attention layer to three sliding-window layers that have more query heads; zero-centred
            # RMSNorm everywhere (q / k norms included); RoPE base and rotary share per layer, long-context scaling only on
            # the layer types named; a sigmoid gate per head on the attention output; sigmoid-routed experts with a
            # selection bias, scaled, plus one shared expert; the first layers dense; SwiGLU clamped on some layers
            n_l = mc.n_layers
            types = list(g("layer_types", default=None) or ["full_attention" if i % 4 == 0 else "sliding_attention" for i in range(n_l)])[:n_l]
            mc.layer_types = tuple("sliding" if t == "sliding_attention" else "full" for t in types)
            mc.n_kv_heads = g("num_attention_groups", "num_key_value_heads", default=mc.n_kv_heads)
            mc.sliding_window = int(g("sliding_window", default=512) or 0)
            other = g("attention_other_setting", default=None) or {}
            if other:
                if other.get("num_attention_groups", mc.n_kv_heads) != mc.n_kv_heads or other.get("head_dim", mc.head_dim) != mc.head_dim:
                    raise ValueError("Step-3.5 layer types with their own KV-head count or head size are not supported")
                mc.layer_n_heads = tuple(other["num_attention_heads"] if t == other.get("attention_type", "sliding_attention") else mc.n_heads
                                         for t in types)
            thetas = g("rope_theta", default=10000.0)
            thetas = list(thetas) if isinstance(thetas, (list, tuple)) else [thetas] * n_l
            shares = list(g("partial_rotary_factors", default=None) or [1.0] * n_l)
            use = list(g("use_rope_layers", default=None) or [True] * n_l)
            only = g("yarn_only_types", default=None) or []
            ropes = []
            for i in range(n_l):
                scaled = not only or types[i] in only
                base = mc.rope if scaled else RopeConfig()
                ropes.append(replace(base, theta=float(thetas[i]), partial_rotary_factor=float(shares[i]) if use[i] else 0.0))
            mc.layer_rope = tuple(ropes)
            mc.rope = ropes[0]
            mc.qk_norm = True
            mc.norm_one_plus = True
            mc.head_gate = bool(g("use_head_wise_attn_gate", default=False))
            mc.n_experts = g("moe_num_experts", default=0) or 0
            mc.n_experts_per_tok = g("moe_top_k", default=0) or 0
            mc.moe_ffn = g("moe_intermediate_size", default=0) or 0
            mc.shared_expert_ffn = g("share_expert_dim", default=0) or 0
            mc.router = str(g("moe_router_activation", default="sigmoid"))
            mc.router_bias = bool(g("use_moe_router_bias", default=True))
            mc.norm_topk_prob = bool(g("norm_expert_weight", default=True))
            mc.routed_scaling = float(g("moe_router_scaling_factor", default=1.0))
            enum = g("moe_layers_enum", default=None)
            moe_layers = {int(x) for x in str(enum).split(",") if x.strip()} if enum is not None else set(range(1, n_l))
            mc.mlp_only_layers = tuple(i for i in range(n_l) if i not in moe_layers)
            mc.swiglu_limits = tuple(float(x or 0.0) for x in (g("swiglu_limits", default=None) or ()))
            mc.swiglu_limits_shared = tuple(float(x or 0.0) for x in (g("swiglu_limits_shared", default=None) or ()))
        if family == "glm4_moe":
            # GLM-4.5 / 4.6: grouped-query attention with half-rotary RoPE and q/k/v biases, DeepSeek-style experts
            # (sigmoid scores + correction bias, shared expert, leading dense layers)
            mc.n_experts = g("n_routed_experts", default=0)
            mc.n_experts_per_tok = g("num_experts_per_tok", default=0)
            mc.moe_ffn = g("moe_intermediate_size", default=0)
            mc.n_shared_experts = g("n_shared_experts", default=0) or 0
            mc.first_dense_layers = g("first_k_dense_replace", default=0)
            mc.router = "sigmoid"
            mc.norm_topk_prob = bool(g("norm_topk_prob", default=True))
            mc.routed_scaling = float(g("routed_scaling_factor", default=1.0))
            mc.n_group = g("n_group", default=1) or 1
            mc.topk_group = g("topk_group", default=1) or 1
            mc.router_bias = True
            if "partial_rotary_factor" not in cfg:
                mc.rope.partial_rotary_factor = 0.5
        if family == "minimax":
            # MiniMax-M2: every layer sparse (sigmoid scores + correction bias, no shared expert), q / k normalised
            # over their whole width, rotary on the first `rotary_dim` of each head
            mc.n_experts = g("num_local_experts", default=0)
            mc.n_experts_per_tok = g("num_experts_per_tok", default=0)
            mc.moe_ffn = g("intermediate_size")
            mc.router = "sigmoid"
            mc.router_bias = True
            mc.norm_topk_prob = True
            mc.qk_norm_full = bool(g("use_qk_norm", default=True))
            if g("rotary_dim", default=None):
                mc.rope.partial_rotary_factor = g("rotary_dim") / mc.head_dim
        if mt == "gpt_oss":
            # GPT-OSS: sliding and full attention alternate, sinks, biases everywhere, YaRN without rounding, top-k then
            # softmax routing with a router bias, experts with biases and the capped (up + 1) * gate * sigmoid(1.702 gate)
            n_l = mc.n_layers
            types = list(g("layer_types", default=None) or ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n_l)])
            mc.layer_types = tuple("sliding" if t == "sliding_attention" else "full" for t in types)
            mc.sliding_window = int(g("sliding_window", default=128) or 0)
            mc.attn_bias = bool(g("attention_bias", default=True))
            mc.n_experts = g("num_local_experts", default=0) or 0
            if mc.n_experts:
                mc.n_experts_per_tok = g("num_experts_per_tok", "experts_per_token", default=4)
                mc.moe_ffn = g("intermediate_size")
                mc.router, mc.norm_topk_prob = "softmax", True
                mc.router_linear_bias = mc.expert_bias = True
                mc.act = "swiglu_oai"
                mc.oai_limit = float(g("swiglu_limit", default=7.0))
        if family == "mixtral":
            # every layer is a sparse block: softmax over the top-k router logits (= softmax then renormalise)
            mc.n_experts = g("num_local_experts", default=8)
            mc.n_experts_per_tok = g("num_experts_per_tok", default=2)
            mc.moe_ffn = g("intermediate_size")
            mc.router = "softmax"
            mc.norm_topk_prob = True
            mc.sliding_window = 0
        if family == "deepseek_v3":
            mc.mla = True
            mc.mla_rope_neox = mt == "glm_moe_dsa"
            mc.q_lora_rank = g("q_lora_rank", default=0) or 0
            mc.kv_lora_rank = g("kv_lora_rank")
            mc.qk_nope_dim = g("qk_nope_head_dim")
            mc.qk_rope_dim = g("qk_rope_head_dim")
            mc.v_head_dim = g("v_head_dim")
            mc.n_experts = g("n_routed_experts", default=0)
            mc.n_experts_per_tok = g("num_experts_per_tok", default=0)
            mc.moe_ffn = g("moe_intermediate_size", default=0)
            mc.n_shared_experts = g("n_shared_experts", default=0) or 0
            mc.first_dense_layers = g("first_k_dense_replace", default=0)
            kinds = g("mlp_layer_types", default=None)          # GLM-5 lists every layer's kind instead
            if kinds:                                            # the list wins where both are given, as in the library
                mc.first_dense_layers = next((i for i, k in enumerate(kinds) if k != "dense"), len(kinds))
                mc.mlp_only_layers = tuple(i for i, k in enumerate(kinds) if k == "dense" and i >= mc.first_dense_layers)
            mc.router = "sigmoid" if g("scoring_func", default="sigmoid") == "sigmoid" else "softmax"
            mc.norm_topk_prob = bool(g("norm_topk_prob", default=True))
            mc.routed_scaling = float(g("routed_scaling_factor", default=1.0))
            mc.n_group = g("n_group", default=1) or 1
            mc.topk_group = g("topk_group", default=1) or 1
            mc.router_bias = True
            mc.head_dim = mc.qk_nope_dim + mc.qk_rope_dim
        return mc

    @staticmethod
    def from_pretrained(path: str | Path) -> "ModelConfig":
        p = Path(path)
        with open(p / "config.json") as f:
            return ModelConfig.from_hf(json.load(f), name=p.name)


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


# ----------------------------------------------------------------------------
# Named presets: the architectures the benchmark configs are quoted on.
# ----------------------------------------------------------------------------
def preset(name: str) -> ModelConfig:
    n = name.lower()
    if n in ("tiny-llama", "tiny"):
        return ModelConfig(name="tiny-llama", family="llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2,
                           head_dim=64, ffn=688, vocab=32000, rms_eps=1e-5, rope=RopeConfig(theta=10000.0),
                           dtype="fp32")
    if n in ("llama-3.1-8b", "llama8b"):
        return ModelConfig(name="llama-3.1-8b", family="llama", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8,
                           head_dim=128, ffn=14336, vocab=128256, rope=RopeConfig(theta=500000.0))
    if n in ("llama-3.1-70b", "llama70b"):
        return ModelConfig(name="llama-3.1-70b", family="llama", n_layers=80, hidden=8192, n_heads=64, n_kv_heads=8,
                           head_dim=128, ffn=28672, vocab=128256, rope=RopeConfig(theta=500000.0), quant="mxfp8")
    if n in ("qwen3-235b-a22b", "qwen3-235b"):
        return ModelConfig(name="qwen3-235b-a22b", family="qwen3_moe", n_layers=94, hidden=4096, n_heads=64,
                           n_kv_heads=4, head_dim=128, ffn=12288, vocab=151936, rms_eps=1e-6,
                           rope=RopeConfig(theta=1000000.0), qk_norm=True, n_experts=128, n_experts_per_tok=8,
                           moe_ffn=1536, router="softmax", quant="mxfp8")
    if n in ("deepseek-v3", "deepseek-v3-671b"):
        return ModelConfig(name="deepseek-v3", family="deepseek_v3", n_layers=61, hidden=7168, n_heads=128,
                           n_kv_heads=128, head_dim=192, ffn=18432, vocab=129280, rms_eps=1e-6,
                           rope=RopeConfig(theta=10000.0), mla=True, q_lora_rank=1536, kv_lora_rank=512,
                           qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128, n_experts=256, n_experts_per_tok=8,
                           moe_ffn=2048, n_shared_experts=1, first_dense_layers=3, router="sigmoid",
                           routed_scaling=2.5, n_group=8, topk_group=4, router_bias=True, quant="dsfp8")
    if n in ("tiny-moe",):
        return ModelConfig(name="tiny-moe", family="qwen3_moe", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2,
                           head_dim=64, ffn=512, vocab=1024, qk_norm=True, n_experts=8, n_experts_per_tok=2,
                           moe_ffn=128, router="softmax", dtype="fp32")
    if n in ("tiny-qwen3",):       # dense with per-head q/k RMSNorm
        return ModelConfig(name="tiny-qwen3", family="qwen3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, rms_eps=1e-6, qk_norm=True, dtype="fp32")
    if n in ("tiny-qwen2",):       # q/k/v biases, tied embeddings
        return ModelConfig(name="tiny-qwen2", family="llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, attn_bias=True, tie_embeddings=True, dtype="fp32")
    if n in ("tiny-glm4-moe",):    # half-rotary RoPE, biases, sigmoid router with correction bias, shared expert, one dense layer
        return ModelConfig(name="tiny-glm4-moe", family="glm4_moe", n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, attn_bias=True, rope=RopeConfig(theta=10000.0, partial_rotary_factor=0.5),
                           n_experts=8, n_experts_per_tok=2, moe_ffn=128, n_shared_experts=1, first_dense_layers=1,
                           router="sigmoid", routed_scaling=1.0, router_bias=True, dtype="fp32")
    if n in ("tiny-mixtral",):     # every layer sparse, top-2 softmax, block_sparse_moe.* tensor names
        return ModelConfig(name="tiny-mixtral", family="mixtral", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, n_experts=4, n_experts_per_tok=2, moe_ffn=256, router="softmax", dtype="fp32")
    if n in ("tiny-minimax",):     # full-width q/k norm, half-rotary, sigmoid router with correction bias on every layer
        return ModelConfig(name="tiny-minimax", family="minimax", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, qk_norm_full=True, rope=RopeConfig(theta=10000.0, partial_rotary_factor=0.5),
                           n_experts=8, n_experts_per_tok=2, moe_ffn=128, router="sigmoid", router_bias=True, dtype="fp32")
    if n in ("tiny-step3p5",):     # full / sliding layers with different query-head counts and RoPE, head gates, clamped SwiGLU
        types = ("full", "sliding", "sliding", "full")
        ropes = tuple(RopeConfig(theta=50000.0 if t == "full" else 10000.0, partial_rotary_factor=0.5 if t == "full" else 1.0) for t in types)
        return ModelConfig(name="tiny-step3p5", family="step3p5", n_layers=4, hidden=256, n_heads=2, n_kv_heads=2, head_dim=128, ffn=512,
                           vocab=1024, qk_norm=True, norm_one_plus=True, layer_types=types, sliding_window=24,
                           layer_n_heads=tuple(4 if t == "sliding" else 2 for t in types), layer_rope=ropes, rope=ropes[0], head_gate=True,
                           n_experts=8, n_experts_per_tok=2, moe_ffn=128, shared_expert_ffn=128, router="sigmoid", router_bias=True,
                           norm_topk_prob=True, routed_scaling=3.0, mlp_only_layers=(0,), swiglu_limits=(0.0, 0.0, 0.0, 0.05),
                           swiglu_limits_shared=(0.0, 0.0, 0.04, 0.04), dtype="fp32")
    if n in ("step-3.5-flash",):   # the published model's shape (benchmarks with weights from a seed): 196 B parameters, 11 B active
        L = 45
        types = tuple("full" if i % 4 == 0 else "sliding" for i in range(L))
        ropes = tuple(RopeConfig(theta=5000000.0 if t == "full" else 10000.0, partial_rotary_factor=0.5 if t == "full" else 1.0) for t in types)
        return ModelConfig(name="step-3.5-flash", family="step3p5", n_layers=L, hidden=4096, n_heads=64, n_kv_heads=8, head_dim=128, ffn=11264,
                           vocab=128896, qk_norm=True, norm_one_plus=True, layer_types=types, sliding_window=512,
                           layer_n_heads=tuple(96 if t == "sliding" else 64 for t in types), layer_rope=ropes, rope=ropes[0], head_gate=True,
                           n_experts=288, n_experts_per_tok=8, moe_ffn=1280, shared_expert_ffn=1280, router="sigmoid", router_bias=True,
                           norm_topk_prob=True, routed_scaling=3.0, mlp_only_layers=(0, 1, 2), swiglu_limits=(0.0,) * 43 + (7.0, 7.0),
                           swiglu_limits_shared=(0.0,) * 43 + (16.0, 16.0), max_position=262144, quant="mxfp8")
    if n in ("tiny-gpt-oss",):     # attention sinks and a sliding window on every other layer's worth of context
        return ModelConfig(name="tiny-gpt-oss", family="gpt_oss", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, attn_bias=True, attn_sinks=True, sliding_window=32, dtype="fp32")
    if n in ("tiny-yarn",):        # YaRN-scaled RoPE on a Llama block
        return ModelConfig(name="tiny-yarn", family="llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, rope=RopeConfig(theta=10000.0, kind="yarn", factor=4.0, original_max_position=64),
                           dtype="fp32")
    if n in ("tiny-qwen3-next",):  # linear, linear, full, linear: gated delta rule + gated attention, experts with a gated shared expert
        return ModelConfig(name="tiny-qwen3-next", family="qwen3_next", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2,
                           head_dim=256, ffn=512, vocab=1024, rms_eps=1e-6, qk_norm=True,
                           rope=RopeConfig(theta=10000.0, partial_rotary_factor=0.25),
                           layer_types=("linear", "linear", "full", "linear"), lin_k_heads=2, lin_v_heads=4, lin_k_dim=64,
                           lin_v_dim=64, lin_conv=4, attn_gate=True, norm_one_plus=True, n_experts=8, n_experts_per_tok=2,
                           moe_ffn=128, router="softmax", shared_expert_ffn=128, shared_expert_gate=True, dtype="fp32")
    if n in ("qwen3-next-80b-a3b", "qwen3-next"):
        return ModelConfig(name="qwen3-next-80b-a3b", family="qwen3_next", n_layers=48, hidden=2048, n_heads=16, n_kv_heads=2,
                           head_dim=256, ffn=5120, vocab=151936, rms_eps=1e-6, qk_norm=True,
                           rope=RopeConfig(theta=10000000.0, partial_rotary_factor=0.25),
                           layer_types=tuple("full" if (i + 1) % 4 == 0 else "linear" for i in range(48)),
                           lin_k_heads=16, lin_v_heads=32, lin_k_dim=128, lin_v_dim=128, lin_conv=4, attn_gate=True,
                           norm_one_plus=True, n_experts=512, n_experts_per_tok=10, moe_ffn=512, router="softmax",
                           shared_expert_ffn=512, shared_expert_gate=True, quant="mxfp8")
    if n in ("tiny-nemotron-h",):  # Mamba-2, attention without positions, relu^2 experts with a shared expert, a plain MLP block
        return ModelConfig(name="tiny-nemotron-h", family="nemotron_h", n_layers=6, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, rms_eps=1e-5, rope=RopeConfig(partial_rotary_factor=0.0),
                           block_types=("mamba", "moe", "attention", "mlp", "mamba", "moe"),
                           layer_types=("linear", "full", "full", "full", "linear", "full"), lin_k_heads=2, lin_k_dim=64,
                           lin_v_heads=8, lin_v_dim=32, lin_conv=4, act="relu2", n_experts=8, n_experts_per_tok=2, moe_ffn=128,
                           shared_expert_ffn=192, router="sigmoid", router_bias=True, routed_scaling=1.5,
                           weight_prefix="backbone.", dtype="fp32")
    if n in ("tiny-gemma4",):      # sliding / full layers with their own head sizes, v = k on full layers, per-layer inputs, shared KV
        return ModelConfig(name="tiny-gemma4", family="gemma4", n_layers=6, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                           ffn=512, vocab=1024, rms_eps=1e-6, qk_norm=True, tie_embeddings=True,
                           layer_types=("sliding", "full", "sliding", "full", "sliding", "full"), sliding_window=32,
                           global_head_dim=128, global_kv_heads=1, k_eq_v=True, kv_shared_layers=2, ple_dim=32, ple_vocab=1024,
                           logit_softcap=30.0, act="gelu_tanh", embed_scale=16.0, rope=RopeConfig(theta=10000.0),
                           rope_global=RopeConfig(theta=1000000.0, kind="proportional", partial_rotary_factor=0.25),
                           weight_prefix="model.", dtype="fp32")
    if n in ("tiny-mla",):
        return ModelConfig(name="tiny-mla", family="deepseek_v3", n_layers=3, hidden=256, n_heads=4, n_kv_heads=4,
                           head_dim=48, ffn=512, vocab=1024, mla=True, q_lora_rank=64, kv_lora_rank=32,
                           qk_nope_dim=32, qk_rope_dim=16, v_head_dim=32, n_experts=8, n_experts_per_tok=2,
                           moe_ffn=128, n_shared_experts=1, first_dense_layers=1, router="sigmoid",
                           routed_scaling=1.5, n_group=2, topk_group=1, router_bias=True, dtype="fp32")
    raise KeyError(f"unknown preset {name!r}")


PRESETS = ("tiny-llama", "llama-3.1-8b", "llama-3.1-70b", "qwen3-235b-a22b", "deepseek-v3", "tiny-moe", "tiny-mla",
           "tiny-qwen3", "tiny-qwen2", "tiny-gemma4", "tiny-nemotron-h", "tiny-qwen3-next", "qwen3-next-80b-a3b", "tiny-glm4-moe", "tiny-mixtral", "tiny-minimax", "tiny-gpt-oss", "tiny-step3p5", "step-3.5-flash", "tiny-yarn")
