"""Step-3.5 (Step-3.5-Flash): checkpoint layout and per-layer attention parameters.

The reference shards this family by heads and by expert width (``src/exo/worker/engines/mlx/auto_parallel.py:1373-1413``:
``q/k/v/o_proj``, the per-head gate ``g_proj``, dense ``mlp`` or ``mlp.switch_mlp`` + ``mlp.share_expert``).  The block runs
on the generic decoder (``transformer.Decoder``) with per-layer parameters carried by the layer's weights: sliding-window
layers have more query heads than full-attention layers, every layer has its own RoPE base and rotary share, long-context
scaling applies to some layer types only, a sigmoid gate per head (a projection of the normed hidden state) multiplies the
attention output, experts are sigmoid-routed with a selection bias and a scale, a shared expert runs beside them, the first
layers are dense, and on some layers SwiGLU is clamped (activated gate capped at the limit, up projection clamped to
+-limit).  All RMSNorm weights are stored zero-centred.  Layers past ``num_hidden_layers`` in a checkpoint (next-token
prediction heads) are not read.

Two tensor layouts load: the hub export (``layers.N.moe.gate.weight``, ``moe.router_bias``, stacked ``moe.{gate,up,down}_proj.weight``
``[E, out, in]``, ``layers.N.share_expert.*``) and MLX conversions (``layers.N.mlp.gate.*``, ``mlp.switch_mlp.*``,
``mlp.share_expert.*``, norm weights with the 1 already added).
"""
from __future__ import annotations

from collections.abc import Callable

import torch

from ..ops import reference as ref
from .config import ModelConfig
from .weights import (_DTYPES, LayerWeights, ModelWeights, ShardSpec, TensorSource, _cols, _rows, expert_range, kv_head_range,
                      quantize_layer, text_model_root, vocab_shard)


def _first(src: TensorSource, names: tuple[str, ...]) -> str:
    """The first of ``names`` the checkpoint has (the first one for sources that have every name)."""
    for n in names:
        if src.has(n):
            return n
    raise KeyError(f"none of {names} in the checkpoint")


def moe_tensor_names(src: TensorSource, p: str) -> dict[str, str]:
    """Names of layer ``p``'s sparse block in whichever layout the checkpoint uses."""
    router = _first(src, (p + "moe.gate.weight", p + "mlp.gate.gate.weight", p + "mlp.gate.weight"))
    bias = _first(src, (p + "moe.router_bias", p + "mlp.gate.router_bias", p + "mlp.router_bias"))
    experts = _first(src, (p + "moe.gate_proj.weight", p + "mlp.switch_mlp.gate_proj.weight"))[:-len("gate_proj.weight")]
    shared = _first(src, (p + "share_expert.gate_proj.weight", p + "mlp.share_expert.gate_proj.weight",
                          p + "moe.share_expert.gate_proj.weight"))[:-len("gate_proj.weight")]
    return {"router": router, "bias": bias, "experts": experts, "shared": shared}


def build_step3p5_weights(cfg: ModelConfig, spec: ShardSpec, src: TensorSource, device="cpu",
                          progress: Callable[[int, int], None] | None = None) -> ModelWeights:
    dt, dev = _DTYPES[cfg.dtype], torch.device(device)
    r, n = spec.tp_rank, spec.tp_size
    H, D = cfg.hidden, cfg.head_dim
    root = text_model_root(cfg, src)

    def fin(t: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
        return t.to(device=dev, dtype=dtype or dt).contiguous()
    # hub checkpoints keep norm weights zero-centred; an MLX conversion (recognised by its tensor names) has added the 1
    mlx_form = not src.has(f"{root}layers.{cfg.n_layers - 1}.moe.gate.weight") and \
        src.has(f"{root}layers.{cfg.n_layers - 1}.mlp.switch_mlp.gate_proj.weight")
    one = 0.0 if mlx_form else 1.0

    def norm(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        return fin(src.get(name, shape).float() + one)
    klo, khi = kv_head_range(cfg, spec)
    layers: dict[int, LayerWeights] = {}
    lrange = spec.layers(cfg)
    for li, i in enumerate(lrange):
        p, a = f"{root}layers.{i}.", f"{root}layers.{i}.self_attn."
        nh = cfg.q_heads(i)
        if nh % n:
            raise ValueError(f"layer {i}: {nh} query heads do not divide over {n} ranks")
        lw = LayerWeights(attn_norm=norm(p + "input_layernorm.weight", (H,)), ffn_norm=norm(p + "post_attention_layernorm.weight", (H,)))
        wq = _rows(src.get(a + "q_proj.weight", (nh * D, H)), r, n)
        wk = src.get(a + "k_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
        wv = src.get(a + "v_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
        lw.wqkv = fin(torch.cat((wq, wk, wv), 0))
        lw.wo = fin(_cols(src.get(a + "o_proj.weight", (H, nh * D)), r, n))
        lw.q_norm, lw.k_norm = norm(a + "q_norm.weight", (D,)), norm(a + "k_norm.weight", (D,))
        if cfg.head_gate:
            lw.w_head_gate = fin(_rows(src.get(a + "g_proj.weight", (nh, H)), r, n))
        lw.n_q = nh // n
        inv, lw.rope_mscale = ref.rope_inv_freq(D, cfg.rope_of(i))
        lw.inv_freq = inv.to(dev)
        lw.window = cfg.window_of(i)
        if cfg.layer_is_moe(i):
            E, F = cfg.n_experts, cfg.moe_ffn
            nm = moe_tensor_names(src, p)
            lw.router = fin(src.get(nm["router"], (E, H)))
            lw.router_bias = fin(src.get(nm["bias"], (E,)), torch.float32)
            elo, ehi = expert_range(cfg, spec)
            gate = src.get(nm["experts"] + "gate_proj.weight", (E, F, H))[elo:ehi]
            up = src.get(nm["experts"] + "up_proj.weight", (E, F, H))[elo:ehi]
            lw.e_gate_up = fin(torch.cat((gate, up), 1))
            lw.e_down = fin(src.get(nm["experts"] + "down_proj.weight", (E, H, F))[elo:ehi])
            Fs, sp = cfg.shared_expert_ffn, nm["shared"]
            lw.s_gate_up = fin(torch.cat((_rows(src.get(sp + "gate_proj.weight", (Fs, H)), r, n),
                                          _rows(src.get(sp + "up_proj.weight", (Fs, H)), r, n)), 0))
            lw.s_down = fin(_cols(src.get(sp + "down_proj.weight", (H, Fs)), r, n))
            lw.act_limit, lw.shared_limit = cfg.swiglu_limit(i), cfg.swiglu_limit(i, shared=True)
        else:
            F, m = cfg.ffn, p + "mlp."
            lw.w_gate_up = fin(torch.cat((_rows(src.get(m + "gate_proj.weight", (F, H)), r, n),
                                          _rows(src.get(m + "up_proj.weight", (F, H)), r, n)), 0))
            lw.w_down = fin(_cols(src.get(m + "down_proj.weight", (H, F)), r, n))
            lw.shared_limit = cfg.swiglu_limit(i, shared=True)      # the dense MLP takes the shared expert's limit
        layers[i] = quantize_layer(cfg, lw)
        if progress is not None:
            progress(li + 1, len(lrange))
    embed = final_norm = lm_head = None
    if spec.is_first_stage or (cfg.tie_embeddings and spec.is_last_stage):
        embed = fin(src.get(root + "embed_tokens.weight", (cfg.vocab, H)))
    if spec.is_last_stage:
        final_norm = norm(root + "norm.weight", (H,))
        name = root + "embed_tokens.weight" if (cfg.tie_embeddings or not src.has("lm_head.weight")) else "lm_head.weight"
        full = src.get(name, (cfg.vocab, H))
        vpad = vocab_shard(cfg.vocab, n)
        lm_head = fin(full[min(r * vpad, cfg.vocab):min((r + 1) * vpad, cfg.vocab)])
        if lm_head.shape[0] < vpad:
            lm_head = torch.cat((lm_head, torch.zeros(vpad - lm_head.shape[0], H, dtype=lm_head.dtype, device=dev)), 0)
    return ModelWeights(embed=embed, layers=layers, final_norm=final_norm, lm_head=lm_head)
