"""Gemma-4 text model: weights and forward for one rank's shard.

The reference shards this family with its own strategy (``src/exo/worker/engines/mlx/auto_parallel.py:590-597``,
``Gemma4ShardingStrategy``) and runs it through ``mlx_lm.models.gemma4``; the semantics followed here are those of
``transformers`` (``models/gemma4/modeling_gemma4.py``).  What differs from the Llama-shaped block in
``models/transformer.py``:

* two kinds of layers: *sliding* (local window, ``head_dim``) and *full* (``global_head_dim``, optionally fewer KV heads
  and ``v = k``), each kind with its own RoPE (the full layers rotate the whole head with zero frequencies beyond the
  rotary share);
* q and k are RMS-normalised per head with a weight, v without one; the softmax scale is 1;
* norms before AND after attention and MLP (``h + norm(attn(norm(h)))``), GeGLU, a per-layer output scalar;
* optional per-layer input embeddings: a second embedding table gives every layer a small vector per token, gated by
  the stream and projected back into it after the MLP;
* optional expert block beside the dense MLP (router on the un-normalised stream, its own norms);
* the last ``kv_shared_layers`` layers compute no keys and values and read the cache of the last earlier layer of
  their kind;
* embeddings scaled by ``sqrt(hidden)``, tied output projection, tanh soft-capping of the logits.

Tensor parallelism: query heads, KV heads (replicated when fewer than ranks) and the MLP width are split as in the
Llama block; the per-layer-input path and the norms are replicated; experts are partitioned whole.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference as ref
from .config import ModelConfig
from .transformer import Decoder, KVPool, StepInputs, resolve
from .weights import (ModelWeights, ShardSpec, TensorSource, _DTYPES, _cols, _rows, expert_range, text_model_root, vocab_shard)


@dataclass
class Gemma4Layer:
    attn_norm: torch.Tensor
    post_attn_norm: torch.Tensor
    pre_ffn_norm: torch.Tensor
    post_ffn_norm: torch.Tensor
    wqkv: torch.Tensor               # [(hq + 2 hkv) * D, H] local ([hq * D, H] on a layer that reads another layer's cache)
    wo: torch.Tensor                 # [H, hq * D] local
    q_norm: torch.Tensor
    k_norm: torch.Tensor | None
    w_gate_up: torch.Tensor          # [2F/N, H]
    w_down: torch.Tensor             # [H, F/N]
    scalar: float = 1.0
    # per-layer inputs
    ple_gate: torch.Tensor | None = None     # [P, H]
    ple_proj: torch.Tensor | None = None     # [H, P]
    ple_norm: torch.Tensor | None = None     # [H]
    # expert block beside the MLP
    router: torch.Tensor | None = None       # [E, H] with the router's input scale folded in
    e_gate_up: torch.Tensor | None = None    # [E_local, 2F, H]
    e_down: torch.Tensor | None = None       # [E_local, H, F] with the per-expert output scale folded in
    post_ffn_norm_1: torch.Tensor | None = None
    post_ffn_norm_2: torch.Tensor | None = None
    pre_ffn_norm_2: torch.Tensor | None = None


@dataclass
class Gemma4Weights(ModelWeights):
    ple_embed: torch.Tensor | None = None        # [V_ple, L * P]
    ple_model_proj: torch.Tensor | None = None   # [L * P, H]
    ple_proj_norm: torch.Tensor | None = None    # [P]


def layer_heads(cfg: ModelConfig, spec: ShardSpec, i: int) -> tuple[int, int, int, int, int]:
    """``(q heads, kv heads, head_dim, first kv head, kv heads in the model)`` of layer ``i`` on this rank."""
    kv_all, D = cfg.attn_dims(i)
    n, r = spec.tp_size, spec.tp_rank
    if cfg.n_heads % n:
        raise ValueError(f"{cfg.n_heads} query heads do not split over {n} ranks")
    if kv_all >= n:
        c = kv_all // n
        lo, cnt = r * c, c
    else:
        lo, cnt = r * kv_all // n, 1
    return cfg.n_heads // n, cnt, D, lo, kv_all


def build_gemma4_weights(cfg: ModelConfig, spec: ShardSpec, src: TensorSource, device="cpu", progress=None) -> Gemma4Weights:
    dt = _DTYPES[cfg.dtype]
    dev = torch.device(device)
    r, n = spec.tp_rank, spec.tp_size
    H, L = cfg.hidden, cfg.n_layers
    root = text_model_root(cfg, src)

    def fin(t: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
        return t.to(device=dev, dtype=dtype or dt).contiguous()

    layers: dict[int, Gemma4Layer] = {}
    lrange = spec.layers(cfg)
    first_shared = L - cfg.kv_shared_layers
    for li, i in enumerate(lrange):
        p = f"{root}layers.{i}."
        a = p + "self_attn."
        hq, hkv, D, klo, kv_all = layer_heads(cfg, spec, i)
        shared = cfg.kv_source_layer(i) != i
        wq = _rows(src.get(a + "q_proj.weight", (cfg.n_heads * D, H)), r, n)
        if shared:
            wqkv, k_norm = wq, None
        else:
            wk = src.get(a + "k_proj.weight", (kv_all * D, H))[klo * D:(klo + hkv) * D]
            full_kv = cfg.k_eq_v and not cfg.layer_is_sliding(i)       # these layers have no v projection: v is k's output
            wv = wk if full_kv else src.get(a + "v_proj.weight", (kv_all * D, H))[klo * D:(klo + hkv) * D]
            wqkv = torch.cat((wq, wk, wv), 0)
            k_norm = fin(src.get(a + "k_norm.weight", (D,)))
        F = cfg.ffn * (2 if (cfg.double_wide_mlp and cfg.kv_shared_layers and i >= first_shared) else 1)
        m = p + "mlp."
        lw = Gemma4Layer(
            attn_norm=fin(src.get(p + "input_layernorm.weight", (H,))),
            post_attn_norm=fin(src.get(p + "post_attention_layernorm.weight", (H,))),
            pre_ffn_norm=fin(src.get(p + "pre_feedforward_layernorm.weight", (H,))),
            post_ffn_norm=fin(src.get(p + "post_feedforward_layernorm.weight", (H,))),
            wqkv=fin(wqkv), wo=fin(_cols(src.get(a + "o_proj.weight", (H, cfg.n_heads * D)), r, n)),
            q_norm=fin(src.get(a + "q_norm.weight", (D,))), k_norm=k_norm,
            w_gate_up=fin(torch.cat((_rows(src.get(m + "gate_proj.weight", (F, H)), r, n),
                                     _rows(src.get(m + "up_proj.weight", (F, H)), r, n)), 0)),
            w_down=fin(_cols(src.get(m + "down_proj.weight", (H, F)), r, n)),
            scalar=float(src.get(p + "layer_scalar", (1,)).float().reshape(-1)[0]) if src.has(p + "layer_scalar") else 1.0)
        if cfg.ple_dim:
            P = cfg.ple_dim
            lw.ple_gate = fin(src.get(p + "per_layer_input_gate.weight", (P, H)))
            lw.ple_proj = fin(src.get(p + "per_layer_projection.weight", (H, P)))
            lw.ple_norm = fin(src.get(p + "post_per_layer_input_norm.weight", (H,)))
        if cfg.moe_beside_mlp:
            E, Fe = cfg.n_experts, cfg.moe_ffn
            scale = src.get(p + "router.scale", (H,)).float() * H ** -0.5
            lw.router = fin(src.get(p + "router.proj.weight", (E, H)).float() * scale[None, :])
            elo, ehi = expert_range(cfg, spec)
            per_expert = src.get(p + "router.per_expert_scale", (E,)).float()[elo:ehi]
            lw.e_gate_up = fin(src.get(p + "experts.gate_up_proj", (E, 2 * Fe, H))[elo:ehi])
            lw.e_down = fin(src.get(p + "experts.down_proj", (E, H, Fe))[elo:ehi].float() * per_expert[:, None, None])
            lw.post_ffn_norm_1 = fin(src.get(p + "post_feedforward_layernorm_1.weight", (H,)))
            lw.post_ffn_norm_2 = fin(src.get(p + "post_feedforward_layernorm_2.weight", (H,)))
            lw.pre_ffn_norm_2 = fin(src.get(p + "pre_feedforward_layernorm_2.weight", (H,)))
        layers[i] = lw
        if progress is not None:
            progress(li + 1, len(lrange))
    embed = fin(src.get(root + "embed_tokens.weight", (cfg.vocab, H)))
    w = Gemma4Weights(embed=embed if (spec.is_first_stage or cfg.tie_embeddings) else None, layers=layers, final_norm=None, lm_head=None)
    if cfg.ple_dim:
        w.ple_embed = fin(src.get(root + "embed_tokens_per_layer.weight", (cfg.ple_vocab, L * cfg.ple_dim)))
        w.ple_model_proj = fin(src.get(root + "per_layer_model_projection.weight", (L * cfg.ple_dim, H)))
        w.ple_proj_norm = fin(src.get(root + "per_layer_projection_norm.weight", (cfg.ple_dim,)))
    if spec.is_last_stage:
        w.final_norm = fin(src.get(root + "norm.weight", (H,)))
        full = embed if (cfg.tie_embeddings or not src.has("lm_head.weight")) else fin(src.get("lm_head.weight", (cfg.vocab, H)))
        vpad = vocab_shard(cfg.vocab, n)
        head = full[min(r * vpad, cfg.vocab):min((r + 1) * vpad, cfg.vocab)]
        if head.shape[0] < vpad:
            head = torch.cat((head, torch.zeros(vpad - head.shape[0], H, dtype=head.dtype, device=dev)), 0)
        w.lm_head = head.contiguous()
    return w


class Gemma4KV(KVPool):
    """Paged KV with per-layer head counts and widths; a layer that shares another's cache gets the same tensors."""

    def __init__(self, cfg: ModelConfig, spec: ShardSpec, n_blocks: int, block_size: int = 16, device="cpu", dtype=None,
                 max_seqs: int = 64):
        self.cfg, self.block_size, self.n_blocks = cfg, block_size, n_blocks
        dt = dtype or (torch.bfloat16 if cfg.dtype == "bf16" else torch.float32)
        self.layers = {}
        self.snapshots, self.n_snapshots = {}, 0
        for i in spec.layers(cfg):
            j = cfg.kv_source_layer(i)
            if j != i and j in self.layers:
                self.layers[i] = self.layers[j]
                continue
            _, hkv, D, _, _ = layer_heads(cfg, spec, j)
            self.layers[i] = (torch.zeros(n_blocks, block_size, hkv, D, dtype=dt, device=device),
                              torch.zeros(n_blocks, block_size, hkv, D, dtype=dt, device=device))

    @staticmethod
    def bytes_per_block(cfg: ModelConfig, spec: ShardSpec, block_size: int = 16) -> int:
        el = 2 if cfg.dtype == "bf16" else 4
        total = 0
        for i in spec.layers(cfg):
            if cfg.kv_source_layer(i) == i:
                _, hkv, D, _, _ = layer_heads(cfg, spec, i)
                total += 2 * block_size * hkv * D * el
        return total


class Gemma4Decoder(Decoder):
    def __init__(self, cfg: ModelConfig, weights: Gemma4Weights, spec: ShardSpec | None = None, comm=None):
        super().__init__(cfg, weights, spec, comm)
        if self.spec.pp_size > 1 and cfg.ple_dim:
            raise NotImplementedError("Gemma-4 per-layer inputs need the token embeddings on every stage: no pipeline stages")
        dev = weights.embed.device
        self.inv_local = ref.rope_inv_freq(cfg.head_dim, cfg.rope)[0].to(dev)
        self.inv_global = ref.rope_inv_freq(cfg.global_head_dim or cfg.head_dim, cfg.rope_global or cfg.rope)[0].to(dev)
        self.ones: dict[int, torch.Tensor] = {}

    def _ones(self, n: int, like: torch.Tensor) -> torch.Tensor:
        t = self.ones.get(n)
        if t is None:
            t = self.ones[n] = torch.ones(n, dtype=like.dtype, device=like.device)
        return t

    def _mega_ready(self, kv, tokens) -> bool:
        return False

    # ------------------------------------------------------------------ pieces
    def _attn(self, i: int, lw: Gemma4Layer, x: torch.Tensor, inp: StepInputs, kv) -> torch.Tensor:
        cfg = self.cfg
        hq, hkv, D, _, _ = layer_heads(cfg, self.spec, i)
        sliding = cfg.layer_is_sliding(i)
        inv = self.inv_local if sliding else self.inv_global
        kc, vc = kv
        qkv = ops.linear(x, lw.wqkv)
        if lw.k_norm is None:        # reads another layer's cache: q only
            q = ops.qk_rope_append(qkv, inp.positions, inv, 1.0, hq, 0, D, kc, vc, inp.slots, lw.q_norm, lw.q_norm, cfg.rms_eps)
        else:
            q = ops.qk_rope_append(qkv, inp.positions, inv, 1.0, hq, hkv, D, kc, vc, inp.slots, lw.q_norm, lw.k_norm,
                                   cfg.rms_eps, v_unit_norm=True)
        o = ops.paged_attention(q, kc, vc, inp.block_tables, inp.seq_lens, inp.cu_q, 1.0,
                                cfg.sliding_window if sliding else 0, None, inp.max_q_len)
        return resolve(self.comm.row_linear(o.reshape(o.shape[0], -1), lw.wo))

    def _mlp(self, lw: Gemma4Layer, x: torch.Tensor) -> torch.Tensor:
        return resolve(self.comm.row_linear(ops.geglu(ops.linear(x, lw.w_gate_up)), lw.w_down))

    def _experts(self, lw: Gemma4Layer, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        logits = ops.linear(ops.rmsnorm(h, self._ones(cfg.hidden, h), cfg.rms_eps)[0], lw.router)
        wts, ids = ops.moe_route(logits, cfg.n_experts_per_tok, "softmax", True, None, 1, 1, 1.0)
        x2 = ops.rmsnorm(h, lw.pre_ffn_norm_2, cfg.rms_eps)[0]
        elo, _ = expert_range(cfg, self.spec)
        y = ops.moe_experts(x2, lw.e_gate_up, lw.e_down, wts, ids, elo, cfg.n_experts, act="gelu_tanh")
        return resolve(self.comm.row_sum(y))

    # ------------------------------------------------------------------ forward
    def forward(self, inp: StepInputs, kv: KVPool, hidden_in: torch.Tensor | None = None, need_logits: bool = True):
        cfg, w = self.cfg, self.w
        eps = cfg.rms_eps
        tokens = inp.tokens.long()
        if self.spec.is_first_stage:
            h = ops.embedding(w.embed, inp.tokens)
            h = (h.float() * torch.tensor(cfg.embed_scale, dtype=h.dtype).float()).to(h.dtype)
        else:
            h = hidden_in
        patches = getattr(self, "embed_patches", None)
        if patches and self.spec.is_first_stage:
            for r0, rows in patches:
                h[r0:r0 + rows.shape[0]] = rows.to(device=h.device, dtype=h.dtype)
            self.embed_patches = None
        ple = None
        if cfg.ple_dim:
            L, P = cfg.n_layers, cfg.ple_dim
            T = h.shape[0]
            tab = ops.embedding(w.ple_embed, inp.tokens.clamp(max=cfg.ple_vocab - 1)).view(T, L, P)
            tab = (tab.float() * torch.tensor(P ** 0.5, dtype=tab.dtype).float()).to(tab.dtype)
            proj = (ops.linear(h, w.ple_model_proj).float() * cfg.hidden ** -0.5).to(h.dtype).view(T * L, P)
            proj = ops.rmsnorm(proj.contiguous(), w.ple_proj_norm, eps)[0].view(T, L, P)
            ple = ((proj.float() + tab.float()) * 2.0 ** -0.5).to(h.dtype)
        for i in self.spec.layers(cfg):
            lw = w.layers[i]
            a = self._attn(i, lw, ops.rmsnorm(h, lw.attn_norm, eps)[0], inp, kv.layers[i])
            h = h + ops.rmsnorm(a, lw.post_attn_norm, eps)[0]
            m = self._mlp(lw, ops.rmsnorm(h, lw.pre_ffn_norm, eps)[0])
            if cfg.moe_beside_mlp:
                m = ops.rmsnorm(m, lw.post_ffn_norm_1, eps)[0] + ops.rmsnorm(self._experts(lw, h), lw.post_ffn_norm_2, eps)[0]
            h = h + ops.rmsnorm(m, lw.post_ffn_norm, eps)[0]
            if ple is not None:
                g = ops.linear(h, lw.ple_gate)
                g = (torch.nn.functional.gelu(g.float(), approximate="tanh") * ple[:, i].float()).to(h.dtype)
                h = h + ops.rmsnorm(ops.linear(g, lw.ple_proj), lw.ple_norm, eps)[0]
            if lw.scalar != 1.0:
                h = h * lw.scalar
        if not self.spec.is_last_stage:
            return h
        if not need_logits:
            return None
        hs = h if (inp.max_q_len == 1 and inp.logit_rows.numel() == h.shape[0]) else h[inp.logit_rows.long()]
        logits = ops.linear(ops.rmsnorm(hs, w.final_norm, eps)[0], w.lm_head)
        if cfg.logit_softcap:
            logits = (torch.tanh(logits.float() / cfg.logit_softcap) * cfg.logit_softcap).to(logits.dtype)
        return logits
