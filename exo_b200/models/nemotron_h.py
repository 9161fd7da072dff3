"""Nemotron-H (Nemotron-Nano-9B-v2, Nemotron-3-Nano-30B-A3B): weights and forward for one rank's shard.

Every layer is ONE mixer behind one RMSNorm, ``h + mixer(norm(h))``, the mixer being a Mamba-2 state-space block,
softmax attention without any position encoding, a non-gated ``relu^2`` MLP, or a block of such experts (sigmoid router
with a selection bias, shared expert, optional latent projection around the routed experts).  The reference shards this
family in ``src/exo/worker/engines/mlx/auto_parallel.py:1416-1538`` (``NemotronHShardingStrategy``: attention by heads,
Mamba-2 by heads and groups, experts whole); the semantics followed here are those of ``transformers``
(``models/nemotron_h/modeling_nemotron_h.py``).

The Mamba-2 state (convolution history + ``[d_state, head_dim]`` per head, fp32) lives in the per-sequence state seats
the gated-delta-rule layers use, and the recurrence runs on the same kernels (``ops.mamba2``).

Tensor parallelism: Mamba-2 heads and their B/C groups are split over the ranks (``n_groups`` must divide), the input
projection is re-ordered at load to ``C | B | x | z | dt | dt`` of the local heads; attention heads, the MLP width and
the shared expert are split as in the Llama block; routed experts are partitioned whole.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference as ref
from .config import ModelConfig
from .transformer import Decoder, KVPool, StepInputs, resolve
from .weights import (ModelWeights, ShardSpec, TensorSource, _DTYPES, _cols, _rows, expert_range, kv_head_range, linear_heads,
                      text_model_root, vocab_shard)


@dataclass
class NemotronLayer:
    kind: str
    norm: torch.Tensor
    # mamba
    m_in: torch.Tensor | None = None         # [2*G*N + 2*W + 2*Hm, H] local rows C | B | x | z | dt | dt
    m_conv_w: torch.Tensor | None = None     # [2*G*N + W, taps] fp32 (rows C | B | x)
    m_conv_b: torch.Tensor | None = None     # fp32
    m_a_log: torch.Tensor | None = None
    m_dt_bias: torch.Tensor | None = None
    m_skip: torch.Tensor | None = None       # D
    m_norm: torch.Tensor | None = None       # [W]
    m_out: torch.Tensor | None = None        # [H, W] local
    # attention
    wqkv: torch.Tensor | None = None
    wo: torch.Tensor | None = None
    # mlp / shared expert
    w_up: torch.Tensor | None = None         # [F/N, H]
    w_down: torch.Tensor | None = None       # [H, F/N]
    # experts
    router: torch.Tensor | None = None       # [E, H] fp32
    router_bias: torch.Tensor | None = None
    e_up: torch.Tensor | None = None         # [E_local, F, H or latent]
    e_down: torch.Tensor | None = None       # [E_local, H or latent, F]
    lat_in: torch.Tensor | None = None       # [latent, H]
    lat_out: torch.Tensor | None = None      # [H, latent]


def build_nemotron_h_weights(cfg: ModelConfig, spec: ShardSpec, src: TensorSource, device="cpu", progress=None) -> ModelWeights:
    dt = _DTYPES[cfg.dtype]
    dev = torch.device(device)
    r, n = spec.tp_rank, spec.tp_size
    H = cfg.hidden
    root = text_model_root(cfg, src, "embeddings.weight")

    def fin(t: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
        return t.to(device=dev, dtype=dtype or dt).contiguous()

    G, N, Hm, P = cfg.lin_k_heads, cfg.lin_k_dim, cfg.lin_v_heads, cfg.lin_v_dim
    W = Hm * P
    layers: dict[int, NemotronLayer] = {}
    lrange = spec.layers(cfg)
    for li, i in enumerate(lrange):
        p = f"{root}layers.{i}."
        m = p + "mixer."
        kind = cfg.block_types[i]
        lw = NemotronLayer(kind=kind, norm=fin(src.get(p + "norm.weight", (H,))))
        if kind == "mamba":
            linear_heads(cfg, spec)                                   # groups must split over the ranks
            # in_proj rows: z [W] | x [W] | B [G*N] | C [G*N] | dt [Hm]; the convolution runs over x | B | C
            w_in = src.get(m + "in_proj.weight", (2 * W + 2 * G * N + Hm, H))
            z, x, Bm, Cm, dtr = w_in.split((W, W, G * N, G * N, Hm), 0)
            dloc = _rows(dtr, r, n)
            lw.m_in = fin(torch.cat((_rows(Cm, r, n), _rows(Bm, r, n), _rows(x, r, n), _rows(z, r, n), dloc, dloc), 0))
            cw = src.get(m + "conv1d.weight", (W + 2 * G * N, 1, cfg.lin_conv)).reshape(W + 2 * G * N, cfg.lin_conv)
            cx, cB, cC = cw.split((W, G * N, G * N), 0)
            lw.m_conv_w = fin(torch.cat((_rows(cC, r, n), _rows(cB, r, n), _rows(cx, r, n)), 0), torch.float32)
            if src.has(m + "conv1d.bias"):
                bx, bB, bC = src.get(m + "conv1d.bias", (W + 2 * G * N,)).split((W, G * N, G * N), 0)
                lw.m_conv_b = fin(torch.cat((_rows(bC, r, n), _rows(bB, r, n), _rows(bx, r, n)), 0), torch.float32)
            lw.m_a_log = fin(_rows(src.get(m + "A_log", (Hm,)), r, n), torch.float32)
            lw.m_dt_bias = fin(_rows(src.get(m + "dt_bias", (Hm,)), r, n), torch.float32)
            lw.m_skip = fin(_rows(src.get(m + "D", (Hm,)), r, n), torch.float32)
            lw.m_norm = fin(_rows(src.get(m + "norm.weight", (W,)), r, n))
            lw.m_out = fin(_cols(src.get(m + "out_proj.weight", (H, W)), r, n))
        elif kind == "attention":
            D = cfg.head_dim
            klo, khi = kv_head_range(cfg, spec)
            wq = _rows(src.get(m + "q_proj.weight", (cfg.n_heads * D, H)), r, n)
            wk = src.get(m + "k_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
            wv = src.get(m + "v_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
            lw.wqkv = fin(torch.cat((wq, wk, wv), 0))
            lw.wo = fin(_cols(src.get(m + "o_proj.weight", (H, cfg.n_heads * D)), r, n))
        elif kind == "mlp":
            lw.w_up = fin(_rows(src.get(m + "up_proj.weight", (cfg.ffn, H)), r, n))
            lw.w_down = fin(_cols(src.get(m + "down_proj.weight", (H, cfg.ffn)), r, n))
        else:
            E, F = cfg.n_experts, cfg.moe_ffn
            inner = cfg.moe_latent or H
            lw.router = fin(src.get(m + "gate.weight", (E, H)), torch.float32)
            lw.router_bias = fin(src.get(m + "gate.e_score_correction_bias", (E,)), torch.float32)
            elo, ehi = expert_range(cfg, spec)
            if src.has(m + "experts.up_proj"):                       # stacked tensors (the library's own layout)
                lw.e_up = fin(src.get(m + "experts.up_proj", (E, F, inner))[elo:ehi])
                lw.e_down = fin(src.get(m + "experts.down_proj", (E, inner, F))[elo:ehi])
            else:
                lw.e_up = fin(torch.stack([src.get(f"{m}experts.{e}.up_proj.weight", (F, inner)) for e in range(elo, ehi)]))
                lw.e_down = fin(torch.stack([src.get(f"{m}experts.{e}.down_proj.weight", (inner, F)) for e in range(elo, ehi)]))
            if cfg.shared_expert_ffn:
                Fs = cfg.shared_expert_ffn
                lw.w_up = fin(_rows(src.get(m + "shared_experts.up_proj.weight", (Fs, H)), r, n))
                lw.w_down = fin(_cols(src.get(m + "shared_experts.down_proj.weight", (H, Fs)), r, n))
            if cfg.moe_latent:
                lw.lat_in = fin(src.get(m + "fc1_latent_proj.weight", (cfg.moe_latent, H)))
                lw.lat_out = fin(src.get(m + "fc2_latent_proj.weight", (H, cfg.moe_latent)))
        layers[i] = lw
        if progress is not None:
            progress(li + 1, len(lrange))
    embed = final_norm = lm_head = None
    if spec.is_first_stage or (cfg.tie_embeddings and spec.is_last_stage):
        embed = fin(src.get(root + "embeddings.weight", (cfg.vocab, H)))
    if spec.is_last_stage:
        final_norm = fin(src.get(root + "norm_f.weight", (H,)))
        full = embed if (cfg.tie_embeddings or not src.has("lm_head.weight")) else fin(src.get("lm_head.weight", (cfg.vocab, H)))
        vpad = vocab_shard(cfg.vocab, n)
        lm_head = full[min(r * vpad, cfg.vocab):min((r + 1) * vpad, cfg.vocab)]
        if lm_head.shape[0] < vpad:
            lm_head = torch.cat((lm_head, torch.zeros(vpad - lm_head.shape[0], H, dtype=lm_head.dtype, device=dev)), 0)
        lm_head = lm_head.contiguous()
    return ModelWeights(embed=embed, layers=layers, final_norm=final_norm, lm_head=lm_head)


class NemotronHDecoder(Decoder):
    def _mega_ready(self, kv, tokens) -> bool:
        return False

    def _mamba(self, lw: NemotronLayer, x: torch.Tensor, inp: StepInputs, state) -> torch.Tensor:
        cfg = self.cfg
        groups, heads = linear_heads(cfg, self.spec)
        conv_state, ssm_state = state
        proj = ops.linear(x, lw.m_in)
        y = ops.mamba2(proj, lw.m_conv_w, lw.m_conv_b, lw.m_a_log, lw.m_dt_bias, lw.m_skip, lw.m_norm, cfg.rms_eps, conv_state,
                       ssm_state, inp.state_slots, inp.cu_q, inp.positions, groups, heads, cfg.lin_k_dim, cfg.lin_v_dim)
        return resolve(self.comm.row_linear(y, lw.m_out))

    def _attention(self, lw: NemotronLayer, x: torch.Tensor, inp: StepInputs, kv) -> torch.Tensor:
        cfg = self.cfg
        kc, vc = kv
        qkv = ops.linear(x, lw.wqkv)
        q = ops.qk_rope_append(qkv, inp.positions, self.inv_freq, 1.0, self.n_q, self.n_kv, cfg.head_dim, kc, vc, inp.slots)
        o = ops.paged_attention(q, kc, vc, inp.block_tables, inp.seq_lens, inp.cu_q, self.scale, 0, None, inp.max_q_len)
        return resolve(self.comm.row_linear(o.reshape(o.shape[0], -1), lw.wo))

    def _mlp_partial(self, lw: NemotronLayer, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.relu2(ops.linear(x, lw.w_up)), lw.w_down)

    def _moe(self, lw: NemotronLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        logits = ref.linear(x.float(), lw.router)
        wts, ids = ops.moe_route(logits, cfg.n_experts_per_tok, "sigmoid", cfg.norm_topk_prob, lw.router_bias, cfg.n_group,
                                 cfg.topk_group, cfg.routed_scaling)
        elo, _ = expert_range(cfg, self.spec)
        xin = ops.linear(x, lw.lat_in) if lw.lat_in is not None else x
        y = ops.moe_experts(xin, lw.e_up, lw.e_down, wts, ids, elo, cfg.n_experts, act="relu2")
        if lw.lat_out is not None:
            y = ops.linear(y, lw.lat_out)          # of this rank's partial sum: the projection is linear
        if lw.w_up is not None:
            y = y + self._mlp_partial(lw, x)
        return resolve(self.comm.row_sum(y))

    def forward(self, inp: StepInputs, kv: KVPool, hidden_in: torch.Tensor | None = None, need_logits: bool = True):
        cfg, w = self.cfg, self.w
        h = ops.embedding(w.embed, inp.tokens) if self.spec.is_first_stage else hidden_in
        patches = getattr(self, "embed_patches", None)
        if patches and self.spec.is_first_stage:
            for r0, rows in patches:
                h[r0:r0 + rows.shape[0]] = rows.to(device=h.device, dtype=h.dtype)
            self.embed_patches = None
        for i in self.spec.layers(cfg):
            lw = w.layers[i]
            x = ops.rmsnorm(h, lw.norm, cfg.rms_eps)[0]
            if lw.kind == "mamba":
                y = self._mamba(lw, x, inp, kv.layers[i])
            elif lw.kind == "attention":
                y = self._attention(lw, x, inp, kv.layers[i])
            elif lw.kind == "mlp":
                y = resolve(self.comm.row_sum(self._mlp_partial(lw, x)))
            else:
                y = self._moe(lw, x)
            h = h + y
        if not self.spec.is_last_stage:
            return h
        if not need_logits:
            return None
        hs = h if (inp.max_q_len == 1 and inp.logit_rows.numel() == h.shape[0]) else h[inp.logit_rows.long()]
        return ops.linear(ops.rmsnorm(hs, w.final_norm, cfg.rms_eps)[0], w.lm_head)
