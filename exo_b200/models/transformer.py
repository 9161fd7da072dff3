"""The decoder forward pass for one rank's shard, written as a flat sequence of hot ops.

There is no ``nn.Module`` tree: a step is a fixed list of kernel launches over the shard's
weight tensors and a paged KV pool, which is what a CUDA graph captures on the decode path.
The same function serves prefill chunks (many tokens per sequence) and decode (one token per
sequence) because the attention op takes ragged query lengths.

Per-layer structure and collective placement follow the reference's tensor-parallel layer
(``src/exo/worker/engines/mlx/auto_parallel.py:628-652`` Llama, ``:688-767`` DeepSeek MLA and
MoE, ``:1121-1283`` Qwen3-MoE): column-parallel q/k/v and gate/up, row-parallel o and down with
one sum over ranks each.  That sum is delegated to ``comm.row_linear`` so the fused
GEMM+all-reduce kernel, the NCCL baseline and the single-rank case share this file.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference as ref
from .config import ModelConfig
from .weights import ModelWeights, ShardSpec, local_heads, expert_range, linear_heads


class LocalComm:
    """Single-rank communicator: every collective is the identity."""
    size = 1
    rank = 0

    def row_linear(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual + sum over ranks of x_r @ w_r.T``."""
        return ops.linear(x, w, residual=residual)

    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return x if residual is None else x + residual

    def all_reduce_stat(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of a few fp32 numbers per token over the ranks (normalisation statistics)."""
        return x

    def row_sum(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.all_reduce(x, residual)

    def gather_vocab(self, logits_local: torch.Tensor) -> torch.Tensor:
        return logits_local

    def send(self, x: torch.Tensor, dst: int) -> None:  # pragma: no cover
        raise RuntimeError("no peer")

    def recv(self, x: torch.Tensor, src: int) -> None:  # pragma: no cover
        raise RuntimeError("no peer")


@dataclass
class StepInputs:
    """Device-side description of one forward step over ``B`` sequences and ``T`` new tokens."""
    tokens: torch.Tensor        # [T] int32/int64
    positions: torch.Tensor     # [T] int32
    slots: torch.Tensor         # [T] int32/64 flat KV slots (block*block_size+offset)
    cu_q: torch.Tensor          # [B+1] int32
    seq_lens: torch.Tensor      # [B] int32 (KV length including the new tokens)
    block_tables: torch.Tensor  # [B, max_blocks] int32
    logit_rows: torch.Tensor    # [B'] int32/64 rows of the T tokens whose logits are wanted
    max_q_len: int = 1
    state_slots: torch.Tensor | None = None   # [B] int32 seats of the sequences' recurrent state (linear-attention layers)


def resolve(h):
    """Tensor behind ``h``: a pending tensor-parallel reduction (``parallel.fused.Handover`` / ``Reduction``) is
    finished first."""
    return h if isinstance(h, torch.Tensor) or h is None else h.value()


def reduced_and_normed(h, norm_w, eps):
    """``(h, rmsnorm(h) * norm_w)`` where ``h`` may still be a pending reduction: the sum over ranks, the residual
    add and the norm are then one kernel."""
    if isinstance(h, torch.Tensor):
        return h, ops.rmsnorm(h, norm_w, eps)[0]
    x = h.norm(norm_w, eps)
    return h, x       # h stays the reduction object: in its two-shot form the stream is sharded by rows, and only a
    #                   consumer that needs every row (``resolve``) pays for gathering it


class KVPool:
    """Paged KV storage for the layers this rank holds (block size 16 by default)."""

    def __init__(self, cfg: ModelConfig, spec: ShardSpec, n_blocks: int, block_size: int = 16,
                 device: str | torch.device = "cpu", dtype: torch.dtype | None = None, max_seqs: int = 64, n_snapshots: int = 0):
        self.cfg, self.block_size, self.n_blocks = cfg, block_size, n_blocks
        dt = dtype or (torch.bfloat16 if cfg.dtype == "bf16" else torch.float32)
        self.layers: dict[int, tuple[torch.Tensor, torch.Tensor | None]] = {}
        # prefix-cache snapshots of the recurrent layers' state: (convolution history, state) per layer, `n_snapshots` slots
        self.snapshots: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.n_snapshots = n_snapshots if cfg.has_linear_layers else 0
        _, hkv = local_heads(cfg, spec)
        for i in spec.layers(cfg):
            if cfg.block_types and cfg.block_types[i] in ("mlp", "moe"):
                self.layers[i] = (None, None)         # a layer without a sequence mixer keeps nothing
                continue
            if cfg.layer_is_linear(i):
                # a gated-delta-rule layer keeps no keys and values: per sequence seat (seat 0 = scratch) the last
                # taps-1 inputs of its convolution and the [dk, dv] state of every value head, the latter in fp32
                hk, hv = linear_heads(cfg, spec)
                conv = torch.zeros(max_seqs + 1, 2 * hk * cfg.lin_k_dim + hv * cfg.lin_v_dim, cfg.lin_conv - 1, dtype=dt, device=device)
                rec = torch.zeros(max_seqs + 1, hv, cfg.lin_k_dim, cfg.lin_v_dim, dtype=torch.float32, device=device)
                self.layers[i] = (conv, rec)
                if self.n_snapshots:
                    self.snapshots[i] = (torch.zeros(self.n_snapshots, *conv.shape[1:], dtype=dt, device=device),
                                         torch.zeros(self.n_snapshots, *rec.shape[1:], dtype=torch.float32, device=device))
            elif cfg.mla:
                c = torch.zeros(n_blocks, block_size, cfg.kv_lora_rank + cfg.qk_rope_dim, dtype=dt, device=device)
                self.layers[i] = (c, None)
            else:
                k = torch.zeros(n_blocks, block_size, hkv, cfg.head_dim, dtype=dt, device=device)
                v = torch.zeros(n_blocks, block_size, hkv, cfg.head_dim, dtype=dt, device=device)
                self.layers[i] = (k, v)

    @staticmethod
    def bytes_per_block(cfg: ModelConfig, spec: ShardSpec, block_size: int = 16) -> int:
        if cfg.family == "gemma4":
            from .gemma4 import Gemma4KV
            return Gemma4KV.bytes_per_block(cfg, spec, block_size)
        el = 2 if cfg.dtype == "bf16" else 4
        n_layers = sum(1 for i in spec.layers(cfg) if not cfg.layer_is_linear(i)
                       and not (cfg.block_types and cfg.block_types[i] in ("mlp", "moe")))
        if cfg.mla:
            return n_layers * block_size * (cfg.kv_lora_rank + cfg.qk_rope_dim) * el
        _, hkv = local_heads(cfg, spec)
        return n_layers * 2 * block_size * hkv * cfg.head_dim * el


    def save_state(self, seat: int, snap: int) -> None:
        """Copy a sequence seat's recurrent state into a snapshot slot (stream-ordered device copies)."""
        for i, (conv_s, rec_s) in self.snapshots.items():
            conv, rec = self.layers[i]
            conv_s[snap].copy_(conv[seat])
            rec_s[snap].copy_(rec[seat])

    def restore_state(self, seat: int, snap: int) -> None:
        for i, (conv_s, rec_s) in self.snapshots.items():
            conv, rec = self.layers[i]
            conv[seat].copy_(conv_s[snap])
            rec[seat].copy_(rec_s[snap])

    @staticmethod
    def state_bytes(cfg: ModelConfig, spec: ShardSpec, max_seqs: int) -> int:
        """Bytes of recurrent state (all gated-delta-rule layers of this shard, ``max_seqs`` seats plus scratch)."""
        n = sum(1 for i in spec.layers(cfg) if cfg.layer_is_linear(i))
        if not n:
            return 0
        el = 2 if cfg.dtype == "bf16" else 4
        hk, hv = linear_heads(cfg, spec)
        per_seat = (2 * hk * cfg.lin_k_dim + hv * cfg.lin_v_dim) * (cfg.lin_conv - 1) * el + hv * cfg.lin_k_dim * cfg.lin_v_dim * 4
        return n * (max_seqs + 1) * per_seat


class Decoder:
    """One rank's model shard + forward."""

    def __init__(self, cfg: ModelConfig, weights: ModelWeights, spec: ShardSpec | None = None, comm=None):
        self.cfg, self.w = cfg, weights
        self.spec = spec or ShardSpec()
        self.comm = comm or LocalComm()
        dev = next(weights.tensors()).device
        rot_dim = cfg.qk_rope_dim if cfg.mla else cfg.head_dim
        inv, mscale = ref.rope_inv_freq(rot_dim, cfg.rope)
        self.inv_freq = inv.to(dev)
        self.rope_mscale = mscale
        self.n_q, self.n_kv = local_heads(cfg, self.spec)
        if cfg.mla:
            self.scale = (cfg.qk_nope_dim + cfg.qk_rope_dim) ** -0.5
            if cfg.rope.kind == "yarn" and cfg.rope.mscale_all_dim:
                m = 0.1 * cfg.rope.mscale_all_dim * __import__("math").log(cfg.rope.factor) + 1.0
                self.scale *= m * m
        else:
            self.scale = cfg.head_dim ** -0.5

    def _mega_ready(self, kv: "KVPool", tokens: torch.Tensor) -> bool:
        """Whether the whole-step decode kernel serves this shard (decided once): a dense bf16 model held by one rank,
        128-wide heads, no attention sinks or sliding window, shapes the kernel is built for."""
        state = getattr(self, "_mega", None)
        if state is None:
            cfg, spec = self.cfg, self.spec
            ok = (tokens.is_cuda and tokens.dtype == torch.int32 and cfg.dtype == "bf16" and spec.tp_size == 1
                  and spec.pp_size == 1 and not cfg.mla and not cfg.layer_types and isinstance(self.w.embed, torch.Tensor)
                  and self.w.embed.dtype == torch.bfloat16
                  and not cfg.is_moe and not cfg.sliding_window and not cfg.attn_sinks and isinstance(self.comm, LocalComm)
                  and isinstance(self.w.lm_head, torch.Tensor) and self.w.lm_head.dtype == torch.bfloat16
                  and getattr(self, "embed_patches", None) is None)
            if ok:
                from ..ops import cuda as K
                layers = [self.w.layers[i] for i in spec.layers(cfg)]
                ok = K.DecodeMega.supported(cfg, layers, self.n_q, self.n_kv, self.inv_freq)
                if ok:
                    self._mega = K.DecodeMega(cfg, layers, [kv.layers[i] for i in spec.layers(cfg)], self.w.embed,
                                              self.w.final_norm, self.w.lm_head, self.n_q, self.n_kv, tokens.device)
                    self._mega_kv = kv
            if not ok:
                self._mega = False
            state = self._mega
        return bool(state) and self._mega_kv is kv and not getattr(self, "embed_patches", None)

    # ------------------------------------------------------------------ attention
    def _attn_gqa(self, lw, h, inp: StepInputs, kv) -> torch.Tensor:
        cfg = self.cfg
        n_q = lw.n_q or self.n_q                                   # layers may have their own head count, RoPE and window
        inv_freq, mscale = (self.inv_freq, self.rope_mscale) if lw.inv_freq is None else (lw.inv_freq, lw.rope_mscale)
        window = cfg.sliding_window if lw.window < 0 else lw.window
        head_gate = None
        if lw.w_head_gate is not None:
            # the gate reads the same normed hidden state as q / k / v: norm once, project twice
            h, x = reduced_and_normed(h, lw.attn_norm, cfg.rms_eps)
            qkv = ops.linear(x, lw.wqkv, lw.bqkv)
            head_gate = torch.nn.functional.linear(x, lw.w_head_gate)
        else:
            qkv = ops.norm_linear(h, lw.attn_norm, cfg.rms_eps, lw.wqkv, lw.bqkv)
        kc, vc = kv
        q_norm, k_norm = lw.q_norm, lw.k_norm
        if cfg.qk_norm_full:
            qkv = self._full_width_qk_norm(qkv, lw)
            q_norm = k_norm = None
        width = (n_q + 2 * self.n_kv) * cfg.head_dim
        q = ops.qk_rope_append(qkv[:, :width] if cfg.attn_gate else qkv, inp.positions, inv_freq, mscale, n_q, self.n_kv,
                               cfg.head_dim, kc, vc, inp.slots, q_norm, k_norm, cfg.rms_eps)
        o = ops.paged_attention(q, kc, vc, inp.block_tables, inp.seq_lens, inp.cu_q, self.scale,
                                window, lw.sinks, inp.max_q_len)
        if head_gate is not None:
            o = (o.view(o.shape[0], n_q, -1) * torch.sigmoid(head_gate.float())[..., None].to(o.dtype))
        o = o.reshape(o.shape[0], -1)
        if cfg.attn_gate:        # the projection's last n_q*D columns gate the attention output per element
            o = ops.sigmoid_gate(o, qkv[:, (n_q + 2 * self.n_kv) * cfg.head_dim:])
        if lw.bo is not None:    # the output projection's bias joins the residual: it is added once, not once per rank
            h = resolve(h) + lw.bo
        return self.comm.row_linear(o, lw.wo, h)

    def _attn_linear(self, lw, h, inp: StepInputs, state) -> torch.Tensor:
        """Gated delta rule in place of softmax attention (``src/exo/worker/engines/mlx/auto_parallel.py:1150-1200`` shards
        the same layer by key-head groups): input projection, then one op for convolution + recurrence + gated norm over
        this rank's heads and the sequences' state seats, then the row-parallel output projection."""
        cfg = self.cfg
        proj = ops.norm_linear(h, lw.attn_norm, cfg.rms_eps, lw.lin_in)
        hk, hv = linear_heads(cfg, self.spec)
        conv_state, rec_state = state
        o = ops.gated_delta(proj, lw.lin_conv_w, lw.lin_a_log, lw.lin_dt_bias, lw.lin_norm, cfg.rms_eps, conv_state, rec_state,
                            inp.state_slots, inp.cu_q, inp.positions, hk, hv, cfg.lin_k_dim, cfg.lin_v_dim)
        return self.comm.row_linear(o, lw.lin_out, h)

    def _full_width_qk_norm(self, qkv: torch.Tensor, lw) -> torch.Tensor:
        """RMSNorm of q over ALL query heads and of k over ALL key heads (MiniMax).  Under tensor parallelism a rank
        holds a slice of the columns: the ranks sum their sums of squares (two numbers per token) instead of gathering
        q and k, which is what the reference does (``src/exo/worker/engines/mlx/auto_parallel.py:1023-1048``).  A KV head
        that several ranks replicate is counted once."""
        cfg, D = self.cfg, self.cfg.head_dim
        nq, nk = self.n_q * D, self.n_kv * D
        q, k = qkv[:, :nq].float(), qkv[:, nq:nq + nk].float()
        rep = max(1, self.spec.tp_size * self.n_kv // cfg.n_kv_heads)         # ranks holding each KV head
        ss = torch.stack((q.pow(2).sum(-1), k.pow(2).sum(-1) / rep), -1)
        ss = self.comm.all_reduce_stat(ss)
        rq = torch.rsqrt(ss[:, :1] / (cfg.n_heads * D) + cfg.rms_eps)
        rk = torch.rsqrt(ss[:, 1:] / (cfg.n_kv_heads * D) + cfg.rms_eps)
        out = qkv.clone()
        out[:, :nq] = (q * rq * lw.q_norm.float()).to(qkv.dtype)
        out[:, nq:nq + nk] = (k * rk * lw.k_norm.float()).to(qkv.dtype)
        return out

    def _attn_mla(self, lw, h, inp: StepInputs, kv) -> torch.Tensor:
        cfg = self.cfg
        h, x = reduced_and_normed(h, lw.attn_norm, cfg.rms_eps)
        T = h.shape[0]
        if lw.wq_a is not None:
            q = ops.norm_linear(ops.linear(x, lw.wq_a), lw.q_a_norm, cfg.rms_eps, lw.wq_b)
        else:
            q = ops.linear(x, lw.wq_b)
        q = q.view(T, self.n_q, cfg.qk_nope_dim + cfg.qk_rope_dim)
        kva = ops.linear(x, lw.wkv_a)
        ckv = kv[0]
        ops.mla_kv_append(kva, lw.kv_a_norm, cfg.rms_eps, inp.positions, self.inv_freq, self.rope_mscale, ckv, inp.slots,
                          cfg.kv_lora_rank)
        # weight absorption: scores are taken in the kv_lora latent space, the cache row is K and V at once
        if T > 64 and getattr(lw, "w_uk_t", None) is None and lw.w_uk.is_cuda:
            lw.w_uk_t = lw.w_uk.transpose(1, 2).contiguous()        # [H, kv_lora, nope]: the prefill GEMMs' layout
        q_full = ops.mla_q_absorb(q, lw.w_uk, inp.positions, self.inv_freq, self.rope_mscale, cfg.qk_nope_dim,
                                  cfg.kv_lora_rank, getattr(lw, "w_uk_t", None))
        o_lat = ops.mla_paged_attention(q_full, ckv, inp.block_tables, inp.seq_lens, inp.cu_q, self.scale,
                                        cfg.kv_lora_rank, inp.max_q_len)
        o = ops.mla_o_absorb(o_lat, lw.w_uv)
        return self.comm.row_linear(o, lw.wo, h)

    # ------------------------------------------------------------------ ffn
    def _ffn_dense(self, lw, h) -> torch.Tensor:
        if lw.shared_limit:      # clamped SwiGLU: the activation is its own op
            act = ops.swiglu(ops.norm_linear(h, lw.ffn_norm, self.cfg.rms_eps, lw.w_gate_up), lw.shared_limit)
        else:
            act = ops.norm_linear(h, lw.ffn_norm, self.cfg.rms_eps, lw.w_gate_up, swiglu=True)
        return self.comm.row_linear(act, lw.w_down, h)

    def _ffn_moe(self, lw, h) -> torch.Tensor:
        """Token-replicated expert parallelism.

        After the attention all-reduce every rank holds all ``T`` hidden rows, so dispatch
        is a local gather of the rows routed to this rank's experts; combine is one sum over
        ranks of the weighted expert outputs (shared-expert partial folded into the same sum).
        """
        cfg = self.cfg
        h, x = reduced_and_normed(h, lw.ffn_norm, cfg.rms_eps)
        if lw.e_gate_up_b is not None:       # GPT-OSS: biased router and experts, its own activation
            logits = ops.linear(x, lw.router).float() + lw.router_b
            wts, ids = ops.moe_route(logits, cfg.n_experts_per_tok, "softmax", True, None, 1, 1, 1.0)
            elo, _ = expert_range(cfg, self.spec)
            y = ops.moe_experts_oai(x, lw.e_gate_up, lw.e_gate_up_b, lw.e_down, lw.e_down_b, wts, ids, elo, cfg.oai_limit)
            return self.comm.row_sum(y, h)
        logits = ops.linear(x, lw.router)
        wts, ids = ops.moe_route(logits, cfg.n_experts_per_tok, cfg.router, cfg.norm_topk_prob, lw.router_bias,
                                 cfg.n_group, cfg.topk_group, cfg.routed_scaling)
        elo, _ = expert_range(cfg, self.spec)
        y = ops.moe_experts(x, lw.e_gate_up, lw.e_down, wts, ids, elo, cfg.n_experts, limit=lw.act_limit)
        if lw.shared_limit and lw.s_gate_up is not None:
            y = ops.linear(ops.swiglu(ops.linear(x, lw.s_gate_up), lw.shared_limit), lw.s_down, residual=y)
        elif lw.s_gate is not None:
            # this rank's slice of the shared expert, scaled per token by sigmoid(x . w_gate) (the gate is replicated)
            sh = ops.linear(ops.linear(x, lw.s_gate_up, swiglu=True), lw.s_down)
            y = ops.scaled_add(y, sh, ops.linear(x, lw.s_gate))
        elif lw.s_gate_up is not None:
            y = ops.linear(ops.linear(x, lw.s_gate_up, swiglu=True), lw.s_down, residual=y)
        return self.comm.row_sum(y, h)      # may stay pending: the next layer's norm is fused into the reduction

    # ------------------------------------------------------------------ forward
    def forward(self, inp: StepInputs, kv: KVPool, hidden_in: torch.Tensor | None = None, need_logits: bool = True):
        """Run this shard over the residual stream ``h [T, H]``.  The last pipeline stage returns
        local-vocab logits ``[B', V/N]`` (``None`` when the caller needs none: a prompt chunk that only fills the
        cache); other stages return ``h`` to send to the next stage."""
        cfg, w = self.cfg, self.w
        if need_logits and inp.max_q_len == 1 and inp.tokens.shape[0] == 1 and self._mega_ready(kv, inp.tokens):
            # batch-1 decode of a dense model on one GPU: the whole step, embedding to logits, is one persistent kernel
            return self._mega(inp.tokens, inp.positions, inp.slots, inp.block_tables, inp.seq_lens, self.inv_freq,
                              self.rope_mscale, cfg.rms_eps, self.scale)
        h = ops.embedding(w.embed, inp.tokens) if self.spec.is_first_stage else hidden_in
        patches = getattr(self, "embed_patches", None)
        if patches and self.spec.is_first_stage:      # input embeddings supplied by the caller (image features); prefill steps only
            for r0, rows in patches:
                h[r0:r0 + rows.shape[0]] = rows.to(device=h.device, dtype=h.dtype)
            self.embed_patches = None
        for i in self.spec.layers(cfg):
            lw = w.layers[i]
            attn = self._attn_linear if cfg.layer_is_linear(i) else self._attn_mla if cfg.mla else self._attn_gqa
            h = attn(lw, h, inp, kv.layers[i])
            h = self._ffn_moe(lw, h) if cfg.layer_is_moe(i) else self._ffn_dense(lw, h)
        if not self.spec.is_last_stage:
            return resolve(h)
        if not need_logits:
            resolve(h)          # completes the last layer's reduction on every rank alike
            return None
        # only the rows whose logits are needed go through the final norm + vocabulary GEMM
        hs = h if (inp.max_q_len == 1 and inp.logit_rows.numel() == h.shape[0]) else resolve(h)[inp.logit_rows.long()]
        return ops.norm_linear(hs, w.final_norm, cfg.rms_eps, w.lm_head)

    def logits(self, inp: StepInputs, kv: KVPool) -> torch.Tensor:
        """Full-vocabulary logits ``[B', V]`` (vocab shards gathered across the TP group)."""
        out = self.forward(inp, kv)
        return self.comm.gather_vocab(out)[:, :self.cfg.vocab]


def default_state_snapshots(cfg: ModelConfig, max_seqs: int) -> int:
    """Snapshot slots for the recurrent state of a hybrid model's cached prefixes (0 for every other model).  Each slot
    is as large as one sequence seat; every rank of an instance derives the same number from the same arguments."""
    return max(2, min(16, max_seqs)) if cfg.has_linear_layers else 0


def make_decoder(cfg: ModelConfig, weights: ModelWeights, spec: ShardSpec | None = None, comm=None) -> Decoder:
    """The forward implementation of the model's family."""
    if cfg.family == "gemma4":
        from .gemma4 import Gemma4Decoder
        return Gemma4Decoder(cfg, weights, spec, comm)
    if cfg.family == "nemotron_h":
        from .nemotron_h import NemotronHDecoder
        return NemotronHDecoder(cfg, weights, spec, comm)
    return Decoder(cfg, weights, spec, comm)


def make_kv_pool(cfg: ModelConfig, spec: ShardSpec, n_blocks: int, block_size: int = 16, device="cpu", dtype=None,
                 max_seqs: int = 64, n_snapshots: int = 0) -> KVPool:
    if cfg.family == "gemma4":
        from .gemma4 import Gemma4KV
        return Gemma4KV(cfg, spec, n_blocks, block_size, device, dtype, max_seqs)
    return KVPool(cfg, spec, n_blocks, block_size, device, dtype, max_seqs, n_snapshots)
