"""Plain PyTorch (fp32-accumulating) definitions of every hot op.

These are the semantic ground truth: the CPU oracle runs on them, and every
sm_100a kernel in ``exo_b200/ops/csrc`` is tested against them.  They replace
the MLX library calls the reference makes for the same work (RMSNorm / RoPE /
SDPA / SwitchGLU / sampling; the call sites are listed in the reference at
``src/exo/worker/engines/mlx/auto_parallel.py:628-652`` and
``src/exo/worker/engines/mlx/generator/generate.py:599-619``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """Returns ``(normed, h)`` where ``h = x + residual`` (or ``x``) and ``normed = h/rms(h)*w``."""
    h = x.float() if residual is None else x.float() + residual.float()
    var = h.pow(2).mean(-1, keepdim=True)
    out = (h * torch.rsqrt(var + eps)) * w.float()
    return out.to(x.dtype), h.to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """``y = x @ w.T (+bias) (+residual)`` with fp32 accumulation; ``w`` is ``[out, in]`` (a block-scaled
    fp8 weight stands for its bf16 dequantisation)."""
    if hasattr(w, "dequantize"):
        w = w.dequantize()
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(gate) * up`` over ``[.., 2F]`` (gate columns first)."""
    F_ = gate_up.shape[-1] // 2
    g, u = gate_up[..., :F_].float(), gate_up[..., F_:].float()
    return (torch.nn.functional.gelu(g, approximate="tanh") * u).to(gate_up.dtype)


def swiglu(gate_up: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` concatenated on the last dim.  ``limit`` > 0: the activated gate is
    capped at ``limit`` and ``up`` clamped to ``+-limit`` (Step-3.5)."""
    g, u = gate_up.float().chunk(2, dim=-1)
    a = F.silu(g)
    if limit:
        a, u = a.clamp(max=limit), u.clamp(-limit, limit)
    return (a * u).to(gate_up.dtype)


def rope_inv_freq(head_dim: int, rope) -> tuple[torch.Tensor, float]:
    """Inverse frequencies (``rot_dim/2`` floats) and the attention magnitude scale.

    Implements default, linear, Llama-3 banded scaling and YaRN (inverse-frequency
    blending with a linear ramp, the convention the reference patches in at
    ``src/exo/worker/engines/mlx/patches/standard_yarn_rope.py:10-67``).
    """
    if rope.kind == "proportional":
        # rotation over the WHOLE head (pairs i, i + head_dim/2) with the frequencies of the first
        # partial_rotary_factor * head_dim / 2 pairs taken against head_dim and the others zero (Gemma-4 full layers)
        n = int(rope.partial_rotary_factor * head_dim // 2)
        inv = 1.0 / (rope.theta ** (torch.arange(0, 2 * n, 2, dtype=torch.float64) / head_dim))
        inv = torch.cat((inv / rope.factor, torch.zeros(head_dim // 2 - n, dtype=torch.float64)))
        return inv.float(), 1.0
    rot = int(head_dim * rope.partial_rotary_factor)
    rot -= rot % 2
    idx = torch.arange(0, rot, 2, dtype=torch.float64)
    inv = 1.0 / (rope.theta ** (idx / rot))
    mscale = 1.0
    if rope.kind == "linear":
        inv = inv / rope.factor
    elif rope.kind == "llama3":
        low_wl = rope.original_max_position / rope.low_freq_factor
        high_wl = rope.original_max_position / rope.high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (rope.original_max_position / wl - rope.low_freq_factor) / (rope.high_freq_factor - rope.low_freq_factor)
        blended = (1 - smooth) * inv / rope.factor + smooth * inv
        inv = torch.where(wl > low_wl, inv / rope.factor, torch.where(wl < high_wl, inv, blended))
    elif rope.kind == "yarn":
        def corr_dim(n_rot: float) -> float:
            return rot * math.log(rope.original_max_position / (n_rot * 2 * math.pi)) / (2 * math.log(rope.theta))
        lo_f, hi_f = corr_dim(rope.beta_fast), corr_dim(rope.beta_slow)
        if getattr(rope, "truncate", True):
            lo_f, hi_f = math.floor(lo_f), math.ceil(hi_f)
        low = max(lo_f, 0)
        high = min(hi_f, rot // 2 - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        extrap_mask = 1 - ramp
        inv = inv / rope.factor * (1 - extrap_mask) + inv * extrap_mask

        def ms(scale: float, m: float) -> float:
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
        if rope.mscale_all_dim:
            mscale = ms(rope.factor, rope.mscale) / ms(rope.factor, rope.mscale_all_dim)
        else:
            mscale = ms(rope.factor, 1.0)
    return inv.float(), float(mscale)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float = 1.0,
         interleaved: bool = False) -> torch.Tensor:
    """Rotary embedding on the first ``2*len(inv_freq)`` dims of ``x [T, heads, D]``.

    ``interleaved=False`` rotates pairs ``(i, i+rot/2)`` (HF Llama); ``True`` rotates
    adjacent pairs ``(2i, 2i+1)`` (DeepSeek's rope sub-vector).
    """
    rot = inv_freq.numel() * 2
    ang = positions.float()[:, None] * inv_freq.float()[None, :]  # [T, rot/2]
    cos, sin = (ang.cos() * mscale)[:, None, :], (ang.sin() * mscale)[:, None, :]
    xr = x[..., :rot].float()
    if interleaved:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)
    else:
        x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
        o = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    out = x.clone()
    out[..., :rot] = o.to(x.dtype)
    return out


def head_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last (head) dim of ``x [T, heads, D]`` (Qwen3 q/k norm)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def kv_append(k: torch.Tensor, v: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
              slots: torch.Tensor) -> None:
    """Scatter ``k, v [T, Hkv, D]`` into paged caches ``[blocks, bs, Hkv, D]`` at flat ``slots [T]``."""
    kc = kcache.view(-1, *kcache.shape[2:])
    vc = vcache.view(-1, *vcache.shape[2:])
    kc[slots.long()] = k.to(kc.dtype)
    vc[slots.long()] = v.to(vc.dtype)


def _gather_seq(cache: torch.Tensor, table: torch.Tensor, n: int) -> torch.Tensor:
    bs = cache.shape[1]
    nb = (n + bs - 1) // bs
    return cache[table[:nb].long()].reshape(nb * bs, *cache.shape[2:])[:n]


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                    seq_lens: torch.Tensor, cu_q: torch.Tensor, scale: float, sliding_window: int = 0,
                    sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Causal GQA attention of new queries over a paged KV cache.

    ``q [T, Hq, D]`` holds the concatenated new tokens of ``B`` sequences, ``cu_q [B+1]``
    their offsets; ``seq_lens[b]`` is the KV length *including* those new tokens (already
    appended).  Query ``j`` of sequence ``b`` sits at position ``seq_lens[b]-q_len+j``.
    """
    T, Hq, D = q.shape
    Hkv = kcache.shape[2]
    Dv = vcache.shape[-1]
    out = torch.empty(T, Hq, Dv, dtype=q.dtype, device=q.device)
    g = Hq // Hkv
    for b in range(seq_lens.numel()):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        if e == s:
            continue
        n = int(seq_lens[b])
        k = _gather_seq(kcache, block_tables[b], n).float()  # [n, Hkv, D]
        v = _gather_seq(vcache, block_tables[b], n).float()
        qb = q[s:e].float().view(e - s, Hkv, g, D)
        sc = torch.einsum("thgd,nhd->hgtn", qb, k) * scale
        qpos = torch.arange(n - (e - s), n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        mask = kpos <= qpos
        if sliding_window:
            mask &= kpos > qpos - sliding_window
        sc = sc.masked_fill(~mask[None, None], float("-inf"))
        if sinks is not None:
            sk = sinks.float().view(Hkv, g, 1, 1).expand(Hkv, g, e - s, 1)
            p = torch.softmax(torch.cat((sc, sk), -1), -1)[..., :-1]
        else:
            p = torch.softmax(sc, -1)
        out[s:e] = torch.einsum("hgtn,nhd->thgd", p, v).reshape(e - s, Hq, Dv).to(q.dtype)
    return out


def mla_paged_attention(q_lat: torch.Tensor, q_rope: torch.Tensor, ckv: torch.Tensor, block_tables: torch.Tensor,
                        seq_lens: torch.Tensor, cu_q: torch.Tensor, scale: float, kv_lora: int) -> torch.Tensor:
    """Weight-absorbed MLA attention over a paged latent cache.

    ``q_lat [T, H, kv_lora]`` is ``q_nope·W_UK``; ``q_rope [T, H, r]``; the cache row per
    token is ``[c_kv (kv_lora) | k_rope (r)]`` shared by all heads.  Returns the attention
    output still in latent space ``[T, H, kv_lora]`` (the caller applies ``W_UV``).
    """
    T, H, _ = q_lat.shape
    out = torch.empty(T, H, kv_lora, dtype=q_lat.dtype, device=q_lat.device)
    for b in range(seq_lens.numel()):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        if e == s:
            continue
        n = int(seq_lens[b])
        c = _gather_seq(ckv, block_tables[b], n).float()  # [n, kv_lora + r]
        sc = (torch.einsum("thc,nc->htn", q_lat[s:e].float(), c[:, :kv_lora])
              + torch.einsum("thr,nr->htn", q_rope[s:e].float(), c[:, kv_lora:])) * scale
        qpos = torch.arange(n - (e - s), n, device=q_lat.device)[:, None]
        mask = torch.arange(n, device=q_lat.device)[None, :] <= qpos
        p = torch.softmax(sc.masked_fill(~mask[None], float("-inf")), -1)
        out[s:e] = torch.einsum("htn,nc->thc", p, c[:, :kv_lora]).to(q_lat.dtype)
    return out


def mla_kv_append(kva: torch.Tensor, norm_w: torch.Tensor, eps: float, positions: torch.Tensor, inv_freq: torch.Tensor,
                  mscale: float, cache: torch.Tensor, slots: torch.Tensor, kv_lora: int) -> None:
    """Write the new tokens' latent-cache rows: ``[rmsnorm(kva[:, :kv_lora]) | rope(kva[:, kv_lora:])]``."""
    c_kv, _ = rmsnorm(kva[:, :kv_lora].contiguous(), norm_w, eps)
    k_rope = rope(kva[:, None, kv_lora:], positions, inv_freq, mscale, True)[:, 0]
    cache.view(-1, cache.shape[-1])[slots.long()] = torch.cat((c_kv, k_rope), -1).to(cache.dtype)


def mla_q_absorb(q: torch.Tensor, w_uk: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float,
                 nope: int) -> torch.Tensor:
    """``q [T, H, nope + r]`` -> ``[T, H, kv_lora + r]``: ``q_nope . W_UK[h]`` in front, the rotated rope part behind."""
    q_lat = torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_uk.float()).to(q.dtype)
    q_rope = rope(q[..., nope:], positions, inv_freq, mscale, True)
    return torch.cat((q_lat, q_rope), -1)


def mla_o_absorb(o_lat: torch.Tensor, w_uv: torch.Tensor) -> torch.Tensor:
    """``o_lat [T, H, kv_lora]`` with ``w_uv [H, v, kv_lora]`` -> ``[T, H * v]``."""
    return torch.einsum("thc,hvc->thv", o_lat.float(), w_uv.float()).to(o_lat.dtype).reshape(o_lat.shape[0], -1)


def moe_route(logits: torch.Tensor, top_k: int, kind: str = "softmax", norm_topk: bool = True,
              bias: torch.Tensor | None = None, n_group: int = 1, topk_group: int = 1,
              scaling: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k routing.  Returns ``(weights [T,k] fp32, expert ids [T,k] int32)``.

    ``softmax``: probabilities over all experts, top-k, optional renormalisation (Qwen3-MoE).
    ``sigmoid``: DeepSeek-V3 — sigmoid scores, selection on ``score+bias`` restricted to the
    best ``topk_group`` of ``n_group`` groups (group score = sum of its two best), weights
    taken from the unbiased scores, renormalised and multiplied by ``scaling``.
    """
    lf = logits.float()
    if kind == "softmax":
        p = torch.softmax(lf, -1)
        w, idx = torch.topk(p, top_k, dim=-1)
        if norm_topk:
            w = w / w.sum(-1, keepdim=True)
        return w * scaling, idx.int()
    s = torch.sigmoid(lf)
    sel = s + bias.float() if bias is not None else s
    if n_group > 1:
        T, E = sel.shape
        gs = sel.view(T, n_group, E // n_group).topk(2, dim=-1)[0].sum(-1)
        gidx = gs.topk(topk_group, dim=-1)[1]
        gmask = torch.zeros_like(gs).scatter_(1, gidx, 1.0)
        sel = sel.masked_fill(gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E) == 0, float("-inf"))
    idx = sel.topk(top_k, dim=-1)[1]
    w = s.gather(1, idx)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling, idx.int()


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, weights: torch.Tensor,
                ids: torch.Tensor, expert_offset: int = 0, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """Weighted sum of experts: ``w_gate_up [E, 2F, H]``, ``w_down [E, H, F]``; ``act`` ``silu`` (SwiGLU), ``gelu_tanh``
    (GeGLU) or ``relu2`` (``w_gate_up [E, F, H]``, no gate: ``down(relu(up x)^2)``).

    Only experts ``expert_offset <= id < expert_offset+E`` are evaluated (the caller's local
    shard under expert parallelism); others contribute zero.
    """
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w_gate_up.shape[0]
    for e in range(E):
        tok, slot = torch.where(ids == e + expert_offset)
        if tok.numel() == 0:
            continue
        pre = linear(x[tok], w_gate_up[e])
        h = swiglu(pre, limit) if act == "silu" else geglu(pre) if act == "gelu_tanh" else torch.relu(pre.float()).pow(2).to(pre.dtype)
        y = linear(h, w_down[e]).float()
        out.index_add_(0, tok, y * weights[tok, slot][:, None])
    return out.to(x.dtype)


def moe_experts_oai(x: torch.Tensor, w_gate_up: torch.Tensor, b_gate_up: torch.Tensor, w_down: torch.Tensor, b_down: torch.Tensor,
                    weights: torch.Tensor, ids: torch.Tensor, expert_offset: int = 0, limit: float = 7.0, alpha: float = 1.702) -> torch.Tensor:
    """GPT-OSS experts: ``w_gate_up [E, 2F, H]`` (gate rows, then up rows) and ``w_down [E, H, F]`` with biases ``[E, 2F]`` /
    ``[E, H]``; ``(up + 1) * gate * sigmoid(alpha * gate)`` with the gate capped at ``limit`` and the up projection clamped to
    ``+-limit``.  Experts outside ``[expert_offset, expert_offset + E)`` contribute zero."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(w_gate_up.shape[0]):
        tok, slot = torch.where(ids == e + expert_offset)
        if tok.numel() == 0:
            continue
        pre = linear(x[tok], w_gate_up[e]).float() + b_gate_up[e].float()
        g, u = pre.chunk(2, dim=-1)
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        h = ((u + 1.0) * g * torch.sigmoid(alpha * g)).to(x.dtype)
        y = linear(h, w_down[e]).float() + b_down[e].float()
        out.index_add_(0, tok, y * weights[tok, slot][:, None])
    return out.to(x.dtype)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor) -> torch.Tensor:
    """Per-row temperature / top-k / top-p / min-p sampling by inverse CDF with ``uniform [B]``.

    ``temperature == 0`` selects argmax.  Filters compose in the order top-k → top-p → min-p
    on the temperature-scaled distribution.  Returns int64 ids ``[B]``.
    """
    B, V = logits.shape
    lf = logits.float()
    greedy = lf.argmax(-1)
    t = temperature.float().clamp_min(1e-6)[:, None]
    probs = torch.softmax(lf / t, -1)
    sp, si = probs.sort(-1, descending=True)
    rank = torch.arange(V, device=logits.device)[None, :]
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V))[:, None]
    keep = rank < k
    cum = sp.cumsum(-1)
    keep &= (cum - sp) < top_p.float()[:, None]
    keep &= sp >= min_p.float()[:, None] * sp[:, :1]
    keep[:, 0] = True
    # inverse CDF over the kept tokens in *vocabulary* order (what the device kernel does)
    kept = torch.zeros_like(probs).scatter_(1, si, sp * keep)
    cdf = kept.cumsum(-1)
    target = uniform.float()[:, None] * cdf[:, -1:]
    pick = (cdf <= target).sum(-1).clamp_max(V - 1)
    # never return a filtered token (target == total mass lands past the last kept one)
    last_kept = (V - 1) - (kept.flip(-1) > 0).float().argmax(-1)
    sampled = torch.minimum(pick, last_kept)
    return torch.where(temperature <= 0, greedy, sampled)


def apply_penalties(logits: torch.Tensor, counts: torch.Tensor, repetition: torch.Tensor,
                    presence: torch.Tensor, frequency: torch.Tensor) -> torch.Tensor:
    """Repetition (multiplicative), presence and frequency (additive) penalties from token counts ``[B,V]``."""
    lf = logits.float()
    seen = counts > 0
    rep = repetition.float()[:, None]
    lf = torch.where(seen, torch.where(lf > 0, lf / rep, lf * rep), lf)
    lf = lf - presence.float()[:, None] * seen.float() - frequency.float()[:, None] * counts.float()
    return lf


def top_logprobs(logits: torch.Tensor, chosen: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(logprob of chosen [B], top-k logprobs [B,k], top-k ids [B,k])`` from raw logits."""
    lp = torch.log_softmax(logits.float(), -1)
    tv, ti = lp.topk(k, dim=-1)
    return lp.gather(1, chosen.long()[:, None])[:, 0], tv, ti


# ----------------------------------------------------------------------------
# Gated delta rule (the linear-attention layers of Qwen3-Next / Qwen3.5)
# ----------------------------------------------------------------------------
def gated_delta_sequence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                         state: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The recurrence itself, one token after another, for ONE sequence.

    ``q, k [L, hv, dk]`` (already L2-normalised, q already scaled), ``v [L, hv, dv]``, ``g, beta [L, hv]``,
    ``state [hv, dk, dv]`` fp32.  Per token: ``S <- S * exp(g)``; ``delta = (v - k . S) * beta``;
    ``S <- S + k (x) delta``; ``o = q . S``.  Returns ``(o [L, hv, dv], S)``."""
    S = state.clone()
    out = torch.empty(v.shape, dtype=torch.float32, device=v.device)
    for t in range(q.shape[0]):
        S = S * g[t].exp()[:, None, None]
        mem = (S * k[t][:, :, None]).sum(1)
        delta = (v[t] - mem) * beta[t][:, None]
        S = S + k[t][:, :, None] * delta[:, None, :]
        out[t] = (S * q[t][:, :, None]).sum(1)
    return out, S


def gated_delta_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                        state: torch.Tensor, chunk: int = 64) -> tuple[torch.Tensor, torch.Tensor]:
    """The same map as ``gated_delta_sequence`` in its chunk-parallel form (matrix products over blocks of ``chunk``
    tokens; the state crosses chunk borders only).  Within a chunk the dependency of token i on the deltas of tokens
    j < i is a unit lower-triangular system, solved by forward substitution; everything else is GEMM-shaped."""
    L, hv, dk = q.shape
    dv = v.shape[-1]
    pad = (-L) % chunk
    if pad:
        z = lambda t: torch.cat((t, t.new_zeros((pad,) + t.shape[1:])), 0)      # noqa: E731
        q, k, v, g, beta = z(q), z(k), z(v), z(g), z(beta)
    n = (L + pad) // chunk
    # [hv, n, chunk, .]
    hd = lambda t: t.reshape(n, chunk, hv, -1).permute(2, 0, 1, 3).float()         # noqa: E731
    q, k, v = hd(q), hd(k), hd(v)
    g = g.reshape(n, chunk, hv).permute(2, 0, 1).float()
    beta = beta.reshape(n, chunk, hv).permute(2, 0, 1).float()
    gc = g.cumsum(-1)                                                  # decay from the chunk's start to each token
    kb, vb = k * beta[..., None], v * beta[..., None]
    tri_incl = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 0)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()  # exp(gc_i - gc_j) for j <= i
    A = -((kb @ k.transpose(-1, -2)) * decay).masked_fill(tri_incl, 0)
    for i in range(1, chunk):                                          # (I - A)^-1 by forward substitution
        row = A[..., i, :i].clone()
        A[..., i, :i] = row + (row.unsqueeze(-1) * A[..., :i, :i].clone()).sum(-2)
    A = A + torch.eye(chunk, dtype=A.dtype, device=A.device)
    u = A @ vb                                                         # deltas if the incoming state were zero
    w = A @ (kb * gc.exp()[..., None])                                 # what the incoming state takes away from them
    S = state.float().clone()
    out = torch.empty(hv, n, chunk, dv, dtype=torch.float32, device=q.device)
    tri_excl = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 1)
    for c in range(n):
        qc, kc = q[:, c], k[:, c]
        attn = ((qc @ kc.transpose(-1, -2)) * decay[:, c]).masked_fill(tri_excl, 0)
        delta = u[:, c] - w[:, c] @ S
        out[:, c] = (qc * gc[:, c, :, None].exp()) @ S + attn @ delta
        last = gc[:, c, -1]
        S = S * last[:, None, None].exp() + (kc * (last[:, None] - gc[:, c]).exp()[..., None]).transpose(-1, -2) @ delta
    out = out.permute(1, 2, 0, 3).reshape(n * chunk, hv, dv)[:L]
    return out, S


def gated_delta(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor,
                eps: float, conv_state: torch.Tensor, rec_state: torch.Tensor, seats: torch.Tensor, cu_q: torch.Tensor,
                positions: torch.Tensor, hk: int, hv: int, dk: int, dv: int, chunk: int = 64) -> torch.Tensor:
    """One gated-delta-rule layer between its input projection and its output projection, over a ragged batch.

    ``proj [T, 2*hk*dk + 2*hv*dv + 2*hv]`` holds, per token, ``q | k | v | z | b | a``.  Per sequence ``s`` (tokens
    ``cu_q[s] .. cu_q[s+1]``, state seat ``seats[s]``; a sequence whose first token has position 0 starts from zero
    state):

    1. ``q | k | v`` go through a causal depthwise convolution with ``conv_w [2*hk*dk + hv*dv, taps]`` whose history is
       the seat's ``conv_state [., channels, taps-1]``, then SiLU;
    2. q and k are L2-normalised per head, q scaled by ``dk**-0.5``; a key head serves ``hv / hk`` value heads;
    3. ``beta = sigmoid(b)``, ``g = -exp(a_log) * softplus(a + dt_bias)``; the recurrence of ``gated_delta_sequence``
       runs from the seat's ``rec_state [., hv, dk, dv]`` and leaves the new state there;
    4. the output is RMS-normalised per value head, times ``norm_w [dv]``, times ``silu(z)``.

    Returns ``[T, hv*dv]`` in ``proj``'s dtype.  Definition followed: ``Qwen3NextGatedDeltaNet.forward`` of the
    ``transformers`` library (the reference runs the same layer through ``mlx_lm.models.qwen3_next``)."""
    T = proj.shape[0]
    kd, vd = hk * dk, hv * dv
    taps = conv_w.shape[1]
    qkv, z, b, a = proj.float().split((2 * kd + vd, vd, hv, hv), -1)
    out = torch.zeros(T, hv, dv, dtype=torch.float32, device=proj.device)
    cu = cu_q.tolist()
    seat_l = seats.tolist()
    w = conv_w.float()
    for s in range(len(cu) - 1):
        t0, t1 = cu[s], cu[s + 1]
        if t1 <= t0:
            continue
        seat = seat_l[s]
        fresh = int(positions[t0]) == 0
        hist = torch.zeros(taps - 1, 2 * kd + vd, device=proj.device) if fresh else conv_state[seat].float().t()
        x = torch.cat((hist, qkv[t0:t1]), 0)                                     # [taps-1+L, C]
        conv_state[seat] = x[-(taps - 1):].t().to(conv_state.dtype)
        y = sum(x[j:j + (t1 - t0)] * w[:, j] for j in range(taps))
        y = torch.nn.functional.silu(y)
        q, k, v = y.split((kd, kd, vd), -1)
        L = t1 - t0
        q, k = q.reshape(L, hk, dk), k.reshape(L, hk, dk)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(hv // hk, 1), k.repeat_interleave(hv // hk, 1)
        beta = torch.sigmoid(b[t0:t1])
        g = -a_log.float().exp() * torch.nn.functional.softplus(a[t0:t1] + dt_bias.float())
        S0 = torch.zeros_like(rec_state[seat]) if fresh else rec_state[seat]
        fn = gated_delta_sequence if L < chunk else gated_delta_chunked
        o, S1 = fn(q, k, v.reshape(L, hv, dv), g, beta, S0.float())
        rec_state[seat] = S1.to(rec_state.dtype)
        out[t0:t1] = o
    out = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    out = out * torch.nn.functional.silu(z.reshape(T, hv, dv))
    return out.reshape(T, vd).to(proj.dtype)


def mamba2(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor | None, a_log: torch.Tensor, dt_bias: torch.Tensor,
           skip: torch.Tensor, norm_w: torch.Tensor, eps: float, conv_state: torch.Tensor, ssm_state: torch.Tensor,
           seats: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor, groups: int, heads: int, d_state: int,
           head_dim: int) -> torch.Tensor:
    """A Mamba-2 mixer between its input and output projections over a ragged batch.

    ``proj [T, 2*groups*d_state + 2*heads*head_dim + 2*heads]`` holds, per token, ``C | B | x | z | dt | dt`` (the time step
    twice: the layout is the gated delta rule's, whose kernels run this recurrence too).  Per sequence (state seat
    ``seats[s]``; a first token at position 0 starts from zero state):

    1. ``C | B | x`` go through the causal depthwise convolution (``conv_w [channels, taps]``, ``conv_b``) with the seat's
       history, then SiLU;
    2. per head ``h`` of group ``g``: ``dt = softplus(dt + dt_bias[h])``, ``S <- S * exp(-exp(a_log[h]) * dt) +
       B_g (x) (dt * x_h)``, ``y_h = C_g . S + skip[h] * x_h`` with ``S [d_state, head_dim]`` kept in
       ``ssm_state [., heads, d_state, head_dim]``;
    3. ``y * silu(z)`` is RMS-normalised over groups of ``heads*head_dim/groups`` channels and scaled by ``norm_w``.

    Definition followed: ``NemotronHMamba2Mixer.torch_forward`` of the ``transformers`` library, with the time step
    limited to ``(0, inf)`` as the kernels of ``mamba_ssm`` and the reference's ``mlx_lm.models.nemotron_h`` do."""
    T = proj.shape[0]
    gn, width = groups * d_state, heads * head_dim
    taps = conv_w.shape[1]
    cbx, z, dt, _ = proj.float().split((2 * gn + width, width, heads, heads), -1)
    out = torch.zeros(T, heads, head_dim, dtype=torch.float32, device=proj.device)
    cu, seat_l = cu_q.tolist(), seats.tolist()
    w = conv_w.float()
    A = -a_log.float().exp()
    rep = heads // groups
    for s in range(len(cu) - 1):
        t0, t1 = cu[s], cu[s + 1]
        if t1 <= t0:
            continue
        seat = seat_l[s]
        fresh = int(positions[t0]) == 0
        hist = torch.zeros(taps - 1, 2 * gn + width, device=proj.device) if fresh else conv_state[seat].float().t()
        xin = torch.cat((hist, cbx[t0:t1]), 0)
        conv_state[seat] = xin[-(taps - 1):].t().to(conv_state.dtype)
        L = t1 - t0
        yc = sum(xin[j:j + L] * w[:, j] for j in range(taps))
        if conv_b is not None:
            yc = yc + conv_b.float()
        yc = torch.nn.functional.silu(yc)
        Cm, Bm, x = yc.split((gn, gn, width), -1)
        Cm = Cm.reshape(L, groups, d_state).repeat_interleave(rep, 1)
        Bm = Bm.reshape(L, groups, d_state).repeat_interleave(rep, 1)
        x = x.reshape(L, heads, head_dim)
        step = torch.nn.functional.softplus(dt[t0:t1] + dt_bias.float())             # [L, heads]
        S = torch.zeros_like(ssm_state[seat], dtype=torch.float32) if fresh else ssm_state[seat].float().clone()
        for t in range(L):
            S = S * (step[t] * A).exp()[:, None, None] + Bm[t][:, :, None] * (step[t][:, None] * x[t])[:, None, :]
            out[t0 + t] = (S * Cm[t][:, :, None]).sum(1) + skip.float()[:, None] * x[t]
        ssm_state[seat] = S.to(ssm_state.dtype)
    y = out.reshape(T, width) * torch.nn.functional.silu(z)
    gsize = width // groups
    yg = y.reshape(T, groups, gsize)
    yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + eps)
    return (yg.reshape(T, width) * norm_w.float()).to(proj.dtype)
