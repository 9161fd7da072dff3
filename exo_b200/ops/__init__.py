"""Hot-op entry points.

Each function takes tensors on one device.  CUDA tensors go to the hand-written
sm_100a kernels in ``exo_b200/ops/csrc`` (bound through ``exo_b200.ops.cuda``); a
missing extension on a CUDA device is an error, never a silent fallback.  CPU tensors
run the fp32 PyTorch definitions in ``exo_b200.ops.reference`` — that path is the
correctness oracle, not a second backend.
"""
from __future__ import annotations

import torch

from . import reference as ref

_cuda = None


def cuda_ops():
    """The ctypes binding of the kernel library (loaded on first use; raises if absent)."""
    global _cuda
    if _cuda is None:
        from . import cuda as _c
        _c.load()
        _cuda = _c
    return _cuda


def rmsnorm(x, w, eps, residual=None):
    if x.is_cuda:
        return cuda_ops().rmsnorm(x, w, eps, residual)
    return ref.rmsnorm(x, w, eps, residual)


def linear(x, w, bias=None, residual=None, swiglu=False):
    """``y = x @ w.T (+bias) (+residual)``; ``swiglu=True`` returns ``silu(y[:, :F]) * y[:, F:]``."""
    if x.is_cuda:
        return cuda_ops().linear(x, w, bias, residual, None, 0.0, swiglu)
    y = ref.linear(x, w, bias, residual)
    return ref.swiglu(y) if swiglu else y


def norm_linear(h, norm_w, eps, w, bias=None, swiglu=False):
    """``linear(rmsnorm(h, norm_w), w)`` — one kernel on the small-batch path.  ``h`` may be a
    tensor-parallel hand-over (``parallel.fused.Handover``): the reduction then happens in this kernel's prologue."""
    if hasattr(h, "norm_linear"):
        return h.norm_linear(norm_w, eps, w, bias, swiglu)
    if h.is_cuda:
        return cuda_ops().linear(h, w, bias, None, norm_w, eps, swiglu)
    y = ref.linear(ref.rmsnorm(h, norm_w, eps)[0], w, bias)
    return ref.swiglu(y) if swiglu else y


def swiglu(gate_up, limit=0.0):
    """``silu(gate) * up``; ``limit`` > 0 caps the activated gate at ``limit`` and clamps ``up`` to ``+-limit``."""
    if gate_up.is_cuda:
        return cuda_ops().swiglu(gate_up, limit)
    return ref.swiglu(gate_up, limit)


def qk_rope_append(qkv, positions, inv_freq, mscale, n_q, n_kv, head_dim, kcache, vcache, slots,
                   q_norm=None, k_norm=None, eps=1e-6, v_unit_norm=False):
    """Split fused ``qkv [T,(n_q+2n_kv)*D]``, apply optional per-head RMSNorm and RoPE to q/k,
    append k/v to the paged cache at ``slots``.  Returns ``q [T, n_q, D]``.  ``v_unit_norm``: v heads are RMS-normalised
    (no weight) before they are stored (Gemma-4).  With ``n_kv == 0`` only q is processed (a layer that reads another
    layer's cache)."""
    if qkv.is_cuda:
        return cuda_ops().qk_rope_append(qkv, positions, inv_freq, mscale, n_q, n_kv, head_dim, kcache, vcache,
                                         slots, q_norm, k_norm, eps, v_unit_norm)
    T = qkv.shape[0]
    q, k, v = qkv.split((n_q * head_dim, n_kv * head_dim, n_kv * head_dim), dim=-1)
    q, k, v = q.reshape(T, n_q, head_dim), k.reshape(T, n_kv, head_dim), v.reshape(T, n_kv, head_dim)
    if q_norm is not None:
        q = ref.head_rmsnorm(q, q_norm, eps)
        if n_kv:
            k = ref.head_rmsnorm(k, k_norm, eps)
    q = ref.rope(q, positions, inv_freq, mscale)
    if n_kv:
        k = ref.rope(k, positions, inv_freq, mscale)
        if v_unit_norm:
            v = ref.head_rmsnorm(v, torch.ones(head_dim, device=v.device), eps)
        ref.kv_append(k, v, kcache, vcache, slots)
    return q


def paged_attention(q, kcache, vcache, block_tables, seq_lens, cu_q, scale, sliding_window=0, sinks=None,
                    max_q_len=None):
    if q.is_cuda:
        return cuda_ops().paged_attention(q, kcache, vcache, block_tables, seq_lens, cu_q, scale, sliding_window,
                                          sinks, max_q_len)
    return ref.paged_attention(q, kcache, vcache, block_tables, seq_lens, cu_q, scale, sliding_window, sinks)


def mla_kv_append(kva, norm_w, eps, positions, inv_freq, mscale, cache, slots, kv_lora):
    """Append the new tokens' rows ``[rmsnorm(latent) | rope(k_rope)]`` to the paged latent cache."""
    if kva.is_cuda:
        return cuda_ops().mla_kv_append(kva, norm_w, eps, positions, inv_freq, mscale, cache, slots, kv_lora)
    return ref.mla_kv_append(kva, norm_w, eps, positions, inv_freq, mscale, cache, slots, kv_lora)


def mla_q_absorb(q, w_uk, positions, inv_freq, mscale, nope, kv_lora, w_uk_t=None):
    """``q [T, H, nope + rope]`` -> queries in cache space ``[T, H, kv_lora + rope]`` (``q_nope . W_UK``, rotated rope)."""
    if q.is_cuda:
        return cuda_ops().mla_q_absorb(q, w_uk, positions, inv_freq, mscale, nope, kv_lora, w_uk_t)
    return ref.mla_q_absorb(q, w_uk, positions, inv_freq, mscale, nope)


def mla_o_absorb(o_lat, w_uv):
    """``o_lat [T, H, kv_lora]`` -> ``[T, H * v]`` through ``W_UV``."""
    if o_lat.is_cuda:
        return cuda_ops().mla_o_absorb(o_lat, w_uv)
    return ref.mla_o_absorb(o_lat, w_uv)


def mla_paged_attention(q_full, ckv, block_tables, seq_lens, cu_q, scale, kv_lora, max_q_len=None):
    """Absorbed MLA attention of ``q_full [T, H, kv_lora + rope]`` over the paged latent cache -> ``[T, H, kv_lora]``."""
    if q_full.is_cuda:
        return cuda_ops().mla_paged_attention(q_full, ckv, block_tables, seq_lens, cu_q, scale, kv_lora, max_q_len)
    return ref.mla_paged_attention(q_full[..., :kv_lora], q_full[..., kv_lora:], ckv, block_tables, seq_lens, cu_q, scale,
                                   kv_lora)


def moe_route(logits, top_k, kind, norm_topk, bias, n_group, topk_group, scaling):
    if logits.is_cuda:
        return cuda_ops().moe_route(logits, top_k, kind, norm_topk, bias, n_group, topk_group, scaling)
    return ref.moe_route(logits, top_k, kind, norm_topk, bias, n_group, topk_group, scaling)


def moe_experts(x, w_gate_up, w_down, weights, ids, expert_offset=0, n_experts_total=None, act="silu", limit=0.0):
    """Weighted sum of the routed experts.  ``act``: ``silu`` / ``gelu_tanh`` (gated) or ``relu2`` (``w_gate_up`` is then the
    single up projection ``[E, F, H]``)."""
    if x.is_cuda:
        return cuda_ops().moe_experts(x, w_gate_up, w_down, weights, ids, expert_offset, n_experts_total, act, limit)
    return ref.moe_experts(x, w_gate_up, w_down, weights, ids, expert_offset, act, limit)


def moe_experts_oai(x, w_gate_up, b_gate_up, w_down, b_down, weights, ids, expert_offset=0, limit=7.0):
    """GPT-OSS experts (biases, capped ``(up + 1) * gate * sigmoid(1.702 gate)``): PyTorch ops on either device (the host reads
    which experts are hit, so a step that runs them cannot be captured in a CUDA graph)."""
    return ref.moe_experts_oai(x, w_gate_up, b_gate_up, w_down, b_down, weights, ids, expert_offset, limit)


def embedding(table, ids):
    if table.is_cuda:
        return cuda_ops().embedding(table, ids)
    return table[ids.long()]


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    if logits.is_cuda:
        return cuda_ops().sample(logits, temperature, top_k, top_p, min_p, uniform)
    return ref.sample(logits, temperature, top_k, top_p, min_p, uniform)


def argmax(logits):
    if logits.is_cuda:
        return cuda_ops().argmax(logits)
    return logits.float().argmax(-1)


def gated_delta(proj, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q, positions, hk, hv, dk, dv):
    """A gated-delta-rule layer between its projections over a ragged batch: causal convolution + SiLU, L2-normalised
    q/k, the recurrence over each sequence's state seat, gated RMSNorm (``reference.gated_delta`` is the definition)."""
    if proj.is_cuda:
        return cuda_ops().gated_delta(proj, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q,
                                      positions, hk, hv, dk, dv)
    return ref.gated_delta(proj, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q, positions,
                           hk, hv, dk, dv)


def sigmoid_gate(x, gate):
    """``x * sigmoid(gate)``, element by element (``gate`` may be a column slice of a wider tensor)."""
    if x.is_cuda:
        return cuda_ops().sigmoid_gate(x, gate)
    return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)


def scaled_add(y, x, logit):
    """``y + x * sigmoid(logit)`` with one ``logit`` per row."""
    if x.is_cuda:
        return cuda_ops().scaled_add(y, x, logit)
    return (y.float() + x.float() * torch.sigmoid(logit.float())).to(y.dtype)


def geglu(gate_up):
    """``gelu_tanh(gate_up[:, :F]) * gate_up[:, F:]``."""
    if gate_up.is_cuda:
        return cuda_ops().geglu(gate_up)
    return ref.geglu(gate_up)


def mamba2(proj, conv_w, conv_b, a_log, dt_bias, skip, norm_w, eps, conv_state, ssm_state, seats, cu_q, positions, groups, heads,
           d_state, head_dim):
    """A Mamba-2 mixer between its projections over a ragged batch (``reference.mamba2`` is the definition)."""
    fn = cuda_ops().mamba2 if proj.is_cuda else ref.mamba2
    return fn(proj, conv_w, conv_b, a_log, dt_bias, skip, norm_w, eps, conv_state, ssm_state, seats, cu_q, positions, groups,
              heads, d_state, head_dim)


def relu2(x):
    """``relu(x)^2`` (torch ops on either device: not a hot path of its own, it sits between two GEMMs)."""
    return torch.relu(x).square()
