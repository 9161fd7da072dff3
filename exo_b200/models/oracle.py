"""CPU oracle: a deliberately naive dense/MoE/MLA decoder with a contiguous KV cache.

It restates, in plain fp32 PyTorch, the math of the mlx-lm Llama / Qwen3-MoE / DeepSeek-V3
models the reference runs (the reference's own CPU path is MLX-CPU).  It shares no code with
the engine's paged/sharded forward beyond ``rope_inv_freq`` and the routing definition, so
agreement between the two is a real check.  Its greedy token ids for the tiny-Llama config
are the golden output every GPU / TP configuration must reproduce.
"""
from __future__ import annotations

import time

import torch
import torch.nn.functional as F

from ..ops import reference as ref
from .config import ModelConfig, preset
from .weights import RandomSource, TensorSource


class OracleModel:
    def __init__(self, cfg: ModelConfig, src: TensorSource):
        self.cfg, self.src = cfg, src
        rot = cfg.qk_rope_dim if cfg.mla else cfg.head_dim
        self.inv_freq, self.mscale = ref.rope_inv_freq(rot, cfg.rope)
        self.k: list[torch.Tensor | None] = [None] * cfg.n_layers
        self.v: list[torch.Tensor | None] = [None] * cfg.n_layers
        self._cache: dict[str, torch.Tensor] = {}
        self.lin_hist: dict[int, torch.Tensor] = {}     # per gated-delta-rule layer: every convolution input so far
        self.lin_state: dict[int, torch.Tensor] = {}    # ... and the [hv, dk, dv] state
        self.one = 1.0 if cfg.norm_one_plus else 0.0    # zero-centred RMSNorm weights (hub layout of the hybrid models)

    def W(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        if name not in self._cache:
            self._cache[name] = self.src.get(name, shape).float()
        return self._cache[name]

    @staticmethod
    def _norm(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _linear_attn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        """Gated delta rule, token by token, straight from the checkpoint's tensors in their stored (per-key-head
        grouped, or split) row order."""
        c, p = self.cfg, f"{self.cfg.weight_prefix}layers.{i}.linear_attn."
        T, H = x.shape[0], c.hidden
        hk, hv, dk, dv = c.lin_k_heads, c.lin_v_heads, c.lin_k_dim, c.lin_v_dim
        kd, vd, r = hk * dk, hv * dv, hv // hk
        if c.lin_split_proj:
            mixed = x @ self.W(p + "in_proj_qkv.weight", (2 * kd + vd, H)).t()
            z = (x @ self.W(p + "in_proj_z.weight", (vd, H)).t()).view(T, hv, dv)
            b = x @ self.W(p + "in_proj_b.weight", (hv, H)).t()
            a = x @ self.W(p + "in_proj_a.weight", (hv, H)).t()
        else:
            qkvz = (x @ self.W(p + "in_proj_qkvz.weight", (2 * kd + 2 * vd, H)).t()).view(T, hk, 2 * dk + 2 * r * dv)
            ba = (x @ self.W(p + "in_proj_ba.weight", (2 * hv, H)).t()).view(T, hk, 2 * r)
            q_, k_, v_, z = qkvz.split((dk, dk, r * dv, r * dv), -1)
            mixed = torch.cat((q_.reshape(T, kd), k_.reshape(T, kd), v_.reshape(T, vd)), -1)
            z = z.reshape(T, hv, dv)
            b, a = ba[..., :r].reshape(T, hv), ba[..., r:].reshape(T, hv)
        hist = self.lin_hist.get(i)
        hist = mixed if hist is None else torch.cat((hist, mixed), 0)
        self.lin_hist[i] = hist
        w = self.W(p + "conv1d.weight", (2 * kd + vd, 1, c.lin_conv))[:, 0]
        n0 = hist.shape[0] - T
        conv = torch.zeros_like(mixed)
        for t in range(T):
            for j in range(c.lin_conv):
                src_t = n0 + t - (c.lin_conv - 1) + j
                if src_t >= 0:
                    conv[t] += hist[src_t] * w[:, j]
        conv = F.silu(conv)
        q, k, v = conv.split((kd, kd, vd), -1)
        q, k, v = q.view(T, hk, dk), k.view(T, hk, dk), v.view(T, hv, dv)
        q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-6) * dk ** -0.5
        k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-6)
        beta = torch.sigmoid(b)
        g = -self.W(p + "A_log", (hv,)).exp() * F.softplus(a + self.W(p + "dt_bias", (hv,)))
        S = self.lin_state.get(i)
        if S is None:
            S = torch.zeros(hv, dk, dv)
        out = torch.zeros(T, hv, dv)
        for t in range(T):
            for h in range(hv):
                kh, qh = k[t, h // r], q[t, h // r]
                S[h] = S[h] * g[t, h].exp()
                delta = (v[t, h] - kh @ S[h]) * beta[t, h]
                S[h] = S[h] + torch.outer(kh, delta)
                out[t, h] = qh @ S[h]
        self.lin_state[i] = S
        out = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + c.rms_eps) * self.W(p + "norm.weight", (dv,))
        out = out * F.silu(z)
        return out.reshape(T, vd) @ self.W(p + "out_proj.weight", (H, vd)).t()

    def _attn(self, i: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c, p = self.cfg, f"{self.cfg.weight_prefix}layers.{i}.self_attn."
        T, H, D = x.shape[0], c.hidden, c.head_dim
        if c.layer_is_linear(i):
            return self._linear_attn(i, x)
        gate = None
        if c.mla:
            qk = c.qk_nope_dim + c.qk_rope_dim
            if c.q_lora_rank:
                qa = x @ self.W(p + "q_a_proj.weight", (c.q_lora_rank, H)).t()
                qa = self._norm(qa, self.W(p + "q_a_layernorm.weight", (c.q_lora_rank,)), c.rms_eps)
                q = qa @ self.W(p + "q_b_proj.weight", (c.n_heads * qk, c.q_lora_rank)).t()
            else:
                q = x @ self.W(p + "q_proj.weight", (c.n_heads * qk, H)).t()
            q = q.view(T, c.n_heads, qk)
            kva = x @ self.W(p + "kv_a_proj_with_mqa.weight", (c.kv_lora_rank + c.qk_rope_dim, H)).t()
            ckv = self._norm(kva[:, :c.kv_lora_rank], self.W(p + "kv_a_layernorm.weight", (c.kv_lora_rank,)), c.rms_eps)
            k_rope = ref.rope(kva[:, None, c.kv_lora_rank:], pos, self.inv_freq, self.mscale, not c.mla_rope_neox)
            q_rope = ref.rope(q[..., c.qk_nope_dim:], pos, self.inv_freq, self.mscale, not c.mla_rope_neox)
            kvb = ckv @ self.W(p + "kv_b_proj.weight", (c.n_heads * (c.qk_nope_dim + c.v_head_dim), c.kv_lora_rank)).t()
            kvb = kvb.view(T, c.n_heads, c.qk_nope_dim + c.v_head_dim)
            k = torch.cat((kvb[..., :c.qk_nope_dim], k_rope.expand(T, c.n_heads, c.qk_rope_dim)), -1)
            v = kvb[..., c.qk_nope_dim:]
            q = torch.cat((q[..., :c.qk_nope_dim], q_rope), -1)
            scale = qk ** -0.5
            if c.rope.kind == "yarn" and c.rope.mscale_all_dim:
                import math
                m = 0.1 * c.rope.mscale_all_dim * math.log(c.rope.factor) + 1.0
                scale *= m * m
            n_kv, dv = c.n_heads, c.v_head_dim
        else:
            n_heads = c.q_heads(i)                                 # Step-3.5: head count, RoPE and window per layer
            if c.layer_rope:
                inv_freq, mscale = ref.rope_inv_freq(D, c.rope_of(i))
            else:
                inv_freq, mscale = self.inv_freq, self.mscale
            if c.attn_gate:
                qg = (x @ self.W(p + "q_proj.weight", (c.n_heads * 2 * D, H)).t()).view(T, c.n_heads, 2 * D)
                q, gate = qg[..., :D].reshape(T, c.n_heads * D), qg[..., D:].reshape(T, c.n_heads * D)
            else:
                q = x @ self.W(p + "q_proj.weight", (n_heads * D, H)).t()
            k = x @ self.W(p + "k_proj.weight", (c.n_kv_heads * D, H)).t()
            v = x @ self.W(p + "v_proj.weight", (c.n_kv_heads * D, H)).t()
            if c.attn_bias:
                q = q + self.W(p + "q_proj.bias", (c.n_heads * D,))
                k = k + self.W(p + "k_proj.bias", (c.n_kv_heads * D,))
                v = v + self.W(p + "v_proj.bias", (c.n_kv_heads * D,))
            if c.qk_norm_full:
                q = self._norm(q, self.W(p + "q_norm.weight", (c.n_heads * D,)), c.rms_eps)
                k = self._norm(k, self.W(p + "k_norm.weight", (c.n_kv_heads * D,)), c.rms_eps)
            q, k, v = q.view(T, n_heads, D), k.view(T, c.n_kv_heads, D), v.view(T, c.n_kv_heads, D)
            if c.qk_norm:
                q = self._norm(q, self.W(p + "q_norm.weight", (D,)) + self.one, c.rms_eps)
                k = self._norm(k, self.W(p + "k_norm.weight", (D,)) + self.one, c.rms_eps)
            q = ref.rope(q, pos, inv_freq, mscale)
            k = ref.rope(k, pos, inv_freq, mscale)
            scale, n_kv, dv = D ** -0.5, c.n_kv_heads, D
        self.k[i] = k if self.k[i] is None else torch.cat((self.k[i], k), 0)
        self.v[i] = v if self.v[i] is None else torch.cat((self.v[i], v), 0)
        K, V = self.k[i], self.v[i]
        n = K.shape[0]
        n_heads = c.n_heads if c.mla else n_heads
        g = n_heads // n_kv
        sc = torch.einsum("thgd,nhd->hgtn", q.view(T, n_kv, g, -1), K) * scale
        qpos = torch.arange(n - T, n)[:, None]
        keys = torch.arange(n)[None, :]
        vis = keys <= qpos
        if c.window_of(i):
            vis &= keys > qpos - c.window_of(i)            # the last `window` keys up to and including the query's own
        sc = sc.masked_fill(~vis[None, None], float("-inf"))
        if c.attn_sinks:
            # one learned logit per head joins the softmax and absorbs probability mass, but contributes no value
            sink = self.W(p + "sinks", (c.n_heads,)).view(n_kv, g, 1, 1).expand(n_kv, g, T, 1)
            pr = torch.softmax(torch.cat((sc, sink), -1), -1)[..., :n]
        else:
            pr = torch.softmax(sc, -1)
        o = torch.einsum("hgtn,nhd->thgd", pr, V).reshape(T, n_heads * dv)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        if c.head_gate:          # one sigmoid gate per head, projected from the layer's (normed) input
            hg = torch.sigmoid(x @ self.W(p + "g_proj.weight", (n_heads, H)).t())
            o = (o.view(T, n_heads, dv) * hg[..., None]).reshape(T, n_heads * dv)
        out = o @ self.W(p + "o_proj.weight", (H, n_heads * dv)).t()
        if c.attn_bias and c.family == "gpt_oss":          # GPT-OSS has a bias on the output projection too
            out = out + self.W(p + "o_proj.bias", (H,))
        return out

    def _ffn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        from .weights import moe_names
        c, H = self.cfg, self.cfg.hidden
        nm = moe_names(c)
        p = f"{self.cfg.weight_prefix}layers.{i}." + (nm["prefix"] if c.layer_is_moe(i) else "mlp.")

        def mlp(prefix: str, F_: int, t: torch.Tensor, names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"),
                limit: float = 0.0) -> torch.Tensor:
            g = t @ self.W(prefix + names[0], (F_, H)).t()
            u = t @ self.W(prefix + names[1], (F_, H)).t()
            a = F.silu(g)
            if limit:
                a, u = a.clamp(max=limit), u.clamp(-limit, limit)
            return (a * u) @ self.W(prefix + names[2], (H, F_)).t()

        if c.family == "step3p5":
            return self._ffn_step(i, x, mlp)
        if not c.layer_is_moe(i):
            return mlp(p, c.ffn, x)
        logits = x @ self.W(p + "gate.weight", (c.n_experts, H)).t()
        bias = self.src.get(p + nm["bias"], (c.n_experts,)) if c.router_bias else None
        wts, ids = ref.moe_route(logits, c.n_experts_per_tok, c.router, c.norm_topk_prob, bias, c.n_group,
                                 c.topk_group, c.routed_scaling)
        y = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(ids.shape[1]):
                e = int(ids[t, j])
                y[t] += wts[t, j] * mlp(f"{p}experts.{e}.", c.moe_ffn, x[t:t + 1], (nm["gate"], nm["up"], nm["down"]))[0]
        if c.n_shared_experts:
            y = y + mlp(p + "shared_experts.", c.moe_ffn * c.n_shared_experts, x)
        if c.shared_expert_ffn:
            sh = mlp(p + "shared_expert.", c.shared_expert_ffn, x)
            if c.shared_expert_gate:
                sh = sh * torch.sigmoid(x @ self.W(p + "shared_expert_gate.weight", (1, H)).t())
            y = y + sh
        return y

    def _ffn_step(self, i: int, x: torch.Tensor, mlp) -> torch.Tensor:
        """Step-3.5: dense MLP or (stacked) sigmoid-routed experts + shared expert, SwiGLU clamped where the layer says so."""
        c, H = self.cfg, self.cfg.hidden
        p = f"{c.weight_prefix}layers.{i}."
        if not c.layer_is_moe(i):
            return mlp(p + "mlp.", c.ffn, x, limit=c.swiglu_limit(i, shared=True))
        E, F_ = c.n_experts, c.moe_ffn
        logits = x @ self.W(p + "moe.gate.weight", (E, H)).t()
        wts, ids = ref.moe_route(logits, c.n_experts_per_tok, c.router, c.norm_topk_prob, self.src.get(p + "moe.router_bias", (E,)),
                                 1, 1, c.routed_scaling)
        wg, wu, wd = (self.W(p + f"moe.{n}_proj.weight", sh) for n, sh in (("gate", (E, F_, H)), ("up", (E, F_, H)), ("down", (E, H, F_))))
        lim = c.swiglu_limit(i)
        y = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(ids.shape[1]):
                e = int(ids[t, j])
                a, u = F.silu(x[t] @ wg[e].t()), x[t] @ wu[e].t()
                if lim:
                    a, u = a.clamp(max=lim), u.clamp(-lim, lim)
                y[t] += wts[t, j] * ((a * u) @ wd[e].t())
        return y + mlp(p + "share_expert.", c.shared_expert_ffn, x, limit=c.swiglu_limit(i, shared=True))

    def forward(self, tokens: torch.Tensor, start_pos: int) -> torch.Tensor:
        """Logits ``[T, V]`` for ``tokens [T]`` appended at ``start_pos``."""
        c = self.cfg
        pos = torch.arange(start_pos, start_pos + tokens.numel())
        h = self.W(c.weight_prefix + "embed_tokens.weight", (c.vocab, c.hidden))[tokens.long()]
        for i in range(c.n_layers):
            p = f"{self.cfg.weight_prefix}layers.{i}."
            h = h + self._attn(i, self._norm(h, self.W(p + "input_layernorm.weight", (c.hidden,)) + self.one, c.rms_eps), pos)
            h = h + self._ffn(i, self._norm(h, self.W(p + "post_attention_layernorm.weight", (c.hidden,)) + self.one, c.rms_eps))
        h = self._norm(h, self.W(c.weight_prefix + "norm.weight", (c.hidden,)) + self.one, c.rms_eps)
        head = c.weight_prefix + "embed_tokens.weight" if c.tie_embeddings else "lm_head.weight"
        return h @ self.W(head, (c.vocab, c.hidden)).t()

    def greedy(self, prompt: torch.Tensor, n_new: int) -> list[int]:
        logits = self.forward(prompt, 0)
        out = [int(logits[-1].argmax())]
        for s in range(n_new - 1):
            logits = self.forward(torch.tensor([out[-1]]), prompt.numel() + s)
            out.append(int(logits[-1].argmax()))
        return out


def oracle_prompt(n: int = 128, vocab: int = 32000, seed: int = 0) -> torch.Tensor:
    g = torch.Generator()
    g.manual_seed(seed + 12345)
    return torch.randint(0, vocab, (n,), generator=g)


def run_oracle(n_prompt: int = 128, n_new: int = 64, seed: int = 0) -> dict:
    """BASELINE config 1: tiny Llama, fp32, CPU, greedy.  Returns tokens and wall time."""
    cfg = preset("tiny-llama")
    model = OracleModel(cfg, RandomSource(seed=seed))
    prompt = oracle_prompt(n_prompt, cfg.vocab, seed)
    t0 = time.perf_counter()
    toks = model.greedy(prompt, n_new)
    return {"tokens": toks, "wall_s": time.perf_counter() - t0, "prompt": prompt.tolist()}


if __name__ == "__main__":
    r = run_oracle()
    print({"tokens": r["tokens"], "wall_s": round(r["wall_s"], 3)})
