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

    def W(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        if name not in self._cache:
            self._cache[name] = self.src.get(name, shape).float()
        return self._cache[name]

    @staticmethod
    def _norm(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _attn(self, i: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c, p = self.cfg, f"model.layers.{i}.self_attn."
        T, H, D = x.shape[0], c.hidden, c.head_dim
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
            k_rope = ref.rope(kva[:, None, c.kv_lora_rank:], pos, self.inv_freq, self.mscale, True)
            q_rope = ref.rope(q[..., c.qk_nope_dim:], pos, self.inv_freq, self.mscale, True)
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
            q = x @ self.W(p + "q_proj.weight", (c.n_heads * D, H)).t()
            k = x @ self.W(p + "k_proj.weight", (c.n_kv_heads * D, H)).t()
            v = x @ self.W(p + "v_proj.weight", (c.n_kv_heads * D, H)).t()
            if c.attn_bias:
                q = q + self.W(p + "q_proj.bias", (c.n_heads * D,))
                k = k + self.W(p + "k_proj.bias", (c.n_kv_heads * D,))
                v = v + self.W(p + "v_proj.bias", (c.n_kv_heads * D,))
            if c.qk_norm_full:
                q = self._norm(q, self.W(p + "q_norm.weight", (c.n_heads * D,)), c.rms_eps)
                k = self._norm(k, self.W(p + "k_norm.weight", (c.n_kv_heads * D,)), c.rms_eps)
            q, k, v = q.view(T, c.n_heads, D), k.view(T, c.n_kv_heads, D), v.view(T, c.n_kv_heads, D)
            if c.qk_norm:
                q = self._norm(q, self.W(p + "q_norm.weight", (D,)), c.rms_eps)
                k = self._norm(k, self.W(p + "k_norm.weight", (D,)), c.rms_eps)
            q = ref.rope(q, pos, self.inv_freq, self.mscale)
            k = ref.rope(k, pos, self.inv_freq, self.mscale)
            scale, n_kv, dv = D ** -0.5, c.n_kv_heads, D
        self.k[i] = k if self.k[i] is None else torch.cat((self.k[i], k), 0)
        self.v[i] = v if self.v[i] is None else torch.cat((self.v[i], v), 0)
        K, V = self.k[i], self.v[i]
        n = K.shape[0]
        g = c.n_heads // n_kv
        sc = torch.einsum("thgd,nhd->hgtn", q.view(T, n_kv, g, -1), K) * scale
        qpos = torch.arange(n - T, n)[:, None]
        keys = torch.arange(n)[None, :]
        vis = keys <= qpos
        if c.sliding_window:
            vis &= keys > qpos - c.sliding_window          # the last `window` keys up to and including the query's own
        sc = sc.masked_fill(~vis[None, None], float("-inf"))
        if c.attn_sinks:
            # one learned logit per head joins the softmax and absorbs probability mass, but contributes no value
            sink = self.W(p + "sinks", (c.n_heads,)).view(n_kv, g, 1, 1).expand(n_kv, g, T, 1)
            pr = torch.softmax(torch.cat((sc, sink), -1), -1)[..., :n]
        else:
            pr = torch.softmax(sc, -1)
        o = torch.einsum("hgtn,nhd->thgd", pr, V).reshape(T, c.n_heads * dv)
        return o @ self.W(p + "o_proj.weight", (H, c.n_heads * dv)).t()

    def _ffn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        from .weights import moe_names
        c, H = self.cfg, self.cfg.hidden
        nm = moe_names(c)
        p = f"model.layers.{i}." + (nm["prefix"] if c.layer_is_moe(i) else "mlp.")

        def mlp(prefix: str, F_: int, t: torch.Tensor, names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")) -> torch.Tensor:
            g = t @ self.W(prefix + names[0], (F_, H)).t()
            u = t @ self.W(prefix + names[1], (F_, H)).t()
            return (F.silu(g) * u) @ self.W(prefix + names[2], (H, F_)).t()

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
        return y

    def forward(self, tokens: torch.Tensor, start_pos: int) -> torch.Tensor:
        """Logits ``[T, V]`` for ``tokens [T]`` appended at ``start_pos``."""
        c = self.cfg
        pos = torch.arange(start_pos, start_pos + tokens.numel())
        h = self.W("model.embed_tokens.weight", (c.vocab, c.hidden))[tokens.long()]
        for i in range(c.n_layers):
            p = f"model.layers.{i}."
            h = h + self._attn(i, self._norm(h, self.W(p + "input_layernorm.weight", (c.hidden,)), c.rms_eps), pos)
            h = h + self._ffn(i, self._norm(h, self.W(p + "post_attention_layernorm.weight", (c.hidden,)), c.rms_eps))
        h = self._norm(h, self.W("model.norm.weight", (c.hidden,)), c.rms_eps)
        head = "model.embed_tokens.weight" if c.tie_embeddings else "lm_head.weight"
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
