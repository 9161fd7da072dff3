"""A latent diffusion transformer (MMDiT-style) and its rectified-flow sampler, in plain PyTorch.

The reference generates images with mflux's FLUX.1 / Qwen-Image models (joint text+image blocks
followed by single-stream blocks, adaLN modulation from the timestep and a pooled text vector,
rectified-flow Euler sampling; ``src/exo/worker/engines/image/models/{flux,qwen}/*``,
``pipeline/runner.py``).  This module has the same structure at configurable size so the
serving path, the pipeline / CFG / patch parallel schedules and the API can be exercised end to
end with weights drawn from a seed, identically on every rank; it stands in for model cards whose
checkpoint folder is not on disk (and for Qwen-Image, whose checkpoint loader is not built).  The
published FLUX.1 checkpoints run on ``flux.FluxModel``, which has this class's interface.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class DitConfig:
    hidden: int = 256
    n_heads: int = 4
    n_joint: int = 2            # blocks with separate text / image streams and joint attention
    n_single: int = 4           # blocks over the concatenated stream
    latent_channels: int = 16
    patch: int = 2
    vae_scale: int = 8          # pixels per latent cell
    text_len: int = 64
    vocab: int = 259
    uses_cfg: bool = False
    guidance: float = 3.5

    @property
    def n_blocks(self) -> int:
        return self.n_joint + self.n_single

    @classmethod
    def for_card(cls, n_layers: int, hidden: int, uses_cfg: bool) -> "DitConfig":
        n_layers = max(2, n_layers)
        return cls(hidden=min(hidden, 512) // 64 * 64 or 64, n_heads=max(1, min(hidden, 512) // 64),
                   n_joint=max(1, n_layers // 3), n_single=n_layers - max(1, n_layers // 3), uses_cfg=uses_cfg)


def steps_for_quality(quality: str) -> int:
    return {"low": 4, "medium": 8, "high": 16}.get(quality, 8)


def _init(gen: torch.Generator, *shape: int, scale: float | None = None) -> torch.Tensor:
    s = scale if scale is not None else 1.0 / math.sqrt(shape[-1])
    return torch.randn(*shape, generator=gen) * s


class Block:
    """One transformer block.  ``joint``: text and image tokens have their own projections and
    modulation and attend jointly; otherwise one set of weights over the concatenated stream."""

    def __init__(self, cfg: DitConfig, joint: bool, gen: torch.Generator):
        H = cfg.hidden
        self.joint, self.H, self.nh = joint, H, cfg.n_heads
        streams = 2 if joint else 1
        self.w_qkv = [_init(gen, 3 * H, H) for _ in range(streams)]
        self.w_o = [_init(gen, H, H) for _ in range(streams)]
        self.w_up = [_init(gen, 4 * H, H) for _ in range(streams)]
        self.w_down = [_init(gen, H, 4 * H) for _ in range(streams)]
        self.w_mod = [_init(gen, 6 * H, H, scale=0.02) for _ in range(streams)]

    def to(self, device) -> "Block":
        for name in ("w_qkv", "w_o", "w_up", "w_down", "w_mod"):
            setattr(self, name, [t.to(device) for t in getattr(self, name)])
        return self

    def _heads(self, x: torch.Tensor) -> torch.Tensor:
        return x.view(x.shape[0], self.nh, self.H // self.nh).transpose(0, 1)

    def qkv(self, x: torch.Tensor, vec: torch.Tensor, s: int):
        """Modulated pre-norm projections of one stream: (q, k, v, gates)."""
        m = F.linear(F.silu(vec), self.w_mod[s]).chunk(6, dim=-1)
        h = F.layer_norm(x, (self.H,)) * (1 + m[1]) + m[0]
        q, k, v = F.linear(h, self.w_qkv[s]).chunk(3, dim=-1)
        return self._heads(q), self._heads(k), self._heads(v), m

    def finish(self, x: torch.Tensor, attn: torch.Tensor, m, s: int) -> torch.Tensor:
        x = x + m[2] * F.linear(attn.transpose(0, 1).reshape(x.shape[0], self.H), self.w_o[s])
        h = F.layer_norm(x, (self.H,)) * (1 + m[4]) + m[3]
        return x + m[5] * F.linear(F.gelu(F.linear(h, self.w_up[s]), approximate="tanh"), self.w_down[s])

    def forward(self, txt: torch.Tensor, img: torch.Tensor, vec: torch.Tensor, kv_cache=None, rows: slice | None = None):
        """``rows`` (with ``kv_cache``): only these image tokens are fresh (patch-parallel step);
        keys / values of the other image tokens come from the cache of the previous step."""
        si = 1 if self.joint else 0
        qt, kt, vt, mt = self.qkv(txt, vec, 0)
        qi, ki, vi, mi = self.qkv(img, vec, si)
        if kv_cache is not None:
            if rows is None:
                kv_cache[0], kv_cache[1] = ki.clone(), vi.clone()
            else:
                kv_cache[0][:, rows], kv_cache[1][:, rows] = ki, vi
                ki, vi = kv_cache[0], kv_cache[1]
        k = torch.cat((kt, ki), dim=1)
        v = torch.cat((vt, vi), dim=1)
        at = F.scaled_dot_product_attention(qt, k, v)
        ai = F.scaled_dot_product_attention(qi, k, v)
        return self.finish(txt, at, mt, 0), self.finish(img, ai, mi, si)


class Dit:
    def __init__(self, cfg: DitConfig, seed: int = 0, blocks: range | None = None, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        gen = torch.Generator().manual_seed(seed)
        H, pc = cfg.hidden, cfg.latent_channels * cfg.patch * cfg.patch
        self.tok_embed = _init(gen, cfg.vocab, H, scale=0.02).to(self.device)
        self.txt_pos = _init(gen, cfg.text_len, H, scale=0.02).to(self.device)
        self.img_in = _init(gen, H, pc).to(self.device)
        self.img_out = _init(gen, pc, H).to(self.device)
        self.t_mlp = (_init(gen, H, 256).to(self.device), _init(gen, H, H).to(self.device))
        self.pool = _init(gen, H, H).to(self.device)
        self.decode_w = _init(gen, 3 * cfg.vae_scale ** 2, cfg.latent_channels, scale=0.35).to(self.device)
        all_blocks = [Block(cfg, i < cfg.n_joint, gen) for i in range(cfg.n_blocks)]     # same draws on every rank
        self.block_range = blocks if blocks is not None else range(cfg.n_blocks)
        self.blocks = {i: all_blocks[i].to(self.device) for i in self.block_range}

    # ---- conditioning ----
    def encode_text(self, prompt: str) -> tuple[torch.Tensor, torch.Tensor]:
        ids = list(prompt.encode("utf-8"))[: self.cfg.text_len - 1] + [256]
        ids += [257] * (self.cfg.text_len - len(ids))
        e = self.tok_embed[torch.tensor(ids, device=self.device)] + self.txt_pos
        return e, torch.tanh(F.linear(e.mean(0), self.pool))

    def time_vec(self, t: float, pooled: torch.Tensor) -> torch.Tensor:
        freqs = torch.exp(-math.log(10000.0) * torch.arange(128, device=self.device) / 128)
        a = t * 1000.0 * freqs
        emb = torch.cat((a.sin(), a.cos()))
        return F.linear(F.silu(F.linear(emb, self.t_mlp[0])), self.t_mlp[1]) + pooled

    # ---- latents <-> tokens <-> pixels ----
    def grid(self, height: int, width: int) -> tuple[int, int]:
        cell = self.cfg.vae_scale * self.cfg.patch
        return max(1, height // cell), max(1, width // cell)

    def patchify(self, lat: torch.Tensor) -> torch.Tensor:        # [C, h, w] -> [tokens, C*p*p]
        C, p = self.cfg.latent_channels, self.cfg.patch
        gh, gw = lat.shape[1] // p, lat.shape[2] // p
        return lat.view(C, gh, p, gw, p).permute(1, 3, 0, 2, 4).reshape(gh * gw, C * p * p)

    def unpatchify(self, tok: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        C, p = self.cfg.latent_channels, self.cfg.patch
        return tok.view(gh, gw, C, p, p).permute(2, 0, 3, 1, 4).reshape(C, gh * p, gw * p)

    def pos_embed(self, gh: int, gw: int) -> torch.Tensor:
        H = self.cfg.hidden
        ys, xs = torch.meshgrid(torch.arange(gh, device=self.device), torch.arange(gw, device=self.device), indexing="ij")
        f = torch.exp(-math.log(10000.0) * torch.arange(H // 4, device=self.device) / (H // 4))
        parts = [fn(c.reshape(-1, 1).float() * f) for c in (ys, xs) for fn in (torch.sin, torch.cos)]
        return torch.cat(parts, dim=-1)

    def decode(self, lat: torch.Tensor) -> torch.Tensor:            # [C, h, w] -> uint8 [H, W, 3]
        s = self.cfg.vae_scale
        px = F.linear(lat.permute(1, 2, 0), self.decode_w)          # [h, w, 3*s*s]
        img = px.view(lat.shape[1], lat.shape[2], 3, s, s).permute(0, 3, 1, 4, 2).reshape(lat.shape[1] * s, lat.shape[2] * s, 3)
        return (torch.sigmoid(img) * 255).round().clamp(0, 255).to(torch.uint8)

    def encode_image(self, rgb: torch.Tensor, gh: int, gw: int) -> torch.Tensor:   # uint8 [H, W, 3] -> [C, h, w]
        p = self.cfg.patch
        x = rgb.permute(2, 0, 1).float().div(255)[None]
        x = F.interpolate(x, size=(gh * p, gw * p), mode="area")[0]                  # [3, h, w]
        logit = torch.logit(x.clamp(0.02, 0.98))
        mix = self.decode_w.view(3, -1, self.cfg.latent_channels).mean(1)             # [3, C]
        return torch.einsum("chw,cd->dhw", logit, torch.linalg.pinv(mix).T)

    # ---- the denoiser ----
    def embed_tokens(self, lat: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        return F.linear(self.patchify(lat), self.img_in) + self.pos_embed(gh, gw)

    def run_blocks(self, txt, img, vec, caches=None, rows: slice | None = None, grid: tuple[int, int] | None = None):
        for i in self.block_range:
            txt, img = self.blocks[i].forward(txt, img, vec, None if caches is None else caches[i], rows)
        return txt, img

    def head_tokens(self, img: torch.Tensor, vec: torch.Tensor | None = None) -> torch.Tensor:
        return F.linear(F.layer_norm(img, (self.cfg.hidden,)), self.img_out)

    def head(self, img: torch.Tensor, gh: int, gw: int, vec: torch.Tensor | None = None) -> torch.Tensor:
        return self.unpatchify(self.head_tokens(img, vec), gh, gw)

    def velocity(self, lat: torch.Tensor, t: float, txt: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        gh, gw = lat.shape[1] // self.cfg.patch, lat.shape[2] // self.cfg.patch
        _, img = self.run_blocks(txt, self.embed_tokens(lat, gh, gw), self.time_vec(t, pooled))
        return self.head(img, gh, gw)


def timesteps(n: int, start: float = 1.0) -> list[float]:
    """Rectified-flow schedule from ``start`` (1 = pure noise) down to 0, shifted toward the noisy end."""
    ts = [start * (1 - i / n) for i in range(n + 1)]
    return [3.0 * t / (1 + 2.0 * t) for t in ts]
