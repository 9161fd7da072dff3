"""FLUX.1 (schnell / dev / Krea / Kontext) from its published checkpoint folders.

The reference drives mflux's FLUX models through adapters (``src/exo/worker/engines/image/models/flux/
{adapter,kontext_adapter,wrappers,config}.py``): 19 joint blocks with separate text / image streams, 38 single blocks
over the concatenated stream, adaLN modulation from timestep + guidance + pooled CLIP text, T5 token features as the
text stream, rotary positions over (frame, row, column), a 16-channel VAE with 2x2 latent patches, rectified-flow Euler
steps on a resolution-shifted schedule.  This module is that model over the folder layout the reference's model cards
name (``transformer/``, ``vae/``, ``text_encoder/`` = CLIP-L, ``text_encoder_2/`` = T5-XXL, tensor names of the
``diffusers`` export), with the interface of ``dit.Dit`` so that the pipeline / CFG / PipeFusion schedules of
``pipeline.DiffusionRunner`` run it unchanged: a rank holds only the blocks of its stage.

The denoiser is written against plain tensors in a dict keyed by the checkpoint's names; the two text encoders are
``transformers``' ``CLIPTextModel`` and ``T5EncoderModel`` (they run once per prompt).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
import torch.nn.functional as F


@dataclass
class FluxConfig:
    n_joint: int = 19
    n_single: int = 38
    n_heads: int = 24
    head_dim: int = 128
    in_channels: int = 64                  # latent channels x patch²
    text_dim: int = 4096                   # T5 feature width
    pooled_dim: int = 768                  # CLIP pooled width
    guidance_embeds: bool = True           # dev / Krea / Kontext: the guidance scale is an input of the model
    axes_dims: tuple[int, ...] = (16, 56, 56)
    theta: float = 10000.0
    mlp_ratio: float = 4.0
    text_len: int = 512                    # 256 for schnell
    dynamic_shift: bool = True             # dev: the schedule moves toward the noisy end with the token count
    kontext: bool = False                  # the reference image rides along as extra tokens at frame 1
    guidance: float = 3.5
    # VAE
    latent_channels: int = 16
    patch: int = 2
    vae_scale: int = 8
    vae_channels: tuple[int, ...] = (128, 256, 512, 512)
    vae_layers: int = 2
    vae_groups: int = 32
    scaling_factor: float = 0.3611
    shift_factor: float = 0.1159
    uses_cfg: bool = False                 # guidance-distilled: one pass per step

    @property
    def hidden(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def n_blocks(self) -> int:
        return self.n_joint + self.n_single

    @classmethod
    def from_folder(cls, root: Path) -> "FluxConfig":
        """From ``transformer/config.json``, ``vae/config.json`` and ``scheduler/scheduler_config.json``."""
        t = json.loads((root / "transformer" / "config.json").read_text())
        kw: dict[str, Any] = dict(
            n_joint=t.get("num_layers", 19), n_single=t.get("num_single_layers", 38), n_heads=t.get("num_attention_heads", 24),
            head_dim=t.get("attention_head_dim", 128), in_channels=t.get("in_channels", 64), text_dim=t.get("joint_attention_dim", 4096),
            pooled_dim=t.get("pooled_projection_dim", 768), guidance_embeds=bool(t.get("guidance_embeds", False)),
            axes_dims=tuple(t.get("axes_dims_rope", (16, 56, 56))))
        if (root / "vae" / "config.json").exists():
            v = json.loads((root / "vae" / "config.json").read_text())
            kw.update(latent_channels=v.get("latent_channels", 16), vae_channels=tuple(v.get("block_out_channels", (128, 256, 512, 512))),
                      vae_layers=v.get("layers_per_block", 2), vae_groups=v.get("norm_num_groups", 32),
                      scaling_factor=v.get("scaling_factor", 0.3611), shift_factor=v.get("shift_factor", 0.1159) or 0.0)
            kw["vae_scale"] = 2 ** (len(kw["vae_channels"]) - 1)
        sched = root / "scheduler" / "scheduler_config.json"
        if sched.exists():
            kw["dynamic_shift"] = bool(json.loads(sched.read_text()).get("use_dynamic_shifting", False))
        else:
            kw["dynamic_shift"] = kw["guidance_embeds"]
        kw["text_len"] = 512 if kw["guidance_embeds"] else 256
        kw["kontext"] = "kontext" in root.name.lower()
        return cls(**kw)


# ---------------------------------------------------------------------------------------------------------------------
# tensor names and shapes (used to draw random weights of the checkpoint's exact layout, and by the tests)
# ---------------------------------------------------------------------------------------------------------------------
def transformer_shapes(c: FluxConfig, blocks: range | None = None) -> dict[str, tuple[int, ...]]:
    H, M = c.hidden, int(c.hidden * c.mlp_ratio)
    s: dict[str, tuple[int, ...]] = {}

    def lin(name: str, o: int, i: int) -> None:
        s[name + ".weight"], s[name + ".bias"] = (o, i), (o,)
    lin("x_embedder", H, c.in_channels)
    lin("context_embedder", H, c.text_dim)
    for e, i in (("timestep_embedder", 256), ("text_embedder", c.pooled_dim)) + ((("guidance_embedder", 256),) if c.guidance_embeds else ()):
        lin(f"time_text_embed.{e}.linear_1", H, i)
        lin(f"time_text_embed.{e}.linear_2", H, H)
    lin("norm_out.linear", 2 * H, H)
    lin("proj_out", c.in_channels, H)
    for b in (blocks if blocks is not None else range(c.n_blocks)):
        if b < c.n_joint:
            p = f"transformer_blocks.{b}."
            lin(p + "norm1.linear", 6 * H, H)
            lin(p + "norm1_context.linear", 6 * H, H)
            for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
                lin(p + "attn." + n, H, H)
            for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
                s[p + f"attn.{n}.weight"] = (c.head_dim,)
            for ff in ("ff", "ff_context"):
                lin(p + ff + ".net.0.proj", M, H)
                lin(p + ff + ".net.2", H, M)
        else:
            p = f"single_transformer_blocks.{b - c.n_joint}."
            lin(p + "norm.linear", 3 * H, H)
            lin(p + "proj_mlp", M, H)
            lin(p + "proj_out", H, H + M)
            for n in ("to_q", "to_k", "to_v"):
                lin(p + "attn." + n, H, H)
            for n in ("norm_q", "norm_k"):
                s[p + f"attn.{n}.weight"] = (c.head_dim,)
    return s


def vae_shapes(c: FluxConfig, encoder: bool = True) -> dict[str, tuple[int, ...]]:
    s: dict[str, tuple[int, ...]] = {}
    ch = c.vae_channels

    def conv(name: str, o: int, i: int, k: int = 3) -> None:
        s[name + ".weight"], s[name + ".bias"] = (o, i, k, k), (o,)

    def norm(name: str, n: int) -> None:
        s[name + ".weight"], s[name + ".bias"] = (n,), (n,)

    def resnet(p: str, i: int, o: int) -> None:
        norm(p + "norm1", i), conv(p + "conv1", o, i), norm(p + "norm2", o), conv(p + "conv2", o, o)
        if i != o:
            conv(p + "conv_shortcut", o, i, 1)

    def mid(p: str, n: int) -> None:
        resnet(p + "resnets.0.", n, n), resnet(p + "resnets.1.", n, n)
        norm(p + "attentions.0.group_norm", n)
        for q in ("to_q", "to_k", "to_v", "to_out.0"):
            s[p + f"attentions.0.{q}.weight"], s[p + f"attentions.0.{q}.bias"] = (n, n), (n,)
    top = ch[-1]
    conv("decoder.conv_in", top, c.latent_channels)
    mid("decoder.mid_block.", top)
    prev = top
    for u, o in enumerate(reversed(ch)):
        for r in range(c.vae_layers + 1):
            resnet(f"decoder.up_blocks.{u}.resnets.{r}.", prev, o)
            prev = o
        if u < len(ch) - 1:
            conv(f"decoder.up_blocks.{u}.upsamplers.0.conv", o, o)
    norm("decoder.conv_norm_out", ch[0]), conv("decoder.conv_out", 3, ch[0])
    if encoder:
        conv("encoder.conv_in", ch[0], 3)
        prev = ch[0]
        for d, o in enumerate(ch):
            for r in range(c.vae_layers):
                resnet(f"encoder.down_blocks.{d}.resnets.{r}.", prev, o)
                prev = o
            if d < len(ch) - 1:
                conv(f"encoder.down_blocks.{d}.downsamplers.0.conv", o, o)
        mid("encoder.mid_block.", top)
        norm("encoder.conv_norm_out", top), conv("encoder.conv_out", 2 * c.latent_channels, top)
    return s


def random_weights(shapes: dict[str, tuple[int, ...]], seed: int, device="cpu", dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Weights of the given layout drawn from a seed (benchmarks and tests: the same draws on every rank, per name).
    Drawn on ``device`` directly, so a full-size model never passes through host memory."""
    out = {}
    dev = torch.device(device)
    for name, shape in sorted(shapes.items()):
        g = torch.Generator(device=dev).manual_seed(seed * 1_000_003 + hash_name(name))
        if name.endswith("bias"):
            t = torch.randn(shape, generator=g, device=dev) * 0.02
        elif len(shape) == 1:
            t = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.02
        else:
            t = torch.randn(shape, generator=g, device=dev, dtype=dtype if dev.type == "cuda" else torch.float32) / math.sqrt(math.prod(shape[1:]))
        out[name] = t.to(dtype)
    return out


def hash_name(name: str) -> int:
    h = 0
    for ch in name.encode():
        h = (h * 131 + ch) % 2_147_483_647
    return h


# ---------------------------------------------------------------------------------------------------------------------
# the VAE
# ---------------------------------------------------------------------------------------------------------------------
class FluxVAE:
    """The 16-channel KL autoencoder (convolutional residual stacks with one attention layer at the lowest resolution)."""

    def __init__(self, cfg: FluxConfig, weights: dict[str, torch.Tensor], device, dtype=torch.float32):
        self.c, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items()}

    def _conv(self, x, name, stride=1, padding=1):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], stride=stride, padding=padding)

    def _norm(self, x, name):
        return F.group_norm(x, self.c.vae_groups, self.w[name + ".weight"], self.w[name + ".bias"], 1e-6)

    def _resnet(self, x, p):
        h = self._conv(F.silu(self._norm(x, p + "norm1")), p + "conv1")
        h = self._conv(F.silu(self._norm(h, p + "norm2")), p + "conv2")
        if p + "conv_shortcut.weight" in self.w:
            x = self._conv(x, p + "conv_shortcut", padding=0)
        return x + h

    def _mid(self, x, p):
        x = self._resnet(x, p + "resnets.0.")
        B, C, Hh, Ww = x.shape
        a = p + "attentions.0."
        h = self._norm(x, a + "group_norm").view(B, C, Hh * Ww).transpose(1, 2)
        q, k, v = (F.linear(h, self.w[a + n + ".weight"], self.w[a + n + ".bias"]) for n in ("to_q", "to_k", "to_v"))
        o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        o = F.linear(o, self.w[a + "to_out.0.weight"], self.w[a + "to_out.0.bias"])
        x = x + o.transpose(1, 2).reshape(B, C, Hh, Ww)
        return self._resnet(x, p + "resnets.1.")

    @torch.no_grad()
    def decode(self, lat: torch.Tensor) -> torch.Tensor:
        """``[C, h, w]`` model latents → uint8 ``[8h, 8w, 3]``."""
        c = self.c
        x = (lat.to(self.device, self.dtype) / c.scaling_factor + c.shift_factor)[None]
        x = self._mid(self._conv(x, "decoder.conv_in"), "decoder.mid_block.")
        for u in range(len(c.vae_channels)):
            for r in range(c.vae_layers + 1):
                x = self._resnet(x, f"decoder.up_blocks.{u}.resnets.{r}.")
            if u < len(c.vae_channels) - 1:
                x = self._conv(F.interpolate(x, scale_factor=2.0, mode="nearest"), f"decoder.up_blocks.{u}.upsamplers.0.conv")
        x = self._conv(F.silu(self._norm(x, "decoder.conv_norm_out")), "decoder.conv_out")[0]
        return ((x.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(1, 2, 0)

    @torch.no_grad()
    def encode(self, rgb: torch.Tensor, h: int, w: int) -> torch.Tensor:
        """uint8 ``[H, W, 3]`` → model latents ``[C, h, w]`` (the posterior's mean), the picture resized to ``8h x 8w``."""
        c = self.c
        x = rgb.to(self.device).permute(2, 0, 1).float()[None] / 127.5 - 1.0
        x = F.interpolate(x, size=(h * c.vae_scale, w * c.vae_scale), mode="bilinear", antialias=True).to(self.dtype)
        x = self._conv(x, "encoder.conv_in")
        for d in range(len(c.vae_channels)):
            for r in range(c.vae_layers):
                x = self._resnet(x, f"encoder.down_blocks.{d}.resnets.{r}.")
            if d < len(c.vae_channels) - 1:
                x = self._conv(F.pad(x, (0, 1, 0, 1)), f"encoder.down_blocks.{d}.downsamplers.0.conv", stride=2, padding=0)
        x = self._mid(x, "encoder.mid_block.")
        x = self._conv(F.silu(self._norm(x, "encoder.conv_norm_out")), "encoder.conv_out")[0]
        return ((x[: c.latent_channels] - c.shift_factor) * c.scaling_factor).float()


# ---------------------------------------------------------------------------------------------------------------------
# the denoiser
# ---------------------------------------------------------------------------------------------------------------------
def sinusoid(x: float, device, dim: int = 256) -> torch.Tensor:
    """``[cos | sin]`` of ``1000 x`` over ``dim/2`` geometric frequencies."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=device) / half)
    a = 1000.0 * x * f
    return torch.cat((a.cos(), a.sin()))


def rope_tables(ids: torch.Tensor, axes: tuple[int, ...], theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``ids [S, len(axes)]`` → cos, sin ``[S, sum(axes)]``; every frequency fills an adjacent pair of channels."""
    cos, sin = [], []
    for i, d in enumerate(axes):
        f = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        a = ids[:, i].double()[:, None] * f
        cos.append(a.cos().repeat_interleave(2, 1).float())
        sin.append(a.sin().repeat_interleave(2, 1).float())
    return torch.cat(cos, 1), torch.cat(sin, 1)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [heads, S, D]``: rotate adjacent channel pairs."""
    a, b = x.float().reshape(*x.shape[:-1], -1, 2).unbind(-1)
    rot = torch.stack((-b, a), -1).flatten(-2)
    return (x.float() * cos + rot * sin).to(x.dtype)


class FluxModel:
    """The FLUX.1 denoiser + VAE + text encoders behind the interface of ``dit.Dit``.

    ``text_encoders``: ``(clip tokenizer, clip model, t5 tokenizer, t5 model)`` or ``None`` — then prompts are hashed into
    deterministic pseudo-features of the right shapes (benchmarks and tests without the encoders' 10 GB)."""

    def __init__(self, cfg: FluxConfig, weights: dict[str, torch.Tensor], vae: FluxVAE | None, *, blocks: range | None = None,
                 device="cpu", dtype=torch.float32, text_encoders=None):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.block_range = blocks if blocks is not None else range(cfg.n_blocks)
        self.w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items()}
        self.vae, self.text = vae, text_encoders
        self.guidance_value = cfg.guidance
        # step counts per quality level and the whole-image steps before patches flow (reference: models/flux/config.py)
        self.default_steps = {"low": 10, "medium": 25, "high": 50} if cfg.guidance_embeds else {"low": 1, "medium": 2, "high": 4}
        self.num_sync_steps = 4 if cfg.guidance_embeds else 1
        self.context: torch.Tensor | None = None        # Kontext: packed latents of the reference picture
        self.context_grid: tuple[int, int] = (0, 0)

    # ---- construction ----
    @classmethod
    def random(cls, cfg: FluxConfig, seed: int = 0, blocks: range | None = None, device="cpu", dtype=torch.float32) -> "FluxModel":
        vae = FluxVAE(cfg, random_weights(vae_shapes(cfg), seed + 1, device), device, torch.float32)
        return cls(cfg, random_weights(transformer_shapes(cfg, blocks), seed, device, dtype), vae, blocks=blocks, device=device, dtype=dtype)

    @classmethod
    def from_folder(cls, root: Path, blocks: range | None = None, device="cpu", dtype=torch.bfloat16, text: bool = True,
                    progress=None) -> "FluxModel":
        """Load the stage's share of a checkpoint folder: the global tensors and the blocks in ``blocks``."""
        from ....models.weights import SafetensorsSource
        cfg = FluxConfig.from_folder(root)
        want = transformer_shapes(cfg, blocks)
        src = SafetensorsSource(root / "transformer", device="cpu", dtype=dtype)
        w = {}
        for i, name in enumerate(want):
            t = src.get(name, None)
            if tuple(t.shape) != want[name]:
                raise ValueError(f"{name}: checkpoint has {tuple(t.shape)}, the configuration says {want[name]}")
            w[name] = t
            if progress is not None and i % 64 == 0:
                progress(i, len(want))
        vsrc = SafetensorsSource(root / "vae", device="cpu", dtype=torch.float32)
        have = set(vsrc.names())
        vae = FluxVAE(cfg, {n: vsrc.get(n, None) for n in vae_shapes(cfg) if n in have}, device, torch.float32)
        enc = None
        if text and (root / "text_encoder").exists() and (root / "text_encoder_2").exists():
            from transformers import AutoTokenizer, CLIPTextModel, T5EncoderModel
            enc = (AutoTokenizer.from_pretrained(root / "tokenizer"), CLIPTextModel.from_pretrained(root / "text_encoder", dtype=dtype).to(device).eval(),
                   AutoTokenizer.from_pretrained(root / "tokenizer_2"), T5EncoderModel.from_pretrained(root / "text_encoder_2", dtype=dtype).to(device).eval())
        return cls(cfg, w, vae, blocks=blocks, device=device, dtype=dtype, text_encoders=enc)

    # ---- small helpers ----
    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.linear(x, self.w[name + ".weight"], self.w[name + ".bias"])

    def _heads(self, x: torch.Tensor) -> torch.Tensor:
        return x.view(x.shape[0], self.cfg.n_heads, self.cfg.head_dim).transpose(0, 1)

    def _rms(self, x: torch.Tensor, name: str) -> torch.Tensor:
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
        return (y * self.w[name + ".weight"].float()).to(x.dtype)

    def _ln(self, x: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x, (self.cfg.hidden,), eps=1e-6)

    # ---- conditioning ----
    @torch.no_grad()
    def encode_text(self, prompt: str) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        if self.text is None:
            g = torch.Generator().manual_seed(hash_name(prompt) + 1)
            n = max(1, min(c.text_len, len(prompt.split()) + 1))
            feats = torch.zeros(c.text_len, c.text_dim)
            feats[:n] = torch.randn(n, c.text_dim, generator=g) * 0.1
            return (self._lin(feats.to(self.device, self.dtype), "context_embedder") if "context_embedder.weight" in self.w else
                    feats.to(self.device, self.dtype)), (torch.randn(c.pooled_dim, generator=g) * 0.5).to(self.device, self.dtype)
        tok1, clip, tok2, t5 = self.text
        a = tok1([prompt], padding="max_length", max_length=tok1.model_max_length, truncation=True, return_tensors="pt")
        pooled = clip(a.input_ids.to(self.device)).pooler_output[0]
        b = tok2([prompt], padding="max_length", max_length=c.text_len, truncation=True, return_tensors="pt")
        feats = t5(b.input_ids.to(self.device)).last_hidden_state[0]
        return self._lin(feats.to(self.dtype), "context_embedder"), pooled.to(self.dtype)

    def time_vec(self, t: float, pooled: torch.Tensor) -> torch.Tensor:
        p = "time_text_embed."
        emb = lambda x, n: self._lin(F.silu(self._lin(x.to(self.dtype), p + n + ".linear_1")), p + n + ".linear_2")   # noqa: E731
        v = emb(sinusoid(t, self.device), "timestep_embedder") + emb(pooled, "text_embedder")
        if self.cfg.guidance_embeds:
            v = v + emb(sinusoid(self.guidance_value, self.device), "guidance_embedder")
        return v

    def schedule(self, steps: int, n_tokens: int) -> list[float]:
        """Noise levels from 1 down to 0; with dynamic shifting they move toward the noisy end as the token count grows."""
        s = [1.0 - i * (1.0 - 1.0 / steps) / max(1, steps - 1) for i in range(steps)]
        if self.cfg.dynamic_shift:
            m = (1.15 - 0.5) / (4096 - 256)
            mu = n_tokens * m + (0.5 - m * 256)
            s = [math.exp(mu) / (math.exp(mu) + (1.0 / x - 1.0)) for x in s]
        return s + [0.0]

    # ---- latents <-> tokens <-> pixels ----
    def grid(self, height: int, width: int) -> tuple[int, int]:
        cell = self.cfg.vae_scale * self.cfg.patch
        return max(1, height // cell), max(1, width // cell)

    def patchify(self, lat: torch.Tensor) -> torch.Tensor:
        C, p = self.cfg.latent_channels, self.cfg.patch
        gh, gw = lat.shape[1] // p, lat.shape[2] // p
        return lat.view(C, gh, p, gw, p).permute(1, 3, 0, 2, 4).reshape(gh * gw, C * p * p)

    def unpatchify(self, tok: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        C, p = self.cfg.latent_channels, self.cfg.patch
        return tok.view(gh, gw, C, p, p).permute(2, 0, 3, 1, 4).reshape(C, gh * p, gw * p)

    def decode(self, lat: torch.Tensor) -> torch.Tensor:
        return self.vae.decode(lat)

    def encode_image(self, rgb: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        return self.vae.encode(rgb, gh * self.cfg.patch, gw * self.cfg.patch).to(self.device)

    def set_context(self, rgb: torch.Tensor | None, gh: int = 0, gw: int = 0) -> None:
        """Kontext: the reference picture's latents become extra image tokens (frame index 1) that every block sees."""
        if rgb is None:
            self.context, self.context_grid = None, (0, 0)
            return
        lat = self.encode_image(rgb, gh, gw)
        self.context, self.context_grid = self._lin(self.patchify(lat).to(self.dtype), "x_embedder"), (gh, gw)

    # ---- the denoiser ----
    def _ids(self, gh: int, gw: int, frame: int = 0) -> torch.Tensor:
        ys, xs = torch.meshgrid(torch.arange(gh, device=self.device), torch.arange(gw, device=self.device), indexing="ij")
        return torch.stack((torch.full_like(ys, frame), ys, xs), -1).reshape(gh * gw, 3)

    def _rope(self, n_txt: int, grid: tuple[int, int], rows: slice | None):
        key = (n_txt, grid, None if rows is None else (rows.start, rows.stop), self.context_grid if self.context is not None else None)
        if getattr(self, "_rope_key", None) == key:
            return self._rope_val
        self._rope_key, self._rope_val = key, self._rope_tables(n_txt, grid, rows)
        return self._rope_val

    def _rope_tables(self, n_txt: int, grid: tuple[int, int], rows: slice | None):
        ids = self._ids(*grid)
        if rows is not None:
            ids = ids[rows]
        if self.context is not None:
            ids = torch.cat((ids, self._ids(*self.context_grid, frame=1)))
        ids = torch.cat((torch.zeros(n_txt, 3, dtype=ids.dtype, device=self.device), ids))
        cos, sin = rope_tables(ids, self.cfg.axes_dims, self.cfg.theta)
        return cos, sin

    def embed_tokens(self, lat: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        return self._lin(self.patchify(lat).to(self.dtype), "x_embedder")

    def _attend(self, qt, kt, vt, qi, ki, vi, rope, cache, rows):
        """Joint attention of the text and image streams.  ``cache`` holds the image keys / values (after the rotation) of the
        previous whole-image step; with ``rows`` only those rows are fresh."""
        cos, sin = rope
        nt = qt.shape[1]
        qt, kt = rope_apply(qt, cos[:nt], sin[:nt]), rope_apply(kt, cos[:nt], sin[:nt])
        qi, ki = rope_apply(qi, cos[nt:], sin[nt:]), rope_apply(ki, cos[nt:], sin[nt:])
        if cache is not None:
            if rows is None:
                cache[0], cache[1] = ki.clone(), vi.clone()
            else:
                n_ctx = 0 if self.context is None else self.context.shape[0]
                n_new = ki.shape[1] - n_ctx
                cache[0][:, rows], cache[1][:, rows] = ki[:, :n_new], vi[:, :n_new]
                if n_ctx:
                    full = cache[0].shape[1] - n_ctx
                    cache[0][:, full:], cache[1][:, full:] = ki[:, n_new:], vi[:, n_new:]
                ki, vi = cache[0], cache[1]
        k, v = torch.cat((kt, ki), 1), torch.cat((vt, vi), 1)
        flat = lambda a: a.transpose(0, 1).reshape(a.shape[1], self.cfg.hidden)     # noqa: E731
        q = torch.cat((qt, qi), 1)                                  # one call over both streams (a 4-D call picks the fused kernel)
        o = flat(self._sdpa(q[None], k[None], v[None])[0])
        return o[:nt], o[nt:]

    def _sdpa(self, q, k, v):
        """Attention through the library's fused kernels; ``EXO_FLUX_SDPA=cudnn|flash|efficient|math`` pins one."""
        import os
        pin = os.environ.get("EXO_FLUX_SDPA", "")
        if not pin or q.device.type != "cuda":
            return F.scaled_dot_product_attention(q, k, v)
        from torch.nn.attention import SDPBackend, sdpa_kernel
        which = {"cudnn": SDPBackend.CUDNN_ATTENTION, "flash": SDPBackend.FLASH_ATTENTION, "efficient": SDPBackend.EFFICIENT_ATTENTION,
                 "math": SDPBackend.MATH}[pin]
        with sdpa_kernel([which]):
            return F.scaled_dot_product_attention(q, k, v)

    def _joint(self, b: int, txt, img, vec, rope, cache, rows):
        p = f"transformer_blocks.{b}."
        sv = F.silu(vec)
        mi, mt = self._lin(sv, p + "norm1.linear").chunk(6), self._lin(sv, p + "norm1_context.linear").chunk(6)
        hi, ht = self._ln(img) * (1 + mi[1]) + mi[0], self._ln(txt) * (1 + mt[1]) + mt[0]
        qi, ki, vi = (self._heads(self._lin(hi, p + "attn." + n)) for n in ("to_q", "to_k", "to_v"))
        qt, kt, vt = (self._heads(self._lin(ht, p + "attn." + n)) for n in ("add_q_proj", "add_k_proj", "add_v_proj"))
        qi, ki = self._rms(qi, p + "attn.norm_q"), self._rms(ki, p + "attn.norm_k")
        qt, kt = self._rms(qt, p + "attn.norm_added_q"), self._rms(kt, p + "attn.norm_added_k")
        at, ai = self._attend(qt, kt, vt, qi, ki, vi, rope, cache, rows)
        img = img + mi[2] * self._lin(ai, p + "attn.to_out.0")
        txt = txt + mt[2] * self._lin(at, p + "attn.to_add_out")
        ff = lambda x, n: self._lin(F.gelu(self._lin(x, p + n + ".net.0.proj"), approximate="tanh"), p + n + ".net.2")   # noqa: E731
        img = img + mi[5] * ff(self._ln(img) * (1 + mi[4]) + mi[3], "ff")
        txt = txt + mt[5] * ff(self._ln(txt) * (1 + mt[4]) + mt[3], "ff_context")
        return txt, img

    def _single(self, b: int, txt, img, vec, rope, cache, rows):
        p = f"single_transformer_blocks.{b - self.cfg.n_joint}."
        shift, scale, gate = self._lin(F.silu(vec), p + "norm.linear").chunk(3)
        nt = txt.shape[0]
        x = torch.cat((txt, img))
        h = self._ln(x) * (1 + scale) + shift
        q, k, v = (self._heads(self._lin(h, p + "attn." + n)) for n in ("to_q", "to_k", "to_v"))
        q, k = self._rms(q, p + "attn.norm_q"), self._rms(k, p + "attn.norm_k")
        at, ai = self._attend(q[:, :nt], k[:, :nt], v[:, :nt], q[:, nt:], k[:, nt:], v[:, nt:], rope, cache, rows)
        mlp = F.gelu(self._lin(h, p + "proj_mlp"), approximate="tanh")
        x = x + gate * self._lin(torch.cat((torch.cat((at, ai)), mlp), -1), p + "proj_out")
        return x[:nt], x[nt:]

    def run_blocks(self, txt, img, vec, caches=None, rows: slice | None = None, grid: tuple[int, int] | None = None):
        """The stage's blocks over the text stream and the image tokens (all of them, or the fresh ``rows`` of a patch step).
        ``grid``: the whole image's token grid (positions); derived from a square image when absent."""
        if grid is None:
            side = int(math.isqrt(img.shape[0]))
            grid = (side, img.shape[0] // side)
        n_img = img.shape[0]
        if self.context is not None:
            img = torch.cat((img, self.context))
        rope = self._rope(txt.shape[0], grid, rows)
        for b in self.block_range:
            step = self._joint if b < self.cfg.n_joint else self._single
            txt, img = step(b, txt, img, vec, rope, None if caches is None else caches[b], rows)
        return txt, img[:n_img]

    def head_tokens(self, img: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        scale, shift = self._lin(F.silu(vec), "norm_out.linear").chunk(2)
        return self._lin(self._ln(img) * (1 + scale) + shift, "proj_out").float()

    def head(self, img: torch.Tensor, gh: int, gw: int, vec: torch.Tensor | None = None) -> torch.Tensor:
        return self.unpatchify(self.head_tokens(img, vec), gh, gw)

    @torch.no_grad()
    def velocity(self, lat: torch.Tensor, t: float, txt: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        gh, gw = lat.shape[1] // self.cfg.patch, lat.shape[2] // self.cfg.patch
        vec = self.time_vec(t, pooled)
        _, img = self.run_blocks(txt, self.embed_tokens(lat, gh, gw), vec, grid=(gh, gw))
        return self.head(img, gh, gw, vec)
