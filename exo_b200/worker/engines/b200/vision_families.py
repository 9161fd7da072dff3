"""Image processors and towers of the vision-language families, and the tensor names they load.

The reference drives three processor families through ``mlx_vlm`` / ``transformers`` classes
(``src/exo/worker/engines/mlx/vision.py:487-624``): the Qwen-VL grid processor (``image_grid_thw``, tokens =
``t*h*w / merge²``), the Kimi-VL native-resolution processor (``image_grid_hws``, a patch budget, 2x2 merge) and the
fixed-budget Gemma processor (every image becomes the same number of soft tokens).  Here each is a small class that
turns PIL images into the tower's input and the per-image token count, written from the published algorithms, plus the
Qwen2-VL tower itself (fused qkv, 2-D rotary positions, per-image attention, LayerNorm + MLP patch merger) in plain
PyTorch on the engine's device, loading the checkpoint's ``visual.*`` tensors
(``src/exo/worker/engines/mlx/vision.py:277-485`` does the loading and key remapping for its towers).

``family_for(config.json)`` picks the processor; ``VisionProcessor`` (``vision.py``) owns the feature cache and the
splice into the prompt whichever family produced the rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn.functional as F

CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
HALF = (0.5, 0.5, 0.5)


def _to_tensor(im, size_wh: tuple[int, int] | None, resample, mean, std) -> torch.Tensor:
    """PIL image → normalised ``[3, H, W]`` fp32 (optionally resized first)."""
    import numpy as np
    im = im.convert("RGB")
    if size_wh is not None and im.size != size_wh:
        im = im.resize(size_wh, resample)
    x = torch.from_numpy(np.asarray(im, dtype=np.uint8).copy()).permute(2, 0, 1).float() * (1.0 / 255.0)
    return (x - torch.tensor(mean)[:, None, None]) / torch.tensor(std)[:, None, None]


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Target size of the Qwen-VL processors: both sides multiples of ``factor`` (patch x merge), the area inside
    ``[min_pixels, max_pixels]``, the aspect ratio kept as far as the rounding allows."""
    if max(h, w) / max(1, min(h, w)) > 200:
        raise ValueError(f"aspect ratio {max(h, w) / min(h, w):.1f} is beyond what the processor takes (200)")
    hb, wb = max(factor, round(h / factor) * factor), max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


@dataclass
class QwenVLProcessor:
    """Qwen2-VL / Qwen2.5-VL / Qwen3-VL: resize to a grid of ``patch``-sized patches, duplicate the frame to fill the
    temporal patch, and lay the patches out so that the ``merge x merge`` patches of one output token are adjacent."""
    patch: int = 14
    merge: int = 2
    temporal: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 28 * 28 * 1280
    mean: tuple[float, ...] = CLIP_MEAN
    std: tuple[float, ...] = CLIP_STD

    @classmethod
    def from_config(cls, pre: dict[str, Any]) -> "QwenVLProcessor":
        size = pre.get("size") or {}
        return cls(patch=pre.get("patch_size", 14), merge=pre.get("merge_size", 2), temporal=pre.get("temporal_patch_size", 2),
                   min_pixels=pre.get("min_pixels") or size.get("shortest_edge", 56 * 56),
                   max_pixels=pre.get("max_pixels") or size.get("longest_edge", 28 * 28 * 1280),
                   mean=tuple(pre.get("image_mean", CLIP_MEAN)), std=tuple(pre.get("image_std", CLIP_STD)))

    def __call__(self, images: list) -> tuple[torch.Tensor, torch.Tensor, list[int]]:
        """→ ``(patches [sum t*h*w, 3*temporal*patch²], grid_thw [n, 3], tokens per image)``."""
        from PIL import Image
        p, m, tp = self.patch, self.merge, self.temporal
        rows, grids = [], []
        for im in images:
            w0, h0 = im.size
            h, w = smart_resize(h0, w0, p * m, self.min_pixels, self.max_pixels)
            x = _to_tensor(im, (w, h), Image.BICUBIC, self.mean, self.std)
            gh, gw = h // p, w // p
            x = x[None].expand(tp, -1, -1, -1)                                   # one still image fills the temporal patch
            x = x.reshape(1, tp, 3, gh // m, m, p, gw // m, m, p)
            x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                             # t, h/m, w/m, m, m, C, tp, p, p
            rows.append(x.reshape(gh * gw, 3 * tp * p * p))
            grids.append((1, gh, gw))
        grid = torch.tensor(grids, dtype=torch.long)
        return torch.cat(rows), grid, [t * h * w // (m * m) for t, h, w in grids]


@dataclass
class KimiVLProcessor:
    """Kimi-VL (MoonViT): native resolution up to a patch budget, then padding to whole ``merge``-blocks.

    An image with more than ``in_token_limit`` patches is shrunk (aspect kept) until it fits; the result is padded with
    zeros on the right / bottom to a multiple of ``patch x merge`` and cut into ``[N, 3, patch, patch]`` patches in
    row-major order; ``image_grid_hws`` carries the patch grid of each image."""
    patch: int = 14
    merge: tuple[int, int] = (2, 2)
    in_token_limit: int = 4096
    mean: tuple[float, ...] = HALF
    std: tuple[float, ...] = HALF

    @classmethod
    def from_config(cls, pre: dict[str, Any]) -> "KimiVLProcessor":
        return cls(patch=pre.get("patch_size", 14), merge=tuple(pre.get("merge_kernel_size", (2, 2))),
                   in_token_limit=pre.get("in_token_limit", 4096), mean=tuple(pre.get("image_mean", HALF)),
                   std=tuple(pre.get("image_std", HALF)))

    def target(self, w: int, h: int) -> tuple[int, int, int, int]:
        """``(resize_w, resize_h, padded_w, padded_h)``."""
        p = self.patch
        if (w // p) * (h // p) > self.in_token_limit:
            s = math.sqrt(self.in_token_limit / ((w / p) * (h / p)))
            w, h = max(p, int(w * s)), max(p, int(h * s))
        cw, ch = p * self.merge[1], p * self.merge[0]
        return w, h, -(-w // cw) * cw, -(-h // ch) * ch

    def __call__(self, images: list) -> tuple[torch.Tensor, torch.Tensor, list[int]]:
        from PIL import Image
        p = self.patch
        rows, grids = [], []
        for im in images:
            w, h, pw, ph = self.target(*im.size)
            x = _to_tensor(im, (w, h), Image.BICUBIC, self.mean, self.std)
            x = F.pad(x, (0, pw - w, 0, ph - h))
            gh, gw = ph // p, pw // p
            rows.append(x.reshape(3, gh, p, gw, p).permute(1, 3, 0, 2, 4).reshape(gh * gw, 3, p, p))
            grids.append((gh, gw))
        mh, mw = self.merge
        return torch.cat(rows), torch.tensor(grids, dtype=torch.long), [gh * gw // (mh * mw) for gh, gw in grids]


@dataclass
class GemmaProcessor:
    """Gemma-3: every image is resized to one square and becomes ``tokens_per_image`` soft tokens (the tower's
    ``size/patch`` squared patches are average-pooled down to that many by the projector)."""
    size: int = 896
    tokens_per_image: int = 256
    mean: tuple[float, ...] = HALF
    std: tuple[float, ...] = HALF

    @classmethod
    def from_config(cls, pre: dict[str, Any], cfg: dict[str, Any] | None = None) -> "GemmaProcessor":
        size = pre.get("size") or {}
        return cls(size=size.get("height", 896), tokens_per_image=(cfg or {}).get("mm_tokens_per_image", 256),
                   mean=tuple(pre.get("image_mean", HALF)), std=tuple(pre.get("image_std", HALF)))

    def __call__(self, images: list) -> tuple[torch.Tensor, None, list[int]]:
        from PIL import Image
        x = torch.stack([_to_tensor(im, (self.size, self.size), Image.BILINEAR, self.mean, self.std) for im in images])
        return x, None, [self.tokens_per_image] * len(images)

    @staticmethod
    def pool(patch_rows: torch.Tensor, tokens: int) -> torch.Tensor:
        """``[side², C]`` tower outputs → ``[tokens, C]`` by average pooling over the patch grid (the projector's first step)."""
        n, c = patch_rows.shape
        side, out = math.isqrt(n), math.isqrt(tokens)
        g = patch_rows.t().reshape(1, c, side, side)
        return F.avg_pool2d(g, side // out, side // out).reshape(c, out * out).t()


def family_for(config: dict[str, Any], preprocessor: dict[str, Any] | None = None):
    """The image processor of a checkpoint, from its ``config.json`` (``model_type``) and ``preprocessor_config.json``;
    ``None`` for a text-only model."""
    mt = str(config.get("model_type", "")).lower()
    pre = preprocessor or {}
    if mt in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "qwen3_5", "qwen3_5_moe"):
        proc = QwenVLProcessor.from_config(pre)
        vc = config.get("vision_config") or {}
        if "patch_size" in vc and "patch_size" not in pre:
            proc.patch = vc["patch_size"]
        if mt.startswith("qwen3") and "image_mean" not in pre:
            proc.mean = proc.std = HALF
        return proc
    if mt in ("kimi_vl", "kimi_k25", "kimi_k2_5"):
        return KimiVLProcessor.from_config(pre)
    if mt == "gemma4":
        return Gemma4Processor.from_config(pre, config)
    if mt in ("gemma3", "gemma3n"):
        return GemmaProcessor.from_config(pre, config)
    return None


# ---------------------------------------------------------------------------------------------------------------------
# Qwen2-VL tower
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class QwenVLTowerConfig:
    depth: int = 32
    embed_dim: int = 1280
    heads: int = 16
    mlp_ratio: float = 4.0
    patch: int = 14
    merge: int = 2
    temporal: int = 2
    out_hidden: int = 3584
    variant: str = "qwen2"          # "qwen3": Qwen3-VL / Qwen3.5 / Qwen3.6 (learned position table, tanh-GELU MLP, other tensor names)
    mlp_dim: int = 0                # qwen3: the MLP's width (qwen2 derives it from mlp_ratio)
    n_pos: int = 2304               # qwen3: entries of the learned position table (a square grid)
    act: str = "gelu_pytorch_tanh"  # qwen3: MLP activation

    @classmethod
    def from_config(cls, vc: dict[str, Any]) -> "QwenVLTowerConfig":
        if "out_hidden_size" in vc:                                             # Qwen3-VL and later
            return cls(depth=vc.get("depth", 27), embed_dim=vc.get("hidden_size", 1152), heads=vc.get("num_heads", 16),
                       patch=vc.get("patch_size", 16), merge=vc.get("spatial_merge_size", 2), temporal=vc.get("temporal_patch_size", 2),
                       out_hidden=vc["out_hidden_size"], variant="qwen3", mlp_dim=vc.get("intermediate_size", 4304),
                       n_pos=vc.get("num_position_embeddings", 2304), act=vc.get("hidden_act", "gelu_pytorch_tanh"))
        return cls(depth=vc.get("depth", 32), embed_dim=vc.get("embed_dim", 1280), heads=vc.get("num_heads", 16),
                   mlp_ratio=vc.get("mlp_ratio", 4.0), patch=vc.get("patch_size", 14), merge=vc.get("spatial_merge_size", 2),
                   temporal=vc.get("temporal_patch_size", 2), out_hidden=vc.get("hidden_size", 3584))


def _rot_half(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, -1)
    return torch.cat((-b, a), -1)


@dataclass
class QwenVLTower:
    """The Qwen2-VL vision transformer over ``QwenVLProcessor`` patches.

    ``weights`` maps the checkpoint's names with the ``visual.`` prefix removed (``patch_embed.proj.weight`` as the 5-D
    convolution kernel, ``blocks.N.{norm1,norm2,attn.qkv,attn.proj,mlp.fc1,mlp.fc2}``, ``merger.{ln_q,mlp.0,mlp.2}``).
    Positions are 2-D rotary (row and column halves of each head's first half), attention is full within an image and
    never crosses images, the MLP activation is ``x * sigmoid(1.702 x)``, and the merger normalises every patch, joins
    the ``merge²`` neighbours and maps them to the decoder's hidden size.

    ``variant == "qwen3"`` (Qwen3-VL, Qwen3.5, Qwen3.6): the patch projection has a bias, a learned ``pos_embed`` table over a
    square grid is interpolated bilinearly to the image's patch grid and added, the MLP is ``linear_fc1`` / ``linear_fc2``
    with the configured activation, and the merger's tensors are ``merger.{norm,linear_fc1,linear_fc2}``.  The extra
    mergers that feed intermediate features to the first decoder layers of Qwen3-VL are not run: the tower returns the
    input embeddings only."""
    cfg: QwenVLTowerConfig
    weights: dict[str, torch.Tensor]
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        self.w = {k: v.to(device=self.device, dtype=self.dtype) for k, v in self.weights.items()}
        k = self.w["patch_embed.proj.weight"]
        if k.dim() == 5 and k.shape[1] != 3 and k.shape[-1] == 3:               # channels-last kernel (MLX checkpoints)
            k = k.permute(0, 4, 1, 2, 3)
        self.w["patch_embed.proj.weight"] = k.reshape(self.cfg.embed_dim, -1)

    @classmethod
    def from_source(cls, src, cfg: QwenVLTowerConfig, device, dtype, prefix: str = "visual.") -> "QwenVLTower":
        """Read the tower's tensors from a checkpoint reader (``models.weights.SafetensorsSource``)."""
        names = [n for n in src.names() if n.startswith(prefix)]
        if not names:
            raise KeyError(f"checkpoint has no {prefix}* tensors")
        return cls(cfg, {n[len(prefix):]: src.get(n, None) for n in names}, torch.device(device), dtype)

    def _position_table(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """The learned position table resampled to every image's grid (bilinear, corners aligned), in patch order."""
        c, tab = self.cfg, self.w["pos_embed.weight"]
        side, m = int(c.n_pos ** 0.5), c.merge
        out = []
        for t, h, w in grid_thw.tolist():
            ys, xs = torch.linspace(0, side - 1, h, device=self.device), torch.linspace(0, side - 1, w, device=self.device)
            y0, x0 = ys.int(), xs.int()
            y1, x1 = (y0 + 1).clip(max=side - 1), (x0 + 1).clip(max=side - 1)
            dy, dx = (ys - y0).to(tab.dtype)[:, None, None], (xs - x0).to(tab.dtype)[None, :, None]
            g = lambda a, b: tab[(a.long()[:, None] * side + b.long()[None, :])]          # noqa: E731   [h, w, E]
            e = g(y0, x0) * (1 - dy) * (1 - dx) + g(y0, x1) * (1 - dy) * dx + g(y1, x0) * dy * (1 - dx) + g(y1, x1) * dy * dx
            e = e.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out)

    def _rotary(self, grid_thw: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        hd = c.embed_dim // c.heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=self.device) / (hd // 2)))
        ids = []
        for t, h, w in grid_thw.tolist():
            m = c.merge
            hp = torch.arange(h, device=self.device)[:, None].expand(h, w)
            wp = torch.arange(w, device=self.device)[None, :].expand(h, w)
            order = lambda g: g.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)   # noqa: E731
            ids.append(torch.stack((order(hp), order(wp)), -1).repeat(t, 1))
        pos = torch.cat(ids).float()                                            # [N, 2]
        ang = torch.cat((pos[:, :1] * inv, pos[:, 1:] * inv), -1)               # [N, hd/2]
        ang = torch.cat((ang, ang), -1)                                         # [N, hd]
        return ang.cos()[:, None, :], ang.sin()[:, None, :]

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        E, H = c.embed_dim, c.heads
        hd = E // H
        x = patches.to(device=self.device, dtype=self.dtype) @ w["patch_embed.proj.weight"].t()
        q3 = c.variant == "qwen3"
        if q3:
            x = x + w["patch_embed.proj.bias"] + self._position_table(grid_thw)
        fc1, fc2 = ("mlp.linear_fc1", "mlp.linear_fc2") if q3 else ("mlp.fc1", "mlp.fc2")
        cos, sin = self._rotary(grid_thw)
        cos, sin = cos.to(self.dtype), sin.to(self.dtype)
        spans = [h * w for t, h, w in grid_thw.tolist() for _ in range(t)] if q3 else \
            (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).tolist()
        for i in range(c.depth):
            b = f"blocks.{i}."
            y = F.layer_norm(x, (E,), w[b + "norm1.weight"], w[b + "norm1.bias"], 1e-6)
            q, k, v = (y @ w[b + "attn.qkv.weight"].t() + w[b + "attn.qkv.bias"]).view(-1, 3, H, hd).unbind(1)
            q, k = q * cos + _rot_half(q) * sin, k * cos + _rot_half(k) * sin
            outs, o = [], 0
            for n in spans:                                                     # attention never crosses images
                qs, ks, vs = (t[o:o + n].transpose(0, 1)[None] for t in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qs, ks, vs)[0].transpose(0, 1).reshape(n, E))
                o += n
            x = x + torch.cat(outs) @ w[b + "attn.proj.weight"].t() + w[b + "attn.proj.bias"]
            y = F.layer_norm(x, (E,), w[b + "norm2.weight"], w[b + "norm2.bias"], 1e-6)
            y = y @ w[b + fc1 + ".weight"].t() + w[b + fc1 + ".bias"]
            if not q3:
                y = y * torch.sigmoid(1.702 * y)
            elif c.act in ("gelu_pytorch_tanh", "gelu_tanh"):
                y = F.gelu(y, approximate="tanh")
            elif c.act == "gelu":
                y = F.gelu(y)
            elif c.act == "silu":
                y = F.silu(y)
            else:
                raise ValueError(f"vision MLP activation {c.act!r}")
            x = x + y @ w[b + fc2 + ".weight"].t() + w[b + fc2 + ".bias"]
        if q3:
            x = F.layer_norm(x, (E,), w["merger.norm.weight"], w["merger.norm.bias"], 1e-6).view(-1, c.merge * c.merge * E)
            x = F.gelu(x @ w["merger.linear_fc1.weight"].t() + w["merger.linear_fc1.bias"])
            return x @ w["merger.linear_fc2.weight"].t() + w["merger.linear_fc2.bias"]
        x = F.layer_norm(x, (E,), w["merger.ln_q.weight"], w["merger.ln_q.bias"], 1e-6).view(-1, c.merge * c.merge * E)
        x = F.gelu(x @ w["merger.mlp.0.weight"].t() + w["merger.mlp.0.bias"])
        return x @ w["merger.mlp.2.weight"].t() + w["merger.mlp.2.bias"]


# ---------------------------------------------------------------------------------------------------------------------
# Gemma-4: aspect-preserving patches with (x, y) positions, its own vision transformer
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Gemma4Processor:
    """Every image is resized (bicubic, aspect ratio kept) to the largest size whose sides are multiples of
    ``pool * patch`` and that gives at most ``max_soft_tokens * pool²`` patches; pixels stay in ``[0, 1]`` (the tower
    rescales).  Returns per image its patch rows ``[n, 3 * patch²]`` (patch pixels in (row, column, channel) order), the
    patches' integer ``(x, y)`` positions and the number of soft tokens (``n / pool²``)."""
    patch: int = 16
    max_soft_tokens: int = 280
    pool: int = 3

    @classmethod
    def from_config(cls, pre: dict[str, Any], cfg: dict[str, Any] | None = None) -> "Gemma4Processor":
        vc = (cfg or {}).get("vision_config") or {}
        return cls(patch=pre.get("patch_size", vc.get("patch_size", 16)), max_soft_tokens=pre.get("max_soft_tokens", 280),
                   pool=pre.get("pooling_kernel_size", vc.get("pooling_kernel_size", 3)))

    def target(self, h: int, w: int) -> tuple[int, int]:
        max_patches = self.max_soft_tokens * self.pool ** 2
        factor = math.sqrt(max_patches * self.patch ** 2 / (h * w))
        side = self.pool * self.patch
        th, tw = int(math.floor(factor * h / side)) * side, int(math.floor(factor * w / side)) * side
        longest = (max_patches // self.pool ** 2) * side
        if th == 0 and tw == 0:
            raise ValueError(f"image {h}x{w} cannot be resized to a multiple of {side}")
        if th == 0:
            th, tw = side, min(int(math.floor(w / h)) * side, longest)
        elif tw == 0:
            tw, th = side, min(int(math.floor(h / w)) * side, longest)
        return th, tw

    def __call__(self, images: list) -> tuple[list[torch.Tensor], list[torch.Tensor], list[int]]:
        import torchvision.transforms.v2.functional as TF
        patches, positions, counts = [], [], []
        for im in images:
            x = TF.pil_to_tensor(im.convert("RGB"))                                    # [3, H, W] uint8
            th, tw = self.target(x.shape[-2], x.shape[-1])
            if (th, tw) != tuple(x.shape[-2:]):
                x = TF.resize(x, [th, tw], interpolation=TF.InterpolationMode.BICUBIC, antialias=True)
            x = x.float() / 255.0
            ph, pw = th // self.patch, tw // self.patch
            rows = x.reshape(3, ph, self.patch, pw, self.patch).permute(1, 3, 2, 4, 0).reshape(ph * pw, -1)
            xs, ys = torch.meshgrid(torch.arange(pw), torch.arange(ph), indexing="xy")
            patches.append(rows)
            positions.append(torch.stack((xs, ys), -1).reshape(ph * pw, 2))
            counts.append(ph * pw // self.pool ** 2)
        return patches, positions, counts


@dataclass
class Gemma4VisionConfig:
    hidden: int = 768
    ffn: int = 3072
    layers: int = 16
    heads: int = 12
    kv_heads: int = 12
    head_dim: int = 64
    eps: float = 1e-6
    theta: float = 100.0
    patch: int = 16
    pool: int = 3
    table: int = 10240
    clipped: bool = False
    standardize: bool = False

    @classmethod
    def from_config(cls, vc: dict[str, Any]) -> "Gemma4VisionConfig":
        rp = vc.get("rope_parameters") or {}
        return cls(hidden=vc.get("hidden_size", 768), ffn=vc.get("intermediate_size", 3072), layers=vc.get("num_hidden_layers", 16),
                   heads=vc.get("num_attention_heads", 12), kv_heads=vc.get("num_key_value_heads", 12), head_dim=vc.get("head_dim", 64),
                   eps=vc.get("rms_norm_eps", 1e-6), theta=rp.get("rope_theta", 100.0), patch=vc.get("patch_size", 16),
                   pool=vc.get("pooling_kernel_size", 3), table=vc.get("position_embedding_size", 10240),
                   clipped=bool(vc.get("use_clipped_linears", False)), standardize=bool(vc.get("standardize", False)))


@dataclass
class Gemma4VisionTower:
    """Gemma-4's vision encoder and its projection into the decoder's hidden size, one image at a time (no padding
    patches: an image's own patches are all the encoder sees, which is what the library's padding mask amounts to).

    ``weights``: the checkpoint's tensors with the ``model.vision_tower.`` prefix removed, plus the embedder's
    ``embed_vision.embedding_projection.weight``.  Patch pixels are mapped to ``[-1, 1]``, projected, and given learned
    (x, y) position embeddings; every layer has norms on both sides of attention and MLP, q / k normalised with a weight
    and v without one, 2-D rotary positions (the first half of each head turns with x, the second with y, both with the
    frequencies of a quarter-width head), softmax scale 1, GeGLU; the pooler averages ``pool x pool`` neighbours and
    scales by ``sqrt(hidden)``; the embedder normalises (no weight) and projects."""
    cfg: Gemma4VisionConfig
    weights: dict[str, torch.Tensor]
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        self.w = {k: v.to(device=self.device, dtype=self.dtype if v.is_floating_point() else v.dtype) for k, v in self.weights.items()}

    @classmethod
    def from_source(cls, src, cfg: Gemma4VisionConfig, device, dtype, prefix: str = "model.vision_tower.",
                    embedder: str = "model.embed_vision.") -> "Gemma4VisionTower":
        names = [n for n in src.names() if n.startswith(prefix)]
        if not names:
            raise KeyError(f"checkpoint has no {prefix}* tensors")
        w = {n[len(prefix):]: src.get(n, None) for n in names}
        w.update({"embed_vision." + n[len(embedder):]: src.get(n, None) for n in src.names() if n.startswith(embedder)})
        return cls(cfg, w, torch.device(device), dtype)

    def _norm(self, x: torch.Tensor, w: torch.Tensor | None) -> torch.Tensor:
        y = x.float() * torch.pow(x.float().pow(2).mean(-1, keepdim=True) + self.cfg.eps, -0.5)
        return (y * w.float() if w is not None else y).to(x.dtype)

    def _linear(self, x: torch.Tensor, name: str) -> torch.Tensor:
        w = self.w
        if self.cfg.clipped:
            x = torch.clamp(x, w[name + ".input_min"], w[name + ".input_max"])
        y = x @ w[name + ".linear.weight"].t()
        if self.cfg.clipped:
            y = torch.clamp(y, w[name + ".output_min"], w[name + ".output_max"])
        return y

    def _rotary(self, pos: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        half = c.head_dim // 2                                                          # channels that turn with one axis
        inv = 1.0 / (c.theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=self.device) / half))
        parts = []
        for axis in range(2):
            ang = pos[:, axis:axis + 1].float() * inv                                   # [N, half/2]
            parts.append(torch.cat((ang, ang), -1))
        ang = torch.cat(parts, -1)                                                      # [N, head_dim]
        return ang.cos()[:, None, :].to(self.dtype), ang.sin()[:, None, :].to(self.dtype)

    @staticmethod
    def _turn(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """Each half of the head is rotated on its own (pairs i, i + quarter within the half)."""
        out = []
        for xs, cs, ss in zip(x.chunk(2, -1), cos.chunk(2, -1), sin.chunk(2, -1)):
            out.append(xs * cs + _rot_half(xs) * ss)
        return torch.cat(out, -1)

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """``patches [n, 3*patch²]`` in ``[0, 1]``, ``positions [n, 2]`` (x, y) → ``[n / pool², decoder hidden]``."""
        c, w = self.cfg, self.w
        pos = positions.to(self.device).long()
        x = (2 * (patches.to(device=self.device, dtype=self.dtype) - 0.5)) @ w["patch_embedder.input_proj.weight"].t()
        table = w["patch_embedder.position_embedding_table"]
        x = x + table[0][pos[:, 0]] + table[1][pos[:, 1]]
        cos, sin = self._rotary(pos)
        n, H, KV, D = x.shape[0], c.heads, c.kv_heads, c.head_dim
        for i in range(c.layers):
            b = f"encoder.layers.{i}."
            y = self._norm(x, w[b + "input_layernorm.weight"])
            q = self._norm(self._linear(y, b + "self_attn.q_proj").view(n, H, D), w[b + "self_attn.q_norm.weight"])
            k = self._norm(self._linear(y, b + "self_attn.k_proj").view(n, KV, D), w[b + "self_attn.k_norm.weight"])
            v = self._norm(self._linear(y, b + "self_attn.v_proj").view(n, KV, D), None)
            q, k = self._turn(q, cos, sin), self._turn(k, cos, sin)
            if KV != H:
                k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
            o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], scale=1.0)
            o = self._linear(o[0].transpose(0, 1).reshape(n, H * D), b + "self_attn.o_proj")
            x = x + self._norm(o, w[b + "post_attention_layernorm.weight"])
            y = self._norm(x, w[b + "pre_feedforward_layernorm.weight"])
            y = F.gelu(self._linear(y, b + "mlp.gate_proj"), approximate="tanh") * self._linear(y, b + "mlp.up_proj")
            x = x + self._norm(self._linear(y, b + "mlp.down_proj"), w[b + "post_feedforward_layernorm.weight"])
        # pool x pool neighbours (by position) are averaged; the grid's width in kernels orders the outputs row by row
        kq = c.pool
        if kq > 1:
            cells = torch.div(pos, kq, rounding_mode="floor")
            per_row = (int(pos[:, 0].max()) + 1) // kq
            idx = cells[:, 0] + per_row * cells[:, 1]
            out = torch.zeros(n // (kq * kq), x.shape[1], dtype=torch.float32, device=self.device)
            out.index_add_(0, idx, x.float() / (kq * kq))
            x = out.to(self.dtype)
        x = x * c.hidden ** 0.5
        if c.standardize:
            x = (x - w["std_bias"]) * w["std_scale"]
        return self._norm(x, None) @ w["embed_vision.embedding_projection.weight"].t()


# ---------------------------------------------------------------------------------------------------------------------
# Kimi-K2.5 / K2.6: MoonViT with a resampled 2-D position table, 2-D rotary positions, 2x2 merge, MLP projector
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class KimiTowerConfig:
    patch: int = 14
    pos_h: int = 64                   # the learned position table's grid
    pos_w: int = 64
    pos_t: int = 4
    heads: int = 16
    layers: int = 27
    hidden: int = 1152
    mlp_dim: int = 4304
    merge: tuple[int, int] = (2, 2)
    out_hidden: int = 1152            # the decoder's hidden size
    proj_eps: float = 1e-5

    @classmethod
    def from_config(cls, vc: dict[str, Any]) -> "KimiTowerConfig":
        h = vc.get("hidden_size", 1152)
        return cls(patch=vc.get("patch_size", 14), pos_h=vc.get("init_pos_emb_height", 64), pos_w=vc.get("init_pos_emb_width", 64),
                   pos_t=vc.get("init_pos_emb_time", 4), heads=vc.get("num_attention_heads", 16), layers=vc.get("num_hidden_layers", 27),
                   hidden=h, mlp_dim=vc.get("intermediate_size", 4304), merge=tuple(vc.get("merge_kernel_size", (2, 2))),
                   out_hidden=vc.get("mm_hidden_size") or h, proj_eps=vc.get("projector_ln_eps", 1e-5))


@dataclass
class KimiTower:
    """The Kimi-K2.5 vision tower and projector over ``KimiVLProcessor`` patches.

    ``weights``: the checkpoint's ``vision_tower.*`` tensors without that prefix (``patch_embed.proj``, ``patch_embed.pos_emb.weight``
    ``[H, W, C]``, ``encoder.blocks.N.{norm0,norm1,wqkv,wo,mlp.fc0,mlp.fc1}``, ``encoder.final_layernorm``) and the projector's
    as ``mm_projector.{pre_norm,proj.0,proj.2}`` (or ``linear_1`` / ``linear_2``).  A patch is a ``patch x patch`` convolution;
    the learned position table is resampled bicubically to the image's grid (frames after the first add a fixed sinusoid of
    the frame index); rotary positions turn adjacent channel pairs, alternately by column and by row; attention is full
    within one image (all of its frames) and never crosses images; the ``merge`` neighbours of the frame-averaged grid are
    normalised one by one, joined, and mapped to the decoder's width by a two-layer GELU MLP."""
    cfg: KimiTowerConfig
    weights: dict[str, torch.Tensor]
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        self.w = {k: v.to(device=self.device, dtype=self.dtype) for k, v in self.weights.items()}
        for old, new in (("mm_projector.linear_1.", "mm_projector.proj.0."), ("mm_projector.linear_2.", "mm_projector.proj.2.")):
            for k in [k for k in self.w if k.startswith(old)]:
                self.w[new + k[len(old):]] = self.w.pop(k)

    @classmethod
    def from_source(cls, src, cfg: KimiTowerConfig, device, dtype, prefix: str = "vision_tower.", projector: str = "mm_projector.") -> "KimiTower":
        names = [n for n in src.names() if n.startswith(prefix)]
        if not names:
            raise KeyError(f"checkpoint has no {prefix}* tensors")
        w = {n[len(prefix):]: src.get(n, None) for n in names}
        w.update({"mm_projector." + n[len(projector):]: src.get(n, None) for n in src.names() if n.startswith(projector)})
        return cls(cfg, w, torch.device(device), dtype)

    def _positions(self, grid_thw: list[tuple[int, int, int]]) -> torch.Tensor:
        c, tab = self.cfg, self.w["patch_embed.pos_emb.weight"]
        out = []
        for t, h, w in grid_thw:
            e = tab if (h, w) == tuple(tab.shape[:2]) else \
                F.interpolate(tab.permute(2, 0, 1)[None].float(), size=(h, w), mode="bicubic")[0].permute(1, 2, 0).to(tab.dtype)
            e = e.reshape(h * w, -1)
            if t > 1:
                half = c.hidden // 2
                omega = 1.0 / 10000 ** (torch.arange(half, dtype=torch.float32, device=self.device) / half)
                ang = torch.arange(t, dtype=torch.float32, device=self.device)[:, None] * omega
                e = (e[None] + torch.cat((ang.sin(), ang.cos()), 1)[:, None].to(e.dtype)).reshape(t * h * w, -1)
            out.append(e)
        return torch.cat(out)

    def _rotary(self, grid_thw: list[tuple[int, int, int]]) -> tuple[torch.Tensor, torch.Tensor]:
        hd = self.cfg.hidden // self.cfg.heads
        f = 1.0 / (10000.0 ** (torch.arange(0, hd, 4, dtype=torch.float32, device=self.device)[: hd // 4] / hd))
        angs = []
        for t, h, w in grid_thw:
            ys, xs = torch.meshgrid(torch.arange(h, device=self.device), torch.arange(w, device=self.device), indexing="ij")
            a = torch.stack((xs.reshape(-1, 1).float() * f, ys.reshape(-1, 1).float() * f), -1).reshape(h * w, hd // 2)
            angs.append(a.repeat(t, 1))
        ang = torch.cat(angs)                                                    # [N, hd/2]: x, y, x, y, ... per frequency
        return ang.cos()[:, None, :], ang.sin()[:, None, :]

    @staticmethod
    def _turn(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        a, b = x.float().reshape(*x.shape[:-1], -1, 2).unbind(-1)
        return torch.stack((a * cos - b * sin, a * sin + b * cos), -1).flatten(-2).to(x.dtype)

    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, grid: torch.Tensor) -> torch.Tensor:
        """``patches [N, 3, patch, patch]``, ``grid [n, 2]`` (h, w) or ``[n, 3]`` (t, h, w) → ``[sum h*w/merge, out_hidden]``."""
        c, w = self.cfg, self.w
        g = [(1, int(r[0]), int(r[1])) if len(r) == 2 else (int(r[0]), int(r[1]), int(r[2])) for r in grid.tolist()]
        E, H = c.hidden, c.heads
        x = F.conv2d(patches.to(device=self.device, dtype=self.dtype), w["patch_embed.proj.weight"], w.get("patch_embed.proj.bias"),
                     stride=c.patch).reshape(patches.shape[0], E)
        x = x + self._positions(g)
        cos, sin = self._rotary(g)
        spans = [t * h * ww for t, h, ww in g]
        for i in range(c.layers):
            b = f"encoder.blocks.{i}."
            y = F.layer_norm(x, (E,), w[b + "norm0.weight"], w[b + "norm0.bias"])
            q, k, v = self._lin(y, b + "wqkv").view(-1, 3, H, E // H).unbind(1)
            q, k = self._turn(q, cos, sin), self._turn(k, cos, sin)
            outs, o = [], 0
            for n in spans:
                qs, ks, vs = (t[o:o + n].transpose(0, 1)[None] for t in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qs, ks, vs)[0].transpose(0, 1).reshape(n, E))
                o += n
            x = x + self._lin(torch.cat(outs), b + "wo")
            y = F.layer_norm(x, (E,), w[b + "norm1.weight"], w[b + "norm1.bias"])
            x = x + self._lin(F.gelu(self._lin(y, b + "mlp.fc0"), approximate="tanh"), b + "mlp.fc1")
        x = F.layer_norm(x, (E,), w["encoder.final_layernorm.weight"], w["encoder.final_layernorm.bias"])
        kh, kw = c.merge
        merged, o = [], 0
        for (t, h, ww), n in zip(g, spans):
            v = x[o:o + n].view(t, h // kh, kh, ww // kw, kw, E).mean(0)           # frames are averaged before the merge
            merged.append(v.permute(0, 2, 1, 3, 4).reshape(-1, kh * kw, E))
            o += n
        m = torch.cat(merged)
        m = F.layer_norm(m, (E,), w["mm_projector.pre_norm.weight"], w["mm_projector.pre_norm.bias"], c.proj_eps).view(-1, kh * kw * E)
        return self._lin(F.gelu(self._lin(m, "mm_projector.proj.0")), "mm_projector.proj.2")
