"""Image inputs for the language engine: a ViT tower + projector, the image pre-processing, and the
splice of the resulting features into a prompt.

Reference role: ``VisionEncoder`` / ``VisionProcessor`` (``src/exo/worker/engines/mlx/vision.py``:
tower + projector loaded from the model repo, ``:201-485``; Qwen-VL style grid processing,
``:487-624``; ``process`` → expanded prompt, embeddings, media regions with content hashes and a
32-entry feature cache, ``:719-818``) and ``patch_embed_tokens`` (``generator/generate.py:82-150``).

Here the tower is a plain PyTorch module on the engine's device (pre-norm ViT, 2-D sin-cos
positions, 2x2 spatial merge, MLP projector to the decoder's hidden size — the Qwen2-VL shape).
Its weights come from the checkpoint when it has ``visual.*`` tensors and are seeded random
otherwise (as with the other random-init bench models), so the data path — pixels → features →
placeholder tokens replaced by features in the prefill step → prefix-cache keys that include the
image hash — is exercised end to end.  The features travel to the engine as
``Engine.submit(embeds=...)``; only single-rank instances take images (the step plan that the
other ranks receive carries token ids, not embeddings).
"""
from __future__ import annotations

import base64
import hashlib
import io
import math
from collections import OrderedDict
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class VisionConfig:
    patch: int = 14
    merge: int = 2                 # merge x merge neighbouring patches become one token
    width: int = 256
    depth: int = 4
    heads: int = 4
    out_hidden: int = 1024
    min_tokens: int = 4
    max_tokens: int = 1024         # per image, after the merge

    @property
    def cell(self) -> int:
        return self.patch * self.merge


def sincos_2d(h: int, w: int, dim: int, device) -> torch.Tensor:
    """``[h*w, dim]`` fixed 2-D positions (half of the channels encode the row, half the column)."""
    def axis(n: int, d: int) -> torch.Tensor:
        pos = torch.arange(n, device=device, dtype=torch.float32)[:, None]
        freq = torch.exp(torch.arange(0, d, 2, device=device, dtype=torch.float32) * (-math.log(10000.0) / d))
        return torch.cat((torch.sin(pos * freq), torch.cos(pos * freq)), -1)
    rows, cols = axis(h, dim // 2), axis(w, dim // 2)
    return torch.cat((rows[:, None, :].expand(h, w, -1), cols[None, :, :].expand(h, w, -1)), -1).reshape(h * w, dim)


class VisionTower:
    """Pre-norm ViT + merge + projector; weights are a flat dict of tensors on ``device``."""

    def __init__(self, cfg: VisionConfig, device, dtype=torch.float32, weights: dict[str, torch.Tensor] | None = None, seed: int = 0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        g = torch.Generator().manual_seed(seed)
        W, p = cfg.width, cfg.patch

        def get(name: str, *shape: int, std: float = 0.02, ones: bool = False) -> torch.Tensor:
            if weights is not None and name in weights and tuple(weights[name].shape) == shape:
                t = weights[name]
            else:
                t = torch.ones(shape) if ones else torch.randn(shape, generator=g) * std
            return t.to(device=self.device, dtype=dtype)
        self.w = {"patch": get("visual.patch_embed.weight", W, 3 * p * p), "patch_b": get("visual.patch_embed.bias", W, std=0.0)}
        for i in range(cfg.depth):
            b = f"visual.blocks.{i}."
            self.w.update({b + "ln1": get(b + "norm1.weight", W, ones=True), b + "ln2": get(b + "norm2.weight", W, ones=True),
                           b + "qkv": get(b + "attn.qkv.weight", 3 * W, W), b + "proj": get(b + "attn.proj.weight", W, W),
                           b + "fc1": get(b + "mlp.fc1.weight", 4 * W, W), b + "fc2": get(b + "mlp.fc2.weight", W, 4 * W)})
        m = cfg.merge * cfg.merge * W
        self.w.update({"ln_out": get("visual.merger.ln_q.weight", W, ones=True), "m1": get("visual.merger.mlp.0.weight", m, m),
                       "m2": get("visual.merger.mlp.2.weight", cfg.out_hidden, m)})

    @torch.no_grad()
    def __call__(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [3, H, W]`` (normalised, H and W multiples of patch*merge) → ``[H/cell * W/cell, out_hidden]``."""
        cfg, w = self.cfg, self.w
        p, W = cfg.patch, cfg.width
        x = pixels.to(device=self.device, dtype=self.dtype)
        gh, gw = x.shape[1] // p, x.shape[2] // p
        patches = x.unfold(1, p, p).unfold(2, p, p).permute(1, 2, 0, 3, 4).reshape(gh * gw, 3 * p * p)
        h = patches @ w["patch"].t() + w["patch_b"] + sincos_2d(gh, gw, W, self.device).to(self.dtype)
        hd = W // cfg.heads
        for i in range(cfg.depth):
            b = f"visual.blocks.{i}."
            y = F.layer_norm(h, (W,), w[b + "ln1"])
            q, k, v = (y @ w[b + "qkv"].t()).view(-1, 3, cfg.heads, hd).permute(1, 2, 0, 3)
            a = F.scaled_dot_product_attention(q[None], k[None], v[None])[0].permute(1, 0, 2).reshape(-1, W)
            h = h + a @ w[b + "proj"].t()
            y = F.layer_norm(h, (W,), w[b + "ln2"])
            h = h + F.gelu(y @ w[b + "fc1"].t()) @ w[b + "fc2"].t()
        h = F.layer_norm(h, (W,), w["ln_out"])
        mg = cfg.merge
        h = h.view(gh // mg, mg, gw // mg, mg, W).permute(0, 2, 1, 3, 4).reshape((gh // mg) * (gw // mg), mg * mg * W)
        return F.gelu(h @ w["m1"].t()) @ w["m2"].t()


MEAN = (0.48145466, 0.4578275, 0.40821073)
STD = (0.26862954, 0.26130258, 0.27577711)


def preprocess(data: bytes, cfg: VisionConfig) -> torch.Tensor:
    """Decode, resize to a grid of whole cells with at most ``max_tokens`` cells (aspect kept), normalise → ``[3, H, W]``."""
    import numpy as np
    from PIL import Image
    with Image.open(io.BytesIO(data)) as im:
        im = im.convert("RGB")
        w0, h0 = im.size
        cell = cfg.cell
        scale = min(1.0, math.sqrt(cfg.max_tokens * cell * cell / max(1, w0 * h0)))
        gw = max(1, min(cfg.max_tokens, round(w0 * scale / cell)))
        gh = max(1, min(cfg.max_tokens // gw, round(h0 * scale / cell)))
        while gw * gh < cfg.min_tokens:
            gw, gh = gw + (gw <= gh), gh + (gh < gw)
        im = im.resize((gw * cell, gh * cell), Image.BICUBIC)
        x = torch.from_numpy(np.asarray(im, dtype=np.float32) / 255.0).permute(2, 0, 1)
    mean, std = torch.tensor(MEAN)[:, None, None], torch.tensor(STD)[:, None, None]
    return (x - mean) / std


@dataclass
class ImageFeatures:
    digest: bytes                 # content hash of the image bytes (keys the prefix cache and the feature cache)
    rows: torch.Tensor            # [n_tokens, hidden]


class VisionProcessor:
    """Images (base64) → features, with a small LRU keyed by content hash."""

    def __init__(self, tower: VisionTower, cache_entries: int = 32):
        self.tower, self.cache_entries = tower, cache_entries
        self.cache: OrderedDict[bytes, torch.Tensor] = OrderedDict()
        self.hits = 0

    def features(self, image_b64: str) -> ImageFeatures:
        raw = base64.b64decode(image_b64.split(",", 1)[1] if image_b64.startswith("data:") else image_b64)
        digest = hashlib.sha256(raw).digest()
        rows = self.cache.get(digest)
        if rows is None:
            rows = self.tower(preprocess(raw, self.tower.cfg))
            self.cache[digest] = rows
            while len(self.cache) > self.cache_entries:
                self.cache.popitem(last=False)
        else:
            self.cache.move_to_end(digest)
            self.hits += 1
        return ImageFeatures(digest, rows)


def splice(ids: list[int], placeholder_id: int | None, images: list[ImageFeatures], fill_id: int, after_first: bool = True):
    """Expand the prompt for its images.  Every occurrence of ``placeholder_id`` (one per image, in order) becomes
    ``n_tokens`` copies of ``fill_id``; images without a placeholder in the text go to the front of the prompt (after the
    first token when ``after_first``).  Returns ``(ids, embeds, media)`` for ``Engine.submit``: ``embeds = [(position,
    rows)]`` and ``media = [(start, end, digest)]``."""
    out: list[int] = []
    embeds: list[tuple[int, torch.Tensor]] = []
    media: list[tuple[int, int, bytes]] = []
    it = iter(images)
    pending = list(images)
    for t in ids:
        if placeholder_id is not None and t == placeholder_id and pending:
            f = next(it)
            pending.pop(0)
            embeds.append((len(out), f.rows))
            media.append((len(out), len(out) + f.rows.shape[0], f.digest))
            out.extend([fill_id] * f.rows.shape[0])
        else:
            out.append(t)
    if pending:      # no placeholders left in the text: put the remaining images in front
        head = out[:1] if (after_first and out) else []
        body = out[len(head):]
        front: list[int] = list(head)
        new_embeds, new_media = [], []
        for f in pending:
            new_embeds.append((len(front), f.rows))
            new_media.append((len(front), len(front) + f.rows.shape[0], f.digest))
            front.extend([fill_id] * f.rows.shape[0])
        shift = len(front) - len(head)
        embeds = new_embeds + [(p + shift, r) for p, r in embeds]
        media = new_media + [(a + shift, b + shift, d) for a, b, d in media]
        out = front + body
    return out, embeds, media
