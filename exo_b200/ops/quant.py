"""Block-scaled fp8 weights: packers, the container the model holds, and the fp32 definition.

Two layouts, both with e4m3 payloads stored row-major ``[N, K]`` (one byte per weight):

* ``mxfp8`` — one e8m0 scale (a power of two, stored as its biased exponent byte) per 32
  consecutive weights of a row: ``scale [N, K/32] uint8``.  This is what the "8-bit" model cards
  are served with (the reference serves them as MLX affine 8-bit group-quantised linears,
  ``src/exo/worker/engines/mlx/auto_parallel.py:787-800``).
* ``dsfp8`` — DeepSeek-V3's checkpoint format: one fp32 scale per 128x128 weight block,
  ``scale [ceil(N/128), ceil(K/128)] float32`` (``weight_scale_inv`` in the HF files).

The definition every kernel is tested against: ``W_deq = bf16(e4m3 * scale)``, then the ordinary
bf16 linear layer.  Activations stay bf16 (weight-only quantisation: the decode path is bound by
the bytes of the weights, which this halves).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

E4M3_MAX = 448.0
MX_BLOCK = 32
DS_BLOCK = 128


TILE_N, TILE_K = 128, 64
TILE_TAIL = 256                                   # per-tile scales: 128 rows x 2 e8m0 bytes, or one fp32 + padding
TILE_BYTES = TILE_N * TILE_K + TILE_TAIL          # 8448: what one pipeline stage of the GEMM copies, contiguous in memory


@dataclass
class Fp8Weight:
    """A quantised ``[N, K]`` (or stacked ``[E, N, K]``) weight matrix.

    Two storage forms.  *Plain*: ``q`` row-major plus ``scale`` (what the packers produce and the
    CPU definition reads).  *Tiled* (what the GPU kernels stream): ``tiles [..., N/128, K/64, 8448]``
    bytes — every 128x64 block of the matrix contiguous, followed by its scales — so that a
    pipeline stage is ONE 8448-byte bulk copy of consecutive DRAM bytes, and the scales arrive in
    shared memory with the weights.  ``to_tiled()`` converts in place and drops the plain form."""
    q: torch.Tensor | None          # float8_e4m3fn, same shape as the weight
    scale: torch.Tensor | None      # uint8 [..., N, K/32] (mxfp8) or float32 [..., ceil(N/128), ceil(K/128)] (dsfp8)
    kind: str                       # "mxfp8" | "dsfp8"
    tiles: torch.Tensor | None = None
    logical_shape: tuple[int, ...] | None = None

    @property
    def shape(self) -> torch.Size:
        return torch.Size(self.logical_shape) if self.q is None else self.q.shape

    @property
    def device(self) -> torch.device:
        return (self.tiles if self.q is None else self.q).device

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    @property
    def dtype(self) -> torch.dtype:
        return torch.bfloat16

    def storage(self) -> list[torch.Tensor]:
        return [t for t in (self.q, self.scale, self.tiles) if t is not None]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.storage())

    def to(self, device) -> "Fp8Weight":
        mv = lambda t: None if t is None else t.to(device)      # noqa: E731
        return Fp8Weight(mv(self.q), mv(self.scale), self.kind, mv(self.tiles), self.logical_shape)

    def to_tiled(self) -> "Fp8Weight":
        if self.tiles is None:
            self.logical_shape = tuple(self.q.shape)
            self.tiles = pack_tiles(self.q, self.scale, self.kind)
            self.q = self.scale = None
        return self

    def plain(self) -> tuple[torch.Tensor, torch.Tensor]:
        if self.q is not None:
            return self.q, self.scale
        return unpack_tiles(self.tiles, self.logical_shape, self.kind)

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return dequantize(self).to(dtype)

    def __getitem__(self, i) -> "Fp8Weight":      # one expert of a stacked weight
        if self.q is None:
            return Fp8Weight(None, None, self.kind, self.tiles[i], tuple(self.logical_shape[1:]))
        return Fp8Weight(self.q[i], self.scale[i], self.kind)


def pack_tiles(q: torch.Tensor, scale: torch.Tensor, kind: str) -> torch.Tensor:
    """``[..., N, K]`` e4m3 + scales -> ``[..., ceil(N/128), ceil(K/64), 8448]`` bytes (zero padded)."""
    *lead, N, K = q.shape
    nt, kt = -(-N // TILE_N), -(-K // TILE_K)
    qb = torch.zeros(*lead, nt * TILE_N, kt * TILE_K, dtype=torch.uint8, device=q.device)
    qb[..., :N, :K] = q.view(torch.uint8)
    body = qb.view(*lead, nt, TILE_N, kt, TILE_K).transpose(-3, -2).reshape(*lead, nt, kt, TILE_N * TILE_K)
    tail = torch.zeros(*lead, nt, kt, TILE_TAIL, dtype=torch.uint8, device=q.device)
    if kind == "mxfp8":
        sb = torch.zeros(*lead, nt * TILE_N, kt * 2, dtype=torch.uint8, device=q.device)
        sb[..., :N, :K // MX_BLOCK] = scale
        tail[..., :] = sb.view(*lead, nt, TILE_N, kt, 2).transpose(-3, -2).reshape(*lead, nt, kt, TILE_TAIL)
    else:
        per_tile = scale.float()[..., :, torch.arange(kt, device=q.device) // 2]          # [..., nt, kt]
        tail[..., :4] = per_tile.contiguous().view(torch.uint8).view(*lead, nt, kt, 4)
    return torch.cat((body, tail), dim=-1).contiguous()


def unpack_tiles(tiles: torch.Tensor, shape: tuple[int, ...], kind: str) -> tuple[torch.Tensor, torch.Tensor]:
    *lead, N, K = shape
    nt, kt = tiles.shape[-3], tiles.shape[-2]
    body = tiles[..., :TILE_N * TILE_K].reshape(*lead, nt, kt, TILE_N, TILE_K).transpose(-3, -2)
    q = body.reshape(*lead, nt * TILE_N, kt * TILE_K)[..., :N, :K].contiguous().view(torch.float8_e4m3fn)
    tail = tiles[..., TILE_N * TILE_K:]
    if kind == "mxfp8":
        sb = tail.reshape(*lead, nt, kt, TILE_N, 2).transpose(-3, -2).reshape(*lead, nt * TILE_N, kt * 2)
        return q, sb[..., :N, :K // MX_BLOCK].contiguous()
    per_tile = tail[..., :4].contiguous().view(torch.float32).reshape(*lead, nt, kt)
    return q, per_tile[..., ::2][..., :-(-K // DS_BLOCK)].contiguous()


def _e8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, e.float() - 127.0)


def quantize_mxfp8(w: torch.Tensor) -> Fp8Weight:
    """1x32 blocks along K with the smallest power-of-two scale that brings the block maximum
    inside e4m3's range (448), so nothing saturates."""
    *lead, N, K = w.shape
    if K % MX_BLOCK:
        raise ValueError(f"mxfp8 needs K % {MX_BLOCK} == 0, got {K}")
    wf = w.float().reshape(*lead, N, K // MX_BLOCK, MX_BLOCK)
    amax = wf.abs().amax(-1)
    exp = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -110) / E4M3_MAX))
    exp = torch.where(amax > 0, exp, torch.full_like(exp, -127.0)).clamp(-127.0, 127.0)
    q = (wf / torch.pow(2.0, exp)[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return Fp8Weight(q.reshape(*lead, N, K).contiguous(), (exp + 127.0).to(torch.uint8).contiguous(), "mxfp8")


def quantize_dsfp8(w: torch.Tensor) -> Fp8Weight:
    """128x128 blocks with fp32 scales ``amax / 448``."""
    *lead, N, K = w.shape
    nb, kb = -(-N // DS_BLOCK), -(-K // DS_BLOCK)
    wf = torch.zeros(*lead, nb * DS_BLOCK, kb * DS_BLOCK, dtype=torch.float32, device=w.device)
    wf[..., :N, :K] = w.float()
    blocks = wf.reshape(*lead, nb, DS_BLOCK, kb, DS_BLOCK)
    scale = (blocks.abs().amax((-3, -1)) / E4M3_MAX).clamp_min(1e-12)
    q = (blocks / scale[..., :, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(*lead, nb * DS_BLOCK, kb * DS_BLOCK)[..., :N, :K].contiguous()
    return Fp8Weight(q, scale.contiguous(), "dsfp8")


def quantize(w: torch.Tensor, kind: str) -> Fp8Weight:
    """Pack ``w``; on a CUDA device the result is left in the tiled form the kernels stream."""
    if kind == "mxfp8":
        out = quantize_mxfp8(w)
    elif kind == "dsfp8":
        out = quantize_dsfp8(w)
    else:
        raise ValueError(f"unknown quantisation {kind!r}")
    return out.to_tiled() if w.is_cuda else out


def dequantize(w: Fp8Weight) -> torch.Tensor:
    """``bf16(e4m3 * scale)`` as float32 values."""
    q, scale = w.plain()
    *lead, N, K = q.shape
    qf = q.float()
    if w.kind == "mxfp8":
        s = _e8m0_to_float(scale).repeat_interleave(MX_BLOCK, dim=-1)
    else:
        s = scale.repeat_interleave(DS_BLOCK, dim=-2).repeat_interleave(DS_BLOCK, dim=-1)[..., :N, :K]
    return (qf * s).bfloat16().float()


def from_checkpoint(q: torch.Tensor, scale_inv: torch.Tensor) -> Fp8Weight:
    """Wrap a DeepSeek-style checkpoint pair (``weight`` in e4m3, ``weight_scale_inv`` fp32 per 128x128 block)."""
    return Fp8Weight(q.contiguous(), scale_inv.float().contiguous(), "dsfp8")
