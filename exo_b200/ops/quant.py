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


@dataclass
class Fp8Weight:
    """A quantised ``[N, K]`` (or stacked ``[E, N, K]``) weight matrix."""
    q: torch.Tensor          # float8_e4m3fn, same shape as the weight
    scale: torch.Tensor      # uint8 [..., N, K/32] (mxfp8) or float32 [..., ceil(N/128), ceil(K/128)] (dsfp8)
    kind: str                # "mxfp8" | "dsfp8"

    @property
    def shape(self) -> torch.Size:
        return self.q.shape

    @property
    def device(self) -> torch.device:
        return self.q.device

    @property
    def is_cuda(self) -> bool:
        return self.q.is_cuda

    @property
    def dtype(self) -> torch.dtype:
        return torch.bfloat16

    def nbytes(self) -> int:
        return self.q.numel() + self.scale.numel() * self.scale.element_size()

    def to(self, device) -> "Fp8Weight":
        return Fp8Weight(self.q.to(device), self.scale.to(device), self.kind)

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return dequantize(self).to(dtype)

    def __getitem__(self, i) -> "Fp8Weight":      # one expert of a stacked weight
        return Fp8Weight(self.q[i], self.scale[i], self.kind)


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
    if kind == "mxfp8":
        return quantize_mxfp8(w)
    if kind == "dsfp8":
        return quantize_dsfp8(w)
    raise ValueError(f"unknown quantisation {kind!r}")


def dequantize(w: Fp8Weight) -> torch.Tensor:
    """``bf16(e4m3 * scale)`` as float32 values."""
    *lead, N, K = w.q.shape
    qf = w.q.float()
    if w.kind == "mxfp8":
        s = _e8m0_to_float(w.scale).repeat_interleave(MX_BLOCK, dim=-1)
    else:
        s = w.scale.repeat_interleave(DS_BLOCK, dim=-2).repeat_interleave(DS_BLOCK, dim=-1)[..., :N, :K]
    return (qf * s).bfloat16().float()


def from_checkpoint(q: torch.Tensor, scale_inv: torch.Tensor) -> Fp8Weight:
    """Wrap a DeepSeek-style checkpoint pair (``weight`` in e4m3, ``weight_scale_inv`` fp32 per 128x128 block)."""
    return Fp8Weight(q.contiguous(), scale_inv.float().contiguous(), "dsfp8")
