"""Weight containers: random initialisation, HF safetensors loading and TP/EP sharding.

The checkpoint format is the HuggingFace repository layout the reference loads through
``mlx_lm.utils.load_model`` (``src/exo/worker/engines/mlx/utils_mlx.py:163-286``):
``config.json`` + ``*.safetensors`` (+ ``model.safetensors.index.json``).  Tensor-parallel
slicing follows the Megatron convention the reference applies per family
(``src/exo/worker/engines/mlx/auto_parallel.py:628-652`` for Llama, ``:688-767`` for
DeepSeek/MoE): q/k/v/gate/up split on the output dim, o/down split on the input dim.
Differences by design: the vocabulary projection is sharded too, KV heads are replicated
when there are fewer of them than ranks, and routed experts are partitioned whole (expert
parallel) instead of being sliced on their FFN dim.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterator

import torch

from ..ops.quant import Fp8Weight, quantize
from .config import ModelConfig

_DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


@dataclass
class ShardSpec:
    """Which slice of the model one rank holds."""
    tp_rank: int = 0
    tp_size: int = 1
    layer_start: int = 0
    layer_end: int = -1  # exclusive; -1 = n_layers
    pp_rank: int = 0
    pp_size: int = 1

    def layers(self, cfg: ModelConfig) -> range:
        return range(self.layer_start, cfg.n_layers if self.layer_end < 0 else self.layer_end)

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1


def _rows(t: torch.Tensor, r: int, n: int) -> torch.Tensor:
    c = t.shape[0] // n
    return t[r * c:(r + 1) * c]


def _cols(t: torch.Tensor, r: int, n: int) -> torch.Tensor:
    c = t.shape[1] // n
    return t[:, r * c:(r + 1) * c]


def kv_head_range(cfg: ModelConfig, spec: ShardSpec) -> tuple[int, int]:
    """KV heads ``[lo, hi)`` owned by this rank; replicated when ``n_kv_heads < tp_size``."""
    n, r = spec.tp_size, spec.tp_rank
    if cfg.n_kv_heads >= n:
        c = cfg.n_kv_heads // n
        return r * c, (r + 1) * c
    h = r * cfg.n_kv_heads // n
    return h, h + 1


def local_heads(cfg: ModelConfig, spec: ShardSpec) -> tuple[int, int]:
    """``(q heads, kv heads)`` on this rank."""
    lo, hi = kv_head_range(cfg, spec)
    return cfg.n_heads // spec.tp_size, hi - lo


def vocab_shard(vocab: int, n: int) -> int:
    """Rows of the vocabulary projection per rank: ceil(vocab / n) rounded up to 8 (16-byte rows
    of bf16 logits for the fused all-gather); the tail of the last rank is zero padding."""
    return -(-(-(-vocab // n)) // 8) * 8 if n > 1 else vocab


def expert_range(cfg: ModelConfig, spec: ShardSpec) -> tuple[int, int]:
    c = cfg.n_experts // spec.tp_size
    return spec.tp_rank * c, (spec.tp_rank + 1) * c


class TensorSource:
    """Produces full (unsharded) tensors by HF name; implementations: random or safetensors."""

    def get(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def has(self, name: str) -> bool:
        return True


class RandomSource(TensorSource):
    """Deterministic N(0, std) tensors: the value of a tensor depends only on (seed, name).

    ``names starting with a norm`` get ones.  Router gates use ``router_std`` (the Qwen3
    benchmark config asks for N(0,1) router logits, i.e. a larger gate init).
    """

    def __init__(self, seed: int = 0, std: float = 0.02, device: str | torch.device = "cpu",
                 dtype: torch.dtype = torch.float32, router_std: float | None = None):
        self.seed, self.std, self.device, self.dtype = seed, std, torch.device(device), dtype
        self.router_std = router_std

    def _gen(self, name: str) -> torch.Generator:
        h = 1469598103934665603
        for ch in name.encode():
            h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        g = torch.Generator(device=self.device)
        g.manual_seed((h ^ (self.seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF)
        return g

    def get(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        if ("norm" in name and name.endswith("weight")) or name.endswith("layer_scalar"):
            return torch.ones(shape, dtype=self.dtype, device=self.device)
        if name.endswith("e_score_correction_bias"):
            return torch.zeros(shape, dtype=torch.float32, device=self.device)
        std = self.std
        if self.router_std is not None and name.endswith("mlp.gate.weight"):
            std = self.router_std
        t = torch.empty(shape, dtype=torch.float32, device=self.device)
        t.normal_(0.0, std, generator=self._gen(name))
        return t.to(self.dtype)


class SafetensorsSource(TensorSource):
    """Lazy reader of a HF checkpoint directory (memory-mapped, one tensor at a time).

    Pre-quantised checkpoints are dequantised tensor by tensor as they are read (the serving quantisation is then
    applied to the result after sharding, ``quantize_layer``), so the cards that name such repositories load:

    * FP8 block-scaled (DeepSeek-V3 style): ``X.weight`` in e4m3 with ``X.weight_scale_inv`` fp32 ``[N/128, K/128]``;
    * FP8 per-tensor / per-channel (compressed-tensors style): ``X.weight`` in e4m3 with ``X.weight_scale``;
    * MLX affine groups of 2 to 6 and 8 bits, and MLX's microscaling modes (``mxfp4``, ``mxfp8``, ``nvfp4``: codes with one scale
      per group and no bias) (the mlx-community ``*-4bit`` / ``*-8bit`` repositories the reference loads with
      ``mlx_lm.utils.load_model``, ``src/exo/worker/engines/mlx/utils_mlx.py:163-286``): ``X.weight`` packed in uint32,
      ``X.scales`` / ``X.biases`` per group of ``group_size`` input features, ``bits`` and ``group_size`` from the
      ``quantization`` entry of ``config.json`` (with per-module overrides).
    """

    _ST = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F8_E4M3": torch.float8_e4m3fn,
           "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "I8": torch.int8, "U32": torch.int32}

    def __init__(self, path: str | Path, device: str | torch.device = "cpu", dtype: torch.dtype = torch.bfloat16):
        self.path, self.device, self.dtype = Path(path), torch.device(device), dtype
        self.index: dict[str, tuple[Path, str, tuple[int, ...], int, int]] = {}
        files = sorted(self.path.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {self.path}")
        for f in files:
            with open(f, "rb") as fh:
                (n,) = struct.unpack("<Q", fh.read(8))
                meta = json.loads(fh.read(n))
            for k, v in meta.items():
                if k == "__metadata__":
                    continue
                b, e = v["data_offsets"]
                self.index[k] = (f, v["dtype"], tuple(v["shape"]), 8 + n + b, e - b)
        self.quant: dict = {}
        cfg_file = self.path / "config.json"
        if cfg_file.exists():
            try:
                c = json.loads(cfg_file.read_text())
                self.quant = c.get("quantization") or c.get("quantization_config") or {}
            except (OSError, ValueError):
                self.quant = {}

    def has(self, name: str) -> bool:
        return name in self.index

    def names(self) -> Iterator[str]:
        return iter(self.index)

    def _raw(self, name: str) -> torch.Tensor:
        f, dt, shp, off, nbytes = self.index[name]
        import numpy as np
        raw = np.memmap(f, dtype=np.uint8, mode="r", offset=off, shape=(nbytes,))
        return torch.frombuffer(bytearray(raw), dtype=self._ST[dt]).view(shp)

    def _mlx_params(self, module: str) -> tuple[int, int]:
        """(bits, group_size) of an MLX-quantised module: the per-module entry wins over the global one."""
        q = self.quant
        over = q.get(module) if isinstance(q.get(module), dict) else None
        bits = int((over or q).get("bits", 4))
        group = int((over or q).get("group_size", 64))
        return bits, group

    def _mlx_mode(self, module: str) -> str:
        q = self.quant
        over = q.get(module) if isinstance(q.get(module), dict) else None
        return (over or q).get("mode", "affine")

    def stored_format(self, name: str) -> str:
        """How ``name`` is stored: ``plain``, ``fp8_block``, ``fp8_scale`` or ``mlx_affine``."""
        if name.endswith(".weight"):
            stem = name[:-len(".weight")]
            dt = self.index[name][1]
            if dt == "F8_E4M3" and stem + ".weight_scale_inv" in self.index:
                return "fp8_block"
            if dt == "F8_E4M3" and stem + ".weight_scale" in self.index:
                return "fp8_scale"
            if dt == "U32" and stem + ".scales" in self.index:
                return "mlx_affine"
        return "plain"

    def get(self, name: str, shape: tuple[int, ...] | None = None) -> torch.Tensor:
        t = self._raw(name)
        fmt = self.stored_format(name)
        if fmt != "plain":
            stem = name[:-len(".weight")]
            if fmt == "fp8_block":
                sc = self._raw(stem + ".weight_scale_inv").float()
                n_out, n_in = t.shape
                blk = self.quant.get("weight_block_size") or [128, 128]       # DeepSeek-V3: 128 x 128 blocks
                bn, bk = int(blk[0]), int(blk[1])
                if -(-n_out // bn) != sc.shape[0] or -(-n_in // bk) != sc.shape[1]:
                    raise ValueError(f"{name}: scale grid {tuple(sc.shape)} does not match {bn} x {bk} blocks of {tuple(t.shape)}")
                t = t.float() * sc.repeat_interleave(bn, 0)[:n_out].repeat_interleave(bk, 1)[:, :n_in]
            elif fmt == "fp8_scale":
                sc = self._raw(stem + ".weight_scale").float()
                t = t.float() * (sc.reshape(-1, 1) if sc.numel() > 1 else sc.reshape(1, 1))
            else:
                bits, group = self._mlx_params(stem)
                if bits not in (2, 3, 4, 5, 6, 8):
                    raise ValueError(f"{name}: {bits}-bit MLX packing is not supported (2- to 6- and 8-bit repositories are)")
                q = _mlx_unpack(t, bits)
                scales = self._raw(stem + ".scales")
                mode = str(self._mlx_mode(stem))
                if stem + ".biases" in self.index:                                    # affine groups: q * scale + bias
                    t = q.float() * scales.float().repeat_interleave(group, -1) + self._raw(stem + ".biases").float().repeat_interleave(group, -1)
                else:
                    # microscaling formats: 4-bit e2m1 or 8-bit e4m3 codes with one power-of-two (e8m0) scale per group of 32,
                    # or e2m1 codes with an e4m3 scale per group of 16 (nvfp4)
                    if bits == 4:
                        vals = _FP4_E2M1.to(q.device)[q]
                    elif bits == 8:
                        vals = q.to(torch.uint8).view(torch.float8_e4m3fn).float()
                    else:
                        raise ValueError(f"{name}: {bits}-bit codes without biases are not a known MLX format")
                    raw = scales.view(torch.uint8) if scales.dtype != torch.uint8 else scales
                    sc = raw.view(torch.float8_e4m3fn).float() if mode == "nvfp4" else torch.exp2(raw.float() - 127.0)
                    group = vals.shape[-1] // sc.shape[-1]
                    t = vals * sc.repeat_interleave(group, -1)
        if shape is not None and tuple(shape) != tuple(t.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != expected {shape}")
        if t.is_floating_point():
            t = t.to(self.dtype)
        return t.to(self.device)


_FP4_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _mlx_unpack(t: torch.Tensor, bits: int) -> torch.Tensor:
    """Codes of an MLX-packed weight ``[..., words]`` (uint32): ``bits``-wide fields, lowest bits first.  Widths that divide 32
    sit whole inside a word; 3-, 5- and 6-bit fields run on across byte boundaries (8 values in 3 or 5 bytes, 4 values in 3
    bytes), so the words are read as a little-endian byte stream and regrouped."""
    mask = (1 << bits) - 1
    if 32 % bits == 0:
        per = 32 // bits
        packed = t.to(torch.int64) & 0xFFFFFFFF
        shifts = torch.arange(per, dtype=torch.int64) * bits
        return ((packed.unsqueeze(-1) >> shifts) & mask).reshape(*t.shape[:-1], t.shape[-1] * per)
    import math
    g_bytes = math.lcm(bits, 8) // 8
    g_vals = g_bytes * 8 // bits
    by = t.contiguous().view(torch.uint8).reshape(*t.shape[:-1], -1, g_bytes).to(torch.int64)
    word = torch.zeros(by.shape[:-1], dtype=torch.int64)
    for j in range(g_bytes):
        word |= by[..., j] << (8 * j)
    shifts = torch.arange(g_vals, dtype=torch.int64) * bits
    return ((word.unsqueeze(-1) >> shifts) & mask).reshape(*t.shape[:-1], -1)


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    """Minimal safetensors writer (used by tests and by the fp8 re-pack cache)."""
    names = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32",
             torch.int64: "I64", torch.uint8: "U8", torch.int8: "I8", torch.float8_e4m3fn: "F8_E4M3",
             torch.uint32: "U32"}
    header, blobs, off = {}, [], 0
    for k, t in tensors.items():
        t = t.contiguous().cpu()
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    # GQA attention
    wqkv: torch.Tensor | None = None   # [(hq + 2 hkv) * D, H] local
    bqkv: torch.Tensor | None = None
    wo: torch.Tensor | None = None     # [H, hq * Dv] local
    bo: torch.Tensor | None = None     # [H]: bias of the output projection (GPT-OSS), added once after the ranks' sum
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    sinks: torch.Tensor | None = None
    # MLA
    wq_a: torch.Tensor | None = None
    q_a_norm: torch.Tensor | None = None
    wq_b: torch.Tensor | None = None   # [h_local * (nope + rope), q_lora]
    wkv_a: torch.Tensor | None = None  # [kv_lora + rope, H]
    kv_a_norm: torch.Tensor | None = None
    w_uk: torch.Tensor | None = None   # [h_local, nope, kv_lora]
    w_uv: torch.Tensor | None = None   # [h_local, v, kv_lora]
    w_uk_t: torch.Tensor | None = None  # [h_local, kv_lora, nope]: transposed copy made on first prefill (GEMM layout)
    # dense FFN
    w_gate_up: torch.Tensor | None = None  # [2F/N, H]  (gate rows then up rows)
    w_down: torch.Tensor | None = None     # [H, F/N]
    # MoE
    router: torch.Tensor | None = None       # [E, H]
    router_bias: torch.Tensor | None = None  # [E]
    e_gate_up: torch.Tensor | None = None    # [E_local, 2F, H]
    e_down: torch.Tensor | None = None       # [E_local, H, F]
    s_gate_up: torch.Tensor | None = None    # shared experts, TP-sliced
    s_down: torch.Tensor | None = None
    s_gate: torch.Tensor | None = None       # [1, H]: sigmoid gate on the shared expert's output (Qwen3-Next)
    router_b: torch.Tensor | None = None     # [E]: bias of the router's linear layer (GPT-OSS)
    e_gate_up_b: torch.Tensor | None = None  # [E_local, 2F]: expert biases (GPT-OSS)
    e_down_b: torch.Tensor | None = None     # [E_local, H]
    # gated-delta-rule layer (rows of lin_in: q | k | v | z | b | a of this rank's heads)
    lin_in: torch.Tensor | None = None       # [2*hk*dk + 2*hv*dv + 2*hv, H] local
    lin_conv_w: torch.Tensor | None = None   # [2*hk*dk + hv*dv, taps] fp32
    lin_a_log: torch.Tensor | None = None    # [hv] fp32
    lin_dt_bias: torch.Tensor | None = None  # [hv] fp32
    lin_norm: torch.Tensor | None = None     # [dv]
    lin_out: torch.Tensor | None = None      # [H, hv*dv] local
    # per-layer attention parameters where layers differ (Step-3.5); the defaults mean "the model-wide value"
    n_q: int = 0                             # local query heads
    inv_freq: torch.Tensor | None = None     # this layer's RoPE frequencies
    rope_mscale: float = 1.0
    window: int = -1                         # sliding window (0 = none, -1 = the model's)
    w_head_gate: torch.Tensor | None = None  # [hq local, H]: one sigmoid gate per head on the attention output
    act_limit: float = 0.0                   # clamped SwiGLU in the routed experts (0 = plain)
    shared_limit: float = 0.0                # ... in the shared expert / the dense MLP


@dataclass
class ModelWeights:
    embed: torch.Tensor | None
    layers: dict[int, LayerWeights]
    final_norm: torch.Tensor | None
    lm_head: torch.Tensor | None  # [V/N, H] local vocab shard

    def nbytes(self) -> int:
        n = 0
        for t in self.tensors():
            n += t.numel() * t.element_size()
        return n

    def tensors(self) -> Iterator[torch.Tensor]:
        for t in (self.embed, self.final_norm, self.lm_head):
            if t is not None:
                yield t
        for lw in self.layers.values():
            for v in vars(lw).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif isinstance(v, Fp8Weight):
                    yield from v.storage()


def text_model_root(cfg: ModelConfig, src: "TensorSource", embed: str = "embed_tokens.weight") -> str:
    """Prefix of the decoder's tensors in a checkpoint.  Multimodal repositories wrap the text model (``model.language_model.``
    in the Qwen-VL / Gemma layouts, ``language_model.model.`` in the Kimi-VL / LLaVA ones), and text-only exports of such
    families drop the wrapper again: the configured prefix is tried first, then the known ones."""
    for root in dict.fromkeys((cfg.weight_prefix, "model.", "model.language_model.", "language_model.model.", "backbone.")):
        if src.has(root + embed):
            return root
    return cfg.weight_prefix


def moe_names(cfg: ModelConfig) -> dict[str, str]:
    """Checkpoint tensor names of a sparse block: Mixtral keeps ``block_sparse_moe.experts.N.w1 / w3 / w2`` (gate, up,
    down); the DeepSeek / Qwen / GLM families ``mlp.experts.N.gate_proj / up_proj / down_proj``."""
    if cfg.family in ("mixtral", "minimax"):
        return {"prefix": "block_sparse_moe.", "gate": "w1.weight", "up": "w3.weight", "down": "w2.weight",
                "bias": "e_score_correction_bias"}
    return {"prefix": "mlp.", "gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
            "bias": "gate.e_score_correction_bias"}


QUANTIZED_FIELDS = ("wqkv", "wo", "w_gate_up", "w_down", "e_gate_up", "e_down", "s_gate_up", "s_down", "wq_a", "wq_b", "wkv_a",
                    "lin_out")


def linear_heads(cfg: ModelConfig, spec: ShardSpec) -> tuple[int, int]:
    """``(key heads, value heads)`` of a gated-delta-rule layer on this rank: key heads are split over the ranks and
    each takes its ``lin_v_heads / lin_k_heads`` value heads along."""
    if cfg.lin_k_heads % spec.tp_size:
        raise ValueError(f"{cfg.lin_k_heads} linear-attention key heads do not split over {spec.tp_size} ranks")
    return cfg.lin_k_heads // spec.tp_size, cfg.lin_v_heads // spec.tp_size


def _linear_attention_weights(cfg: ModelConfig, spec: ShardSpec, src: "TensorSource", p: str, lw: "LayerWeights", fin,
                              hf_form: bool) -> None:
    """Read one gated-delta-rule layer and bring its input projection into the row order ``q | k | v | z | b | a``.

    Qwen3-Next stores ``in_proj_qkvz`` / ``in_proj_ba`` grouped per key head (``[q k v.. z..]`` and ``[b.. a..]`` of one key
    head, then the next); Qwen3.5 stores ``in_proj_qkv`` (already ``q | k | v`` over all heads), ``in_proj_z``, ``in_proj_b``
    and ``in_proj_a``.  ``hf_form``: the convolution weight is ``[C, 1, taps]`` (hub layout) rather than ``[C, taps, 1]``."""
    H, r, n = cfg.hidden, spec.tp_rank, spec.tp_size
    hk, hv, dk, dv = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_k_dim, cfg.lin_v_dim
    kd, vd, ratio = hk * dk, hv * dv, hv // hk
    a = p + "linear_attn."
    if cfg.lin_split_proj:
        wqkv = src.get(a + "in_proj_qkv.weight", (2 * kd + vd, H))
        wq, wk, wv = wqkv[:kd], wqkv[kd:2 * kd], wqkv[2 * kd:]
        wz = src.get(a + "in_proj_z.weight", (vd, H))
        wb = src.get(a + "in_proj_b.weight", (hv, H))
        wa = src.get(a + "in_proj_a.weight", (hv, H))
    else:
        g = src.get(a + "in_proj_qkvz.weight", (2 * kd + 2 * vd, H)).view(hk, 2 * dk + 2 * ratio * dv, H)
        wq, wk = g[:, :dk].reshape(kd, H), g[:, dk:2 * dk].reshape(kd, H)
        wv = g[:, 2 * dk:2 * dk + ratio * dv].reshape(vd, H)
        wz = g[:, 2 * dk + ratio * dv:].reshape(vd, H)
        ba = src.get(a + "in_proj_ba.weight", (2 * hv, H)).view(hk, 2 * ratio, H)
        wb, wa = ba[:, :ratio].reshape(hv, H), ba[:, ratio:].reshape(hv, H)
    lw.lin_in = fin(torch.cat([_rows(t, r, n) for t in (wq, wk, wv, wz, wb, wa)], 0))
    C, taps = 2 * kd + vd, cfg.lin_conv
    cw = src.get(a + "conv1d.weight", (C, 1, taps) if hf_form else (C, taps, 1)).reshape(C, taps)
    lw.lin_conv_w = fin(torch.cat((_rows(cw[:kd], r, n), _rows(cw[kd:2 * kd], r, n), _rows(cw[2 * kd:], r, n)), 0), torch.float32)
    lw.lin_a_log = fin(_rows(src.get(a + "A_log", (hv,)), r, n), torch.float32)
    lw.lin_dt_bias = fin(_rows(src.get(a + "dt_bias", (hv,)), r, n), torch.float32)
    lw.lin_norm = fin(src.get(a + "norm.weight", (dv,)))
    lw.lin_out = fin(_cols(src.get(a + "out_proj.weight", (H, vd)), r, n))


def _expert_tensor(src: "TensorSource", m: str, e: int, part: str, shape: tuple[int, ...]) -> torch.Tensor:
    """Weight ``part`` (``gate_proj.weight`` ...) of routed expert ``e``: one tensor per expert (hub layout), or a slice of
    the stacked ``switch_mlp.<part>`` tensor that MLX conversions write."""
    name = f"{m}experts.{e}.{part}"
    if not src.has(name) and src.has(f"{m}experts.gate_up_proj"):
        # checkpoints saved by recent `transformers`: all experts in `experts.gate_up_proj [E, 2F, H]` (gate rows, then up rows)
        # and `experts.down_proj [E, H, F]`
        cache = getattr(src, "_fused", None)
        if cache is None or cache[0] != m:
            cache = (m, src.get(f"{m}experts.gate_up_proj", None), src.get(f"{m}experts.down_proj", None))
            src._fused = cache
        kind = {"gate_proj.weight": 0, "w1.weight": 0, "up_proj.weight": 1, "w3.weight": 1}.get(part, 2)
        if kind == 2:
            return cache[2][e]
        F_ = cache[1].shape[1] // 2
        return cache[1][e, kind * F_:(kind + 1) * F_]
    if src.has(name) or not src.has(f"{m}switch_mlp.{part}"):
        return src.get(name, shape)
    cache = getattr(src, "_stacked", None)
    if cache is None or cache[0] != m:           # the stacked tensors of one layer at a time
        cache = (m, {})
        src._stacked = cache
    if part not in cache[1]:
        cache[1][part] = src.get(f"{m}switch_mlp.{part}", None)
    return cache[1][part][e]



def _mxfp4_blocks(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``blocks [..., K/32, 16]`` bytes of two e2m1 codes each (low nibble first) and ``scales [..., K/32]`` (e8m0) → ``[..., K]``."""
    b = blocks.to(torch.int64)
    codes = torch.stack((b & 0xF, b >> 4), -1).reshape(*blocks.shape[:-1], 32)
    vals = _FP4_E2M1[codes] * torch.exp2(scales.float() - 127.0)[..., None]
    return vals.reshape(*blocks.shape[:-2], -1)


def _gpt_oss_experts(cfg: ModelConfig, spec: ShardSpec, src: "TensorSource", m: str, lw: "LayerWeights", fin) -> None:
    """GPT-OSS sparse block: ``router.{weight,bias}``; ``experts.gate_up_proj [E, H, 2F]`` with gate and up columns interleaved
    (or ``gate_up_proj_blocks`` / ``_scales``: 4-bit e2m1 codes in 32-value blocks with a power-of-two scale, rows first), its
    bias ``[E, 2F]``; ``experts.down_proj [E, F, H]`` (or blocks ``[E, H, F/32, 16]``) and its bias.  Stored here as gate rows then
    up rows ``[E_local, 2F, H]`` and ``[E_local, H, F]``; experts are split over the ranks."""
    E, F, H = cfg.n_experts, cfg.moe_ffn, cfg.hidden
    elo, ehi = expert_range(cfg, spec)
    lw.router = fin(src.get(m + "router.weight", (E, H)))
    lw.router_b = fin(src.get(m + "router.bias", (E,)), torch.float32)
    x = m + "experts."
    if src.has(x + "gate_up_proj_blocks") and not src.has(x + "gate_up_proj"):
        gu = _mxfp4_blocks(src.get(x + "gate_up_proj_blocks", None)[elo:ehi], src.get(x + "gate_up_proj_scales", None)[elo:ehi])      # [e, 2F, H]
        dn = _mxfp4_blocks(src.get(x + "down_proj_blocks", None)[elo:ehi], src.get(x + "down_proj_scales", None)[elo:ehi])            # [e, H, F]
    else:
        gu = src.get(x + "gate_up_proj", (E, H, 2 * F))[elo:ehi].transpose(1, 2)
        dn = src.get(x + "down_proj", (E, F, H))[elo:ehi].transpose(1, 2)
    gb = src.get(x + "gate_up_proj_bias", (E, 2 * F))[elo:ehi]
    lw.e_gate_up = fin(torch.cat((gu[:, 0::2], gu[:, 1::2]), 1))           # de-interleave: gate rows, then up rows
    lw.e_gate_up_b = fin(torch.cat((gb[:, 0::2], gb[:, 1::2]), 1), torch.float32)
    lw.e_down = fin(dn)
    lw.e_down_b = fin(src.get(x + "down_proj_bias", (E, H))[elo:ehi], torch.float32)


def quantize_layer(cfg: ModelConfig, lw: "LayerWeights") -> "LayerWeights":
    """Pack this layer's projection matrices as block-scaled fp8 when the model card is served
    quantised (``cfg.quant``); norms, router, and the absorbed MLA factors stay bf16.  Runs on the
    weights' own device after sharding, one layer at a time, so the bf16 copy of a layer is
    dropped before the next one is read."""
    if cfg.quant == "none":
        return lw
    for name in QUANTIZED_FIELDS:
        w = getattr(lw, name, None)
        if isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16 and w.shape[-1] % 32 == 0:
            setattr(lw, name, quantize(w, cfg.quant))
    return lw


def build_weights(cfg: ModelConfig, spec: ShardSpec, src: TensorSource, device: str | torch.device = "cpu",
                  progress: Callable[[int, int], None] | None = None) -> ModelWeights:
    """Materialise this rank's shard from ``src`` (full tensors are sliced, then dropped)."""
    if cfg.family == "gemma4":
        from .gemma4 import build_gemma4_weights
        return build_gemma4_weights(cfg, spec, src, device, progress)
    if cfg.family == "nemotron_h":
        from .nemotron_h import build_nemotron_h_weights
        return build_nemotron_h_weights(cfg, spec, src, device, progress)
    if cfg.family == "step3p5":
        from .step3p5 import build_step3p5_weights
        return build_step3p5_weights(cfg, spec, src, device, progress)
    dt = _DTYPES[cfg.dtype]
    dev = torch.device(device)
    r, n = spec.tp_rank, spec.tp_size
    H, D = cfg.hidden, cfg.head_dim

    def fin(t: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
        return t.to(device=dev, dtype=dtype or dt).contiguous()

    layers: dict[int, LayerWeights] = {}
    lrange = spec.layers(cfg)
    root = text_model_root(cfg, src)
    # hybrid models: hub checkpoints keep RMSNorm weights zero-centred and the convolution as [C, 1, taps]; MLX
    # conversions have already added the 1 and moved the tap axis
    hf_form = True
    if cfg.has_linear_layers and isinstance(src, SafetensorsSource):
        first = next(i for i in range(cfg.n_layers) if cfg.layer_is_linear(i))
        hf_form = src.index[f"{root}layers.{first}.linear_attn.conv1d.weight"][2][-1] != 1
    one = 1.0 if (cfg.norm_one_plus and hf_form) else 0.0

    def norm(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        t = src.get(name, shape)
        return fin(t.float() + one) if one else fin(t)

    for li, i in enumerate(lrange):
        p = f"{root}layers.{i}."
        lw = LayerWeights(attn_norm=norm(p + "input_layernorm.weight", (H,)),
                          ffn_norm=norm(p + "post_attention_layernorm.weight", (H,)))
        a = p + "self_attn."
        lw.window = cfg.window_of(i)
        if cfg.layer_is_linear(i):
            _linear_attention_weights(cfg, spec, src, p, lw, fin, hf_form)
        elif cfg.mla:
            qk = cfg.qk_nope_dim + cfg.qk_rope_dim
            hl = cfg.n_heads // n
            if cfg.q_lora_rank:
                lw.wq_a = fin(src.get(a + "q_a_proj.weight", (cfg.q_lora_rank, H)))
                lw.q_a_norm = fin(src.get(a + "q_a_layernorm.weight", (cfg.q_lora_rank,)))
                wq_b = src.get(a + "q_b_proj.weight", (cfg.n_heads * qk, cfg.q_lora_rank))
            else:
                wq_b = src.get(a + "q_proj.weight", (cfg.n_heads * qk, H))
            wkv_a = src.get(a + "kv_a_proj_with_mqa.weight", (cfg.kv_lora_rank + cfg.qk_rope_dim, H))
            if cfg.mla_rope_neox:
                # this model turns the rotary dims as (i, i + d/2) pairs; the kernels turn adjacent pairs.  Re-ordering the
                # rotary rows of both projections (row 2i <- i, row 2i + 1 <- i + d/2) makes the two the same rotation, and
                # q . k does not change when both sides are re-ordered alike
                dr = cfg.qk_rope_dim
                perm = torch.stack((torch.arange(dr // 2), torch.arange(dr // 2) + dr // 2), 1).reshape(-1)
                wq_b = wq_b.view(cfg.n_heads, qk, -1).clone()
                wq_b[:, cfg.qk_nope_dim:] = wq_b[:, cfg.qk_nope_dim:][:, perm]
                wq_b = wq_b.view(cfg.n_heads * qk, -1)
                wkv_a = wkv_a.clone()
                wkv_a[cfg.kv_lora_rank:] = wkv_a[cfg.kv_lora_rank:][perm]
            lw.wq_b = fin(_rows(wq_b, r, n))
            lw.wkv_a = fin(wkv_a)
            lw.kv_a_norm = fin(src.get(a + "kv_a_layernorm.weight", (cfg.kv_lora_rank,)))
            wkv_b = src.get(a + "kv_b_proj.weight", (cfg.n_heads * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora_rank))
            wkv_b = wkv_b.view(cfg.n_heads, cfg.qk_nope_dim + cfg.v_head_dim, cfg.kv_lora_rank)[r * hl:(r + 1) * hl]
            lw.w_uk = fin(wkv_b[:, :cfg.qk_nope_dim])
            lw.w_uv = fin(wkv_b[:, cfg.qk_nope_dim:])
            lw.wo = fin(_cols(src.get(a + "o_proj.weight", (H, cfg.n_heads * cfg.v_head_dim)), r, n))
        else:
            klo, khi = kv_head_range(cfg, spec)
            gate_rows: tuple[torch.Tensor, ...] = ()
            if cfg.attn_gate:          # q_proj holds [q, gate] per head: the gate rows go behind v
                qg = src.get(a + "q_proj.weight", (cfg.n_heads * 2 * D, H)).view(cfg.n_heads, 2, D, H)
                wq = _rows(qg[:, 0].reshape(cfg.n_heads * D, H), r, n)
                gate_rows = (_rows(qg[:, 1].reshape(cfg.n_heads * D, H), r, n),)
            else:
                wq = _rows(src.get(a + "q_proj.weight", (cfg.n_heads * D, H)), r, n)
            wk = src.get(a + "k_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
            wv = src.get(a + "v_proj.weight", (cfg.n_kv_heads * D, H))[klo * D:khi * D]
            lw.wqkv = fin(torch.cat((wq, wk, wv) + gate_rows, 0))
            if cfg.attn_bias:
                bq = _rows(src.get(a + "q_proj.bias", (cfg.n_heads * D,)), r, n)
                bk = src.get(a + "k_proj.bias", (cfg.n_kv_heads * D,))[klo * D:khi * D]
                bv = src.get(a + "v_proj.bias", (cfg.n_kv_heads * D,))[klo * D:khi * D]
                lw.bqkv = fin(torch.cat((bq, bk, bv), 0))
            lw.wo = fin(_cols(src.get(a + "o_proj.weight", (H, cfg.n_heads * D)), r, n))
            if cfg.attn_bias and cfg.family == "gpt_oss" and src.has(a + "o_proj.bias"):
                lw.bo = fin(src.get(a + "o_proj.bias", (H,)))
            if cfg.qk_norm:
                lw.q_norm = norm(a + "q_norm.weight", (D,))
                lw.k_norm = norm(a + "k_norm.weight", (D,))
            if cfg.qk_norm_full:      # one weight per output column of q / k: this rank's slice of it
                lw.q_norm = fin(_rows(src.get(a + "q_norm.weight", (cfg.n_heads * D,)), r, n))
                lw.k_norm = fin(src.get(a + "k_norm.weight", (cfg.n_kv_heads * D,))[klo * D:khi * D])
            if cfg.attn_sinks:
                lw.sinks = fin(_rows(src.get(a + "sinks", (cfg.n_heads,)), r, n), torch.float32)
        m = p + moe_names(cfg)["prefix"]
        if cfg.layer_is_moe(i) and not src.has(m + "gate.weight") and src.has(p + "mlp.gate.weight"):
            m = p + "mlp."               # (recent `transformers` saves Mixtral-style blocks under `mlp.` as well)
        if cfg.layer_is_moe(i) and cfg.expert_bias:
            _gpt_oss_experts(cfg, spec, src, m, lw, fin)
        elif cfg.layer_is_moe(i):
            E, F = cfg.n_experts, cfg.moe_ffn
            nm = moe_names(cfg)
            lw.router = fin(src.get(m + "gate.weight", (E, H)))
            if cfg.router_bias and src.has(m + nm["bias"]):      # (DeepSeek-V2 checkpoints have no selection bias)
                lw.router_bias = fin(src.get(m + nm["bias"], (E,)), torch.float32)
            elo, ehi = expert_range(cfg, spec)
            gus, dns = [], []
            for e in range(elo, ehi):
                ep = f"{m}experts.{e}."
                gus.append(torch.cat((_expert_tensor(src, m, e, nm["gate"], (F, H)), _expert_tensor(src, m, e, nm["up"], (F, H))), 0))
                dns.append(_expert_tensor(src, m, e, nm["down"], (H, F)))
            lw.e_gate_up = fin(torch.stack(gus))
            lw.e_down = fin(torch.stack(dns))
            if cfg.n_shared_experts:
                Fs = F * cfg.n_shared_experts
                sp = m + "shared_experts."
                lw.s_gate_up = fin(torch.cat((_rows(src.get(sp + "gate_proj.weight", (Fs, H)), r, n),
                                              _rows(src.get(sp + "up_proj.weight", (Fs, H)), r, n)), 0))
                lw.s_down = fin(_cols(src.get(sp + "down_proj.weight", (H, Fs)), r, n))
            if cfg.shared_expert_ffn:
                Fs, sp = cfg.shared_expert_ffn, m + "shared_expert."
                lw.s_gate_up = fin(torch.cat((_rows(src.get(sp + "gate_proj.weight", (Fs, H)), r, n),
                                              _rows(src.get(sp + "up_proj.weight", (Fs, H)), r, n)), 0))
                lw.s_down = fin(_cols(src.get(sp + "down_proj.weight", (H, Fs)), r, n))
                if cfg.shared_expert_gate:
                    lw.s_gate = fin(src.get(m + "shared_expert_gate.weight", (1, H)))
        else:
            F = cfg.ffn
            lw.w_gate_up = fin(torch.cat((_rows(src.get(m + "gate_proj.weight", (F, H)), r, n),
                                          _rows(src.get(m + "up_proj.weight", (F, H)), r, n)), 0))
            lw.w_down = fin(_cols(src.get(m + "down_proj.weight", (H, F)), r, n))
        layers[i] = quantize_layer(cfg, lw)
        if progress is not None:
            progress(li + 1, len(lrange))
    embed = final_norm = lm_head = None
    if spec.is_first_stage or (cfg.tie_embeddings and spec.is_last_stage):
        embed = fin(src.get(root + "embed_tokens.weight", (cfg.vocab, H)))
    if spec.is_last_stage:
        final_norm = norm(root + "norm.weight", (H,))
        head = next((h for h in ("lm_head.weight", root[:-len("model.")] + "lm_head.weight") if src.has(h)), None) \
            if root.endswith("model.") else ("lm_head.weight" if src.has("lm_head.weight") else None)
        name = root + "embed_tokens.weight" if cfg.tie_embeddings or head is None else head
        full = src.get(name, (cfg.vocab, H))
        vpad = vocab_shard(cfg.vocab, n)
        lm_head = fin(full[min(r * vpad, cfg.vocab):min((r + 1) * vpad, cfg.vocab)])
        if lm_head.shape[0] < vpad:  # last rank pads so that every rank has the same shard height
            lm_head = torch.cat((lm_head, torch.zeros(vpad - lm_head.shape[0], H, dtype=lm_head.dtype, device=dev)), 0)
    return ModelWeights(embed=embed, layers=layers, final_norm=final_norm, lm_head=lm_head)


def fast_random_weights(cfg: ModelConfig, spec: ShardSpec, device: str | torch.device, seed: int = 0,
                        router_std: float | None = None) -> ModelWeights:
    """Random-init directly at shard shapes (benchmarks): never materialises a full tensor.

    Values differ from ``build_weights(RandomSource)`` (each rank draws its own stream), so
    this is for throughput runs where only the shapes and the N(0, 0.02) statistics matter.
    """
    class _Shard(TensorSource):
        def __init__(self) -> None:
            self.g = torch.Generator(device=device)
            self.g.manual_seed(seed * 1000003 + spec.tp_rank * 7919 + spec.pp_rank * 104729)

        def get(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
            if "norm" in name and name.endswith("weight"):
                return torch.ones(shape, dtype=_DTYPES[cfg.dtype], device=device)
            if name.endswith("e_score_correction_bias"):
                return torch.zeros(shape, dtype=torch.float32, device=device)
            std = router_std if (router_std is not None and name.endswith("mlp.gate.weight")) else 0.02
            t = torch.empty(shape, dtype=_DTYPES[cfg.dtype], device=device)
            t.normal_(0.0, std, generator=self.g)
            return t

    return _fast_shard(cfg, spec, _Shard(), device)


def _fast_shard(cfg: ModelConfig, spec: ShardSpec, src: TensorSource, device) -> ModelWeights:
    dt = _DTYPES[cfg.dtype]
    n = spec.tp_size
    H, D = cfg.hidden, cfg.head_dim
    hq, hkv = local_heads(cfg, spec)
    layers: dict[int, LayerWeights] = {}
    for i in spec.layers(cfg):
        p = f"L{i}."
        lw = LayerWeights(attn_norm=torch.ones(H, dtype=dt, device=device), ffn_norm=torch.ones(H, dtype=dt, device=device))
        if cfg.layer_is_linear(i):
            hk, hv = linear_heads(cfg, spec)
            kd, vd = hk * cfg.lin_k_dim, hv * cfg.lin_v_dim
            lw.lin_in = src.get(p + "lin_in", (2 * kd + 2 * vd + 2 * hv, H))
            lw.lin_conv_w = src.get(p + "lin_conv", (2 * kd + vd, cfg.lin_conv)).float() * 10
            lw.lin_a_log = src.get(p + "lin_a", (hv,)).float()
            lw.lin_dt_bias = src.get(p + "lin_dt", (hv,)).float()
            lw.lin_norm = torch.ones(cfg.lin_v_dim, dtype=dt, device=device)
            lw.lin_out = src.get(p + "lin_out", (H, vd))
        elif cfg.mla:
            qk = cfg.qk_nope_dim + cfg.qk_rope_dim
            if cfg.q_lora_rank:
                lw.wq_a = src.get(p + "qa", (cfg.q_lora_rank, H))
                lw.q_a_norm = torch.ones(cfg.q_lora_rank, dtype=dt, device=device)
                lw.wq_b = src.get(p + "qb", (hq * qk, cfg.q_lora_rank))
            else:
                lw.wq_b = src.get(p + "qb", (hq * qk, H))
            lw.wkv_a = src.get(p + "kva", (cfg.kv_lora_rank + cfg.qk_rope_dim, H))
            lw.kv_a_norm = torch.ones(cfg.kv_lora_rank, dtype=dt, device=device)
            lw.w_uk = src.get(p + "uk", (hq, cfg.qk_nope_dim, cfg.kv_lora_rank))
            lw.w_uv = src.get(p + "uv", (hq, cfg.v_head_dim, cfg.kv_lora_rank))
            lw.wo = src.get(p + "o", (H, hq * cfg.v_head_dim))
        else:
            hq = cfg.q_heads(i) // n
            lw.wqkv = src.get(p + "qkv", ((hq + 2 * hkv + (hq if cfg.attn_gate else 0)) * D, H))
            lw.wo = src.get(p + "o", (H, hq * D))
            if cfg.family == "step3p5":      # per-layer head count, RoPE, window, head gate and SwiGLU limits
                from ..ops import reference as ref
                lw.n_q, lw.window = hq, cfg.window_of(i)
                inv, lw.rope_mscale = ref.rope_inv_freq(D, cfg.rope_of(i))
                lw.inv_freq = inv.to(device)
                if cfg.head_gate:
                    lw.w_head_gate = src.get(p + "hg", (hq, H))
                lw.act_limit, lw.shared_limit = cfg.swiglu_limit(i), cfg.swiglu_limit(i, shared=True)
            if cfg.qk_norm:
                lw.q_norm = torch.ones(D, dtype=dt, device=device)
                lw.k_norm = torch.ones(D, dtype=dt, device=device)
            if cfg.qk_norm_full:
                hq, hkv = local_heads(cfg, spec)
                lw.q_norm = torch.ones(hq * D, dtype=dt, device=device)
                lw.k_norm = torch.ones(hkv * D, dtype=dt, device=device)
        if cfg.layer_is_moe(i):
            E, F = cfg.n_experts, cfg.moe_ffn
            el = E // n
            lw.router = src.get("model.layers.%d.mlp.gate.weight" % i, (E, H))
            if cfg.router_bias:
                lw.router_bias = torch.zeros(E, dtype=torch.float32, device=device)
            lw.e_gate_up = src.get(p + "egu", (el, 2 * F, H))
            lw.e_down = src.get(p + "ed", (el, H, F))
            if cfg.n_shared_experts or cfg.shared_expert_ffn:
                Fs = (F * cfg.n_shared_experts or cfg.shared_expert_ffn) // n
                lw.s_gate_up = src.get(p + "sgu", (2 * Fs, H))
                lw.s_down = src.get(p + "sd", (H, Fs))
                if cfg.shared_expert_gate:
                    lw.s_gate = src.get(p + "sg", (1, H))
        else:
            lw.w_gate_up = src.get(p + "gu", (2 * cfg.ffn // n, H))
            lw.w_down = src.get(p + "d", (H, cfg.ffn // n))
        layers[i] = quantize_layer(cfg, lw)
    embed = src.get("embed", (cfg.vocab, H)) if spec.is_first_stage else None
    final_norm = torch.ones(H, dtype=dt, device=device) if spec.is_last_stage else None
    lm_head = src.get("lm_head", (vocab_shard(cfg.vocab, n), H)) if spec.is_last_stage else None
    return ModelWeights(embed, layers, final_norm, lm_head)
