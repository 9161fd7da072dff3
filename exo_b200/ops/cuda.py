"""ctypes binding of ``_kernels.so`` (the sm_100a kernel library).

Launchers take raw device pointers and the current CUDA stream, so every call is graph
capturable and costs one ctypes dispatch.  Tensors are allocated by the caller's framework
(PyTorch) — the kernels themselves never allocate.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

from . import reference as ref
from .quant import Fp8Weight

_lib: C.CDLL | None = None
_SO = Path(os.environ.get("EXO_KERNELS_SO") or Path(__file__).resolve().parent / "_kernels.so")     # override: A/B runs of two builds

BF16, F32 = 0, 1
_DT = {torch.bfloat16: BF16, torch.float32: F32}


class KernelError(RuntimeError):
    pass


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            raise KernelError(f"{_SO} is missing: run `python -m exo_b200.build` (CUDA ops have no fallback)")
        _lib = C.CDLL(str(_SO))
        for name in dir(_Sig):
            if name.startswith("exo_"):
                fn = getattr(_lib, name)
                fn.restype, fn.argtypes = getattr(_Sig, name)
    return _lib


_p, _i, _f, _l = C.c_void_p, C.c_int, C.c_float, C.c_long


class _Sig:
    exo_rmsnorm = (_i, [_p, _p, _p, _p, _p, _i, _i, _f, _i, _p])
    exo_swiglu = (_i, [_p, _p, _i, _i, _i, _p])
    exo_swiglu_clamp = (_i, [_p, _p, _i, _i, _f, _i, _p])
    exo_moe_experts_gemv_fp8 = (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p])
    exo_gated_delta = (_i, [_p, _i, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _i, _p, _p, _i, _p])
    exo_sigmoid_gate = (_i, [_p, _p, _i, _p, _i, _i, _i, _p])
    exo_scaled_add = (_i, [_p, _p, _p, _p, _i, _i, _i, _p])
    exo_embedding = (_i, [_p, _p, _p, _i, _i, _i, _i, _p])
    exo_qk_rope_append = (_i, [_p, _p, _p, _f, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _p])
    exo_geglu = (_i, [_p, _p, _i, _i, _i, _p])
    exo_argmax_chunks = (_i, [_i, _i])
    exo_argmax = (_i, [_p, _p, _p, _p, _i, _i, _i, _l, _i, _p])
    exo_sample = (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _l, _i, _p])
    exo_decode_mega_variant = (_i, [_i, _i, _i, _i, _i, _i])
    exo_decode_mega_workspace = (_l, [_i, _i, _i, _i])
    exo_decode_mega = (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _f, _f, _f, _i, _i, _i, _i, _i, _i, _i,
                            _i, _p, _p])
    exo_sample_workspace = (_l, [_i])
    exo_sample_fast = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _l, _i, _p])
    exo_paged_decode_workspace = (_l, [_i, _i, _i, _i])
    exo_paged_decode_splits = (_i, [_i, _i, _i])
    exo_paged_decode = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p])
    exo_token_seq = (_i, [_p, _p, _i, _p])
    exo_paged_ragged = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p])
    exo_prefill_attn_tc = (_i, [_p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p])
    exo_decode_attn_tc = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p])
    exo_decode_attn_tc_splits = (_i, [_i, _i, _i])
    exo_decode_attn_tc_workspace = (_l, [_i, _i, _i])
    exo_linear_small = (_i, [_p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _p])
    exo_linear_tiled = (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p])
    exo_gemv_stream_init = (_i, [])
    exo_gemv_stream_last_error = (_i, [])
    exo_gemv_stream_supported = (_i, [_i, _i, _i, _i])
    exo_gemv_stream = (_i, [_p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _p])
    exo_gemm_init = (_i, [_l])
    exo_gemm_last_error = (_i, [])
    exo_gemm_splits = (_i, [_i, _i, _i])
    exo_gemm_bf16 = (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p])
    exo_gemm_bf16_swiglu = (_i, [_p, _p, _p, _i, _i, _i, _p])
    exo_gemm_bf16_gated = (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p])
    exo_gemm_bf16_swiglu_gated = (_i, [_p, _p, _p, _i, _i, _i, _i, _p])
    exo_gemm_fp8w = (_i, [_p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _p])
    exo_gemm_fp8w_f16 = (_i, [_p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _p])
    exo_bf16_to_f16 = (_i, [_p, _p, _l, _p])
    exo_mla_attn_splits = (_i, [_i, _i])
    exo_mla_attn_workspace = (_l, [_i, _i, _i])
    exo_mla_attn_tc = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _p])
    exo_mla_kv_append = (_i, [_p, _p, _f, _p, _p, _f, _p, _p, _i, _i, _i, _p])
    exo_mla_q_absorb = (_i, [_p, _p, _p, _p, _f, _p, _i, _i, _i, _i, _i, _i, _p])
    exo_mla_o_absorb = (_i, [_p, _p, _p, _i, _i, _i, _i, _p])
    exo_moe_route = (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p])
    exo_moe_tile_rows = (_i, [_i, _i])
    exo_moe_max_tiles = (_i, [_i, _i, _i])
    exo_moe_plan_ints = (_l, [_i, _i])
    exo_moe_experts_grouped = (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p])
    exo_moe_experts_gemv = (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p])


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _chk(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}" + (" (unsupported shape/dtype)" if rc == -2 else "")
                          + (f": {torch.cuda.get_device_name()}" if rc > 0 else ""))


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


launch_count = 0  # launches issued through this module (read by the benchmark)

# ---- EXO_KERNEL_CHECKS=1: the stand-in for a memory checker ----------------------------------------------------------
# Outputs are allocated with a guard band behind them that is filled with a pattern before the launch and verified
# after it (an out-of-bounds store of a kernel shows up as a broken band, attributed to the op that made it), index
# tensors that kernels dereference unchecked (KV slots, block tables, token ids) are validated on the host, and the
# kernel library, when it was built with the same variable set, waits for every kernel and reports its fault as the
# launcher's return code.  Every check synchronises: this is a debugging flavour, never on in serving or benchmarks.
CHECKS = os.environ.get("EXO_KERNEL_CHECKS") == "1"
_GUARD = 256          # guard elements behind every output
_guards: list[tuple[torch.Tensor, int, str]] = []


def _empty(*shape, dtype, device, what: str = "output") -> torch.Tensor:
    if not CHECKS:
        return torch.empty(*shape, dtype=dtype, device=device)
    shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else tuple(shape)
    n = 1
    for d in shape:
        n *= int(d)
    flat = torch.empty(n + _GUARD, dtype=dtype, device=device)
    flat[n:].view(torch.uint8).fill_(0xA5)
    _guards.append((flat, n, what))
    return flat[:n].view(shape)


def _empty_like(x: torch.Tensor, what: str = "output") -> torch.Tensor:
    return _empty(tuple(x.shape), dtype=x.dtype, device=x.device, what=what) if CHECKS else torch.empty_like(x)


def verify_guards() -> None:
    """Raise if any kernel since the last call wrote behind the end of one of its outputs (checks mode only)."""
    if not _guards:
        return
    torch.cuda.synchronize()
    bad = [what for flat, n, what in _guards if not bool((flat[n:].view(torch.uint8) == 0xA5).all())]
    _guards.clear()
    if bad:
        raise KernelError(f"guard band behind {bad[0]} was overwritten: a kernel stored out of bounds")


def _check_indices(what: str, idx: torch.Tensor, limit: int) -> None:
    """Checks mode: every entry of an index tensor a kernel dereferences must lie in ``[0, limit)``."""
    if CHECKS and idx.numel():
        lo, hi = int(idx.min()), int(idx.max())
        if lo < 0 or hi >= limit:
            raise KernelError(f"{what}: index range [{lo}, {hi}] outside [0, {limit})")


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ------------------------------------------------------------------------------------------
def rmsnorm(x, w, eps, residual=None):
    x = x.contiguous()
    out = _empty_like(x, "rmsnorm out")
    h = _empty_like(x, "rmsnorm h") if residual is not None else x
    _chk(load().exo_rmsnorm(_ptr(x), _ptr(residual), _ptr(w), _ptr(out), _ptr(h) if residual is not None else None,
                            x.shape[0], x.shape[1], eps, _dt(x), _st()), "rmsnorm")
    _count()
    return out, h


def swiglu(gate_up, limit=0.0):
    gate_up = gate_up.contiguous()
    rows, F2 = gate_up.shape
    out = torch.empty(rows, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    if limit:
        _chk(load().exo_swiglu_clamp(_ptr(gate_up), _ptr(out), rows, F2 // 2, float(limit), _dt(gate_up), _st()), "swiglu_clamp")
    else:
        _chk(load().exo_swiglu(_ptr(gate_up), _ptr(out), rows, F2 // 2, _dt(gate_up), _st()), "swiglu")
    _count()
    return out


def gated_delta(proj, conv_w, a_log, dt_bias, norm_w, eps, conv_state, rec_state, seats, cu_q, positions, hk, hv, dk, dv):
    """Convolution + gated delta rule + gated norm of one linear-attention layer (three launches, no host reads)."""
    proj = proj.contiguous()
    T, ld = proj.shape
    B = cu_q.numel() - 1
    C = 2 * hk * dk + hv * dv
    if ld != C + hv * dv + 2 * hv or conv_state.dtype != proj.dtype or rec_state.dtype != torch.float32:
        raise KernelError(f"gated_delta: projection width {ld} / state dtypes do not fit hk={hk} hv={hv} dk={dk} dv={dv}")
    if CHECKS:
        _check_indices("state seats", seats, rec_state.shape[0])
    y = _empty(T, C, dtype=proj.dtype, device=proj.device, what="gated_delta conv")
    out = _empty(T, hv * dv, dtype=proj.dtype, device=proj.device, what="gated_delta out")
    _chk(load().exo_gated_delta(_ptr(proj), ld, _ptr(conv_w), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w), float(eps),
                                _ptr(conv_state), _ptr(rec_state), _ptr(seats), _ptr(cu_q), _ptr(positions), T, B, hk, hv,
                                dk, dv, conv_w.shape[1], _ptr(y), _ptr(out), _dt(proj), 0, None, None, 0, _st()), "gated_delta")
    _count(3)          # (a fourth, the output norm, when a small grid has its heads split by columns)
    return out


def mamba2(proj, conv_w, conv_b, a_log, dt_bias, skip, norm_w, eps, conv_state, ssm_state, seats, cu_q, positions, groups, heads,
           d_state, head_dim):
    """Mamba-2 mixer between its projections (columns C | B | x | z | dt | dt): the gated-delta-rule kernels in their
    state-space mode plus the grouped gated norm (four launches, no host reads)."""
    proj = proj.contiguous()
    T, ld = proj.shape
    B = cu_q.numel() - 1
    C = 2 * groups * d_state + heads * head_dim
    if ld != C + heads * head_dim + 2 * heads or conv_state.dtype != proj.dtype or ssm_state.dtype != torch.float32:
        raise KernelError(f"mamba2: projection width {ld} / state dtypes do not fit groups={groups} heads={heads}")
    if CHECKS:
        _check_indices("state seats", seats, ssm_state.shape[0])
    y = _empty(T, C, dtype=proj.dtype, device=proj.device, what="mamba2 conv")
    out = _empty(T, heads * head_dim, dtype=proj.dtype, device=proj.device, what="mamba2 out")
    gsize = heads * head_dim // groups
    _chk(load().exo_gated_delta(_ptr(proj), ld, _ptr(conv_w), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w), float(eps),
                                _ptr(conv_state), _ptr(ssm_state), _ptr(seats), _ptr(cu_q), _ptr(positions), T, B, groups, heads,
                                d_state, head_dim, conv_w.shape[1], _ptr(y), _ptr(out), _dt(proj), 1, _ptr(conv_b), _ptr(skip),
                                gsize, _st()), "mamba2")
    _count(4)
    return out


def sigmoid_gate(x, gate):
    x = x.contiguous()
    rows, n = x.shape
    if gate.stride(-1) != 1 or gate.shape != x.shape:
        gate = gate.contiguous()
    out = _empty_like(x, "sigmoid_gate out")
    _chk(load().exo_sigmoid_gate(_ptr(x), _ptr(gate), gate.stride(0), _ptr(out), rows, n, _dt(x), _st()), "sigmoid_gate")
    _count()
    return out


def scaled_add(y, x, logit):
    y, x, logit = y.contiguous(), x.contiguous(), logit.contiguous()
    rows, n = x.shape
    out = _empty_like(x, "scaled_add out")
    _chk(load().exo_scaled_add(_ptr(y), _ptr(x), _ptr(logit), _ptr(out), rows, n, _dt(x), _st()), "scaled_add")
    _count()
    return out


def geglu(gate_up):
    gate_up = gate_up.contiguous()
    rows, F2 = gate_up.shape
    out = torch.empty(rows, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _chk(load().exo_geglu(_ptr(gate_up), _ptr(out), rows, F2 // 2, _dt(gate_up), _st()), "geglu")
    _count()
    return out


def embedding(table, ids):
    ids = ids.to(torch.int32)
    _check_indices("embedding token ids", ids, table.shape[0])
    out = _empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device, what="embedding out")
    _chk(load().exo_embedding(_ptr(table), _ptr(ids), _ptr(out), ids.numel(), table.shape[1], table.shape[0],
                              _dt(table), _st()), "embedding")
    _count()
    return out


SMALL_M = 2   # rows served by CUDA-core kernels; above that the tensor-core GEMM streams weights better
_stream_ready: set[int] = set()
use_stream_gemv = os.environ.get("EXO_DISABLE_STREAM_GEMV") != "1"
GEMM_PARTIAL_FLOATS = 16 << 20
_gemm_ready: set[int] = set()


def ensure_gemm_init(device) -> None:
    """Per-device scratch of the tensor-core kernels (error word, split-K buffers); not capturable."""
    dev = device.index or 0
    if dev not in _gemm_ready:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("first tensor-core kernel call on a device must not be inside graph capture")
        _chk(load().exo_gemm_init(GEMM_PARTIAL_FLOATS), "gemm_init")
        _gemm_ready.add(dev)


def gated_gemm_ok(M: int, N: int, K: int, swiglu_out: bool) -> bool:
    """Shapes for which :func:`gemm_bf16` accepts ``gate_parity`` (the all-gather -> GEMM form)."""
    return (gemm_impl is not None and M >= 256 and K >= 64 and K % 8 == 0
            and (not swiglu_out or (N % 2 == 0 and use_fused_swiglu)))


def gemm_bf16(x, w, bias=None, residual=None, swiglu_out=False, out=None, gate_parity=None):
    """tcgen05 GEMM ``x[M,K] @ w[N,K].T``; per-device scratch is set up on first use, which
    must therefore happen outside CUDA-graph capture (the executor warms up before capturing).

    ``gate_parity``: ``x`` is the broadcast output of a deferred-wait two-shot reduction on that parity
    (``parallel.fused``): each CTA waits for the flag of the rank that owns its activation rows before loading them,
    so the GEMM starts on the rows that are there while the others are still crossing NVLink (all-gather -> GEMM)."""
    lib = load()
    ensure_gemm_init(x.device)
    M, K = x.shape
    N = w.shape[0]
    if swiglu_out and M >= 256 and bias is None and residual is None and N % 2 == 0 and use_fused_swiglu:
        # prefill: gate and up tiles share a CTA and the activation is applied in the epilogue
        out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
        if gate_parity is not None:
            _chk(lib.exo_gemm_bf16_swiglu_gated(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(gate_parity), _st()),
                 "gemm_bf16_swiglu_gated")
        else:
            _chk(lib.exo_gemm_bf16_swiglu(_ptr(x), _ptr(w), _ptr(out), M, N, K, _st()), "gemm_bf16_swiglu")
        _count()
        return out
    if gate_parity is not None:
        if swiglu_out or M < 256:
            raise KernelError("gated GEMM takes prefill shapes (M >= 256) and, with SwiGLU, the fused epilogue")
        if out is None:
            out = torch.empty(M, N, dtype=x.dtype, device=x.device)
        _chk(lib.exo_gemm_bf16_gated(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, N, int(gate_parity),
                                     _st()), "gemm_bf16_gated")
        _count()
        return out
    if out is None or swiglu_out:
        out = _empty(M, N, dtype=x.dtype, device=x.device, what="gemm out")
    splits = lib.exo_gemm_splits(M, N, K)
    while splits > 1 and splits * M * N > GEMM_PARTIAL_FLOATS:
        splits -= 1
    _chk(lib.exo_gemm_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, N, splits, _st()),
         "gemm_bf16")
    _count()
    return swiglu(out) if swiglu_out else out


def linear_fp8(x, w, bias=None, residual=None, norm_w=None, eps=0.0, swiglu_out=False, out=None):
    """Block-scaled fp8 weights, bf16 activations: the weights cross HBM as bytes and are widened to
    bf16 inside the tcgen05 GEMM's pipeline (every batch size; the norm is a separate kernel)."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16:
        raise KernelError("fp8 weights are served with bf16 activations")
    if norm_w is not None:
        x, _ = rmsnorm(x, norm_w, eps)
    if out is None or swiglu_out:
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if M == 0:
        return swiglu(out) if swiglu_out else out
    ensure_gemm_init(x.device)
    lib = load()
    splits = lib.exo_gemm_splits(M, N, K)
    while splits > 1 and splits * M * N > GEMM_PARTIAL_FLOATS:
        splits -= 1
    kind = 1 if w.kind == "mxfp8" else 2
    if fp8_f16_operands and K % 8 == 0 and N * K >= FP8_F16_MIN_WEIGHTS:
        # f16 on both sides of the MMA: the activations are converted once (saturating), the weights with the hardware
        # e4m3 -> f16 converter inside the GEMM
        x16 = torch.empty(M, K, dtype=torch.float16, device=x.device)
        _chk(lib.exo_bf16_to_f16(_ptr(x), _ptr(x16), M * K, _st()), "bf16_to_f16")
        _chk(lib.exo_gemm_fp8w_f16(_ptr(x16), _ptr(w.to_tiled().tiles), kind, _ptr(bias), _ptr(residual),
                                   _ptr(out), M, N, K, N, splits, _st()), "gemm_fp8w_f16")
        _count(2)
    else:
        _chk(lib.exo_gemm_fp8w(_ptr(x), _ptr(w.to_tiled().tiles), kind, _ptr(bias), _ptr(residual),
                               _ptr(out), M, N, K, N, splits, _st()), "gemm_fp8w")
        _count()
    return swiglu(out) if swiglu_out else out


def gemm_check() -> None:
    """Raise if any tensor-core or streaming kernel since the last check recorded a wait that ran out.  The status
    words live in host-mapped memory: this reads them without touching the device, so the kernels of interest
    must have completed (the caller has just read back the step's results)."""
    code = load().exo_gemm_last_error()
    if code:
        raise KernelError(f"tcgen05 GEMM reported device-side timeout code {code}")
    code = load().exo_gemv_stream_last_error()
    if code:
        raise KernelError(f"streaming GEMV reported device-side timeout code {code}")


class DeviceWaitTimeout(KernelError):
    """A bounded wait on a peer GPU ran out inside a collective kernel (status word 2)."""


_status_words: dict[int, "C.Array"] = {}


def check_status(device=None) -> None:
    """Raise if any kernel of the library recorded an expired wait since the last call.

    The three status words (tensor-core kernels, streaming GEMV, peer-memory collectives) sit in pinned host
    memory that the GPU writes directly, so this is three host loads: the serving loop calls it after every
    step, right after the sampled ids have been read back (the step's kernels have then completed)."""
    dev = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    words = _status_words.get(dev)
    if words is None:
        lib = load()
        lib.exo_status_host_ptr.restype = C.c_void_p
        lib.exo_status_host_ptr.argtypes = []
        with torch.cuda.device(dev):
            ptr = lib.exo_status_host_ptr()
        if not ptr:
            raise KernelError("cannot allocate the device status block")
        words = _status_words[dev] = (C.c_int * 4).from_address(ptr)
    tc, gemv, comm = words[0], words[1], words[2]
    if not (tc or gemv or comm):
        return
    words[0] = words[1] = words[2] = 0
    if comm:
        raise DeviceWaitTimeout(f"cuda:{dev}: a collective kernel gave up waiting for a peer GPU (code {comm})")
    raise KernelError(f"cuda:{dev}: a kernel's pipeline wait ran out (tensor-core code {tc}, streaming GEMV code {gemv})")


gemm_impl = None if os.environ.get("EXO_DISABLE_TCGEN05") == "1" else gemm_bf16
use_fused_swiglu = os.environ.get("EXO_DISABLE_FUSED_SWIGLU") != "1"
# below this many weights a projection is bound by its launch and split-K costs, and the extra activation-conversion
# launch of the f16 form costs more than the cheaper widening saves (measured: 6144x4096 13.3 -> 12.8 us, 70B TP8 slower)
FP8_F16_MIN_WEIGHTS = 48 << 20
fp8_f16_operands = os.environ.get("EXO_FP8_F16_OPERANDS", "1") == "1"     # 0: bf16 operands (five instead of two widening instructions per pair)


def ensure_stream_init(device) -> None:
    dev = device.index or 0
    if dev not in _stream_ready:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("first streaming-GEMV call on a device must not be inside graph capture")
        _chk(load().exo_gemv_stream_init(), "gemv_stream_init")
        _stream_ready.add(dev)


def linear(x, w, bias=None, residual=None, norm_w=None, eps=0.0, swiglu_out=False, out=None):
    """Dispatch by batch rows: M <= 2 → streaming GEMV; bf16 larger M → tcgen05 GEMM; fp32 larger M → CUDA-core
    tiled kernel (oracle configs only).  ``out`` (contiguous ``[M, N]``, no SwiGLU) receives the result where the
    kernel can write it directly, else it is copied there."""
    if out is not None:
        M, N = x.shape[0], w.shape[0]
        direct = (not swiglu_out and out.is_contiguous() and M > SMALL_M
                  and (isinstance(w, Fp8Weight) or (x.dtype == torch.bfloat16 and gemm_impl is not None and norm_w is None
                                                    and x.shape[1] >= 64 and x.shape[1] % 8 == 0)))
        if not direct:
            out.copy_(linear(x, w, bias, residual, norm_w, eps, swiglu_out))
            return out
    x = x.contiguous()
    M, K = x.shape
    N = w.shape[0]
    lib = load()
    if isinstance(w, Fp8Weight):
        return linear_fp8(x, w, bias, residual, norm_w, eps, swiglu_out, out)
    if (use_stream_gemv and 0 < M <= 2 and x.dtype == torch.bfloat16
            and lib.exo_gemv_stream_supported(M, N, K, int(swiglu_out))):
        ensure_stream_init(x.device)
        out = torch.empty(M, N // 2 if swiglu_out else N, dtype=x.dtype, device=x.device)
        _chk(lib.exo_gemv_stream(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), _ptr(norm_w), eps, M, N, K,
                                 int(swiglu_out), _st()), "gemv_stream")
        _count()
        return out
    if M <= SMALL_M or (x.dtype != torch.bfloat16 and M <= 8):
        out = torch.empty(M, N // 2 if swiglu_out else N, dtype=x.dtype, device=x.device)
        if M:
            _chk(lib.exo_linear_small(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), _ptr(norm_w), eps, M, N,
                                      K, int(swiglu_out), _dt(x), _st()), "linear_small")
            _count()
        return out
    if norm_w is not None:
        x, _ = rmsnorm(x, norm_w, eps)
    if x.dtype == torch.bfloat16 and gemm_impl is not None and K >= 64 and K % 8 == 0:
        return gemm_impl(x, w, bias, residual, swiglu_out, out)
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    _chk(lib.exo_linear_tiled(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, _dt(x), _st()),
         "linear_tiled")
    _count()
    return swiglu(out) if swiglu_out else out


def qk_rope_append(qkv, positions, inv_freq, mscale, n_q, n_kv, head_dim, kcache, vcache, slots, q_norm=None,
                   k_norm=None, eps=1e-6, v_unit_norm=False):
    qkv = qkv.contiguous()
    T = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qk_rope_append: {qkv.shape[1]} columns for {n_q} + 2 x {n_kv} heads of {head_dim}")
    if n_kv:
        _check_indices("KV slots", slots, kcache.shape[0] * kcache.shape[1])
    q = _empty(T, n_q, head_dim, dtype=qkv.dtype, device=qkv.device, what="rope q")
    rot = inv_freq.numel() * 2
    _chk(load().exo_qk_rope_append(_ptr(qkv), _ptr(positions), _ptr(inv_freq), float(mscale), n_q, n_kv, head_dim, rot,
                                   _ptr(q), _ptr(kcache), _ptr(vcache), _ptr(slots), _ptr(q_norm), _ptr(k_norm),
                                   float(eps), T, _dt(qkv), int(bool(v_unit_norm)), _st()), "qk_rope_append")
    _count()
    return q


_ws: dict[tuple, torch.Tensor] = {}
_tickets: dict[int | None, torch.Tensor] = {}


def _workspace(dev: torch.device, n_floats: int) -> torch.Tensor:
    key = (dev.index,)
    t = _ws.get(key)
    if t is None or t.numel() < n_floats:
        t = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=dev)
        _ws[key] = t
    return t


# tensor-core prefill attention (head_dim 128, 16-key pages, bf16); EXO_DISABLE_TC_ATTENTION=1 forces the generic kernel
prefill_attention_impl = None if os.environ.get("EXO_DISABLE_TC_ATTENTION") == "1" else "tcgen05"
decode_attention_tc = os.environ.get("EXO_DISABLE_TC_DECODE") != "1"


def paged_attention(q, kcache, vcache, block_tables, seq_lens, cu_q, scale, sliding_window=0, sinks=None,
                    max_q_len=None):
    lib = load()
    q = q.contiguous()
    T, Hq, D = q.shape
    nblk, bs, Hkv, _ = kcache.shape
    B = seq_lens.numel()
    out = _empty_like(q, "attention out")
    max_blocks = block_tables.shape[1]
    if CHECKS:
        _check_indices("block tables", block_tables, nblk)
        _check_indices("sequence lengths", seq_lens, max_blocks * bs + 1)
    if max_q_len == 1 and T == B:
        tk = _tickets.get(q.device.index)
        if tk is None or tk.numel() < B * Hq:
            tk = _tickets[q.device.index] = torch.zeros(max(B * Hq, 1 << 14), dtype=torch.int32, device=q.device)
        if (prefill_attention_impl is not None and decode_attention_tc and q.dtype == torch.bfloat16 and sinks is None
                and D == 128 and bs == 16 and Hq % Hkv == 0 and Hq // Hkv in (1, 2, 4, 8)):
            ensure_gemm_init(q.device)
            ns = lib.exo_decode_attn_tc_splits(B, Hkv, max_blocks * bs)
            ws = _workspace(q.device, lib.exo_decode_attn_tc_workspace(B, Hq, ns))
            _chk(lib.exo_decode_attn_tc(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(seq_lens), _ptr(out),
                                        _ptr(ws), _ptr(tk), float(scale), B, Hq, Hkv, D, nblk, max_blocks, bs, ns,
                                        int(sliding_window), _st()), "decode_attn_tc")
            _count()
            return out
        ns = lib.exo_paged_decode_splits(B, Hkv, max_blocks * bs)
        ws = _workspace(q.device, lib.exo_paged_decode_workspace(B, Hq, D, ns))
        _chk(lib.exo_paged_decode(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(seq_lens), _ptr(out),
                                  _ptr(ws), _ptr(tk), float(scale), B, Hq, Hkv, D, max_blocks, bs, ns,
                                  int(sliding_window), _ptr(sinks), _dt(q), _st()), "paged_decode")
        _count()
        return out
    if prefill_attention_impl is not None and q.dtype == torch.bfloat16 and sinks is None and D == 128 and bs == 16:
        ensure_gemm_init(q.device)
        rc = lib.exo_prefill_attn_tc(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(seq_lens), _ptr(cu_q),
                                     _ptr(out), float(scale), T, B, Hq, Hkv, D, nblk, max_blocks, bs, int(sliding_window),
                                     _st())
        if rc == 0:
            _count()
            return out
        if rc not in (-2, -5):      # -2 / -5: shape not handled there -> generic kernel below
            _chk(rc, "prefill_attn_tc")
    tok_seq = torch.empty(T, dtype=torch.int32, device=q.device)
    _chk(lib.exo_token_seq(_ptr(cu_q), _ptr(tok_seq), B, _st()), "token_seq")
    _chk(lib.exo_paged_ragged(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(seq_lens), _ptr(cu_q),
                              _ptr(tok_seq), _ptr(out), float(scale), T, Hq, Hkv, D, max_blocks, bs,
                              int(sliding_window), _ptr(sinks), _dt(q), _st()), "paged_ragged")
    _count(2)
    return out


def argmax(logits):
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = load()
    chunks = lib.exo_argmax_chunks(rows, V)
    pv = torch.empty(rows * chunks, dtype=torch.float32, device=logits.device)
    pi = torch.empty(rows * chunks, dtype=torch.int32, device=logits.device)
    _chk(lib.exo_argmax(_ptr(logits), _ptr(out), _ptr(pv), _ptr(pi), chunks, rows, V, logits.stride(0), _dt(logits),
                        _st()), "argmax")
    _count(2)
    return out


# ---- whole-step decode kernel (batch 1, dense models, one GPU) -----------------------------------------------------
# Off unless asked for: on Llama-3.1-8B the one-kernel step measured slower than the per-op path (the five dependent phases
# of a layer each stall the weight stream for a few microseconds, which the per-op kernels overlap through PDL).
use_decode_mega = os.environ.get("EXO_DECODE_MEGA") == "1"


class DecodeMega:
    """Device-side tables and scratch of ``exo_decode_mega`` for one model shard: built once, reused every step."""

    FIELDS = ("wqkv", "bqkv", "wo", "w_gate_up", "w_down", "attn_norm", "ffn_norm", "q_norm", "k_norm")

    def __init__(self, cfg, layers, kv_layers, embed, final_norm, lm_head, n_q, n_kv, device):
        lib = load()
        rows = []
        self.keep = []
        for lw, (kc, vc) in zip(layers, kv_layers):
            ptrs = []
            for f in self.FIELDS:
                t = getattr(lw, f, None)
                ptrs.append(0 if t is None else t.data_ptr())
                if t is not None and not t.is_contiguous():
                    raise ValueError(f"{f} must be contiguous")
            rows.append(ptrs + [kc.data_ptr(), vc.data_ptr()])
            self.keep.append((lw, kc, vc))
        self.table = torch.tensor(rows, dtype=torch.int64).to(device)
        self.n_layers = len(rows)
        H, F = cfg.hidden, lw.w_down.shape[1]
        self.H, self.F, self.n_q, self.n_kv, self.D = H, F, n_q, n_kv, cfg.head_dim
        self.embed, self.final_norm, self.lm_head, self.vocab = embed, final_norm, lm_head, lm_head.shape[0]
        self.ws = torch.zeros(int(lib.exo_decode_mega_workspace(H, F, n_q, n_kv)), dtype=torch.uint8, device=device)
        self.block_size = kv_layers[0][0].shape[1]
        self.n_sm = torch.cuda.get_device_properties(device).multi_processor_count
        self.trace = (torch.zeros(148 * 1024, dtype=torch.int64, device=device)
                      if os.environ.get("EXO_DECODE_MEGA_TRACE") == "1" else None)

    @staticmethod
    def supported(cfg, layers, n_q, n_kv, inv_freq) -> bool:
        if not use_decode_mega or not layers:
            return False
        lw = layers[0]
        plain = all(isinstance(getattr(l, f, None), torch.Tensor) and getattr(l, f).dtype == torch.bfloat16
                    for l in layers for f in ("wqkv", "wo", "w_gate_up", "w_down"))
        if not plain:
            return False
        F = lw.w_down.shape[1]
        return bool(load().exo_decode_mega_variant(cfg.hidden, F, n_q, n_kv, cfg.head_dim, inv_freq.numel() * 2))

    def __call__(self, tokens, positions, slots, block_table, seq_lens, inv_freq, mscale, eps, scale):
        """One decode step from the token id ``tokens [1]`` (int32) to ``logits [1, vocab]``."""
        logits = torch.empty(1, self.vocab, dtype=torch.bfloat16, device=tokens.device)
        _chk(load().exo_decode_mega(_ptr(self.table), self.n_layers, _ptr(self.embed), _ptr(tokens), _ptr(self.final_norm),
                                    _ptr(self.lm_head), _ptr(logits), self.vocab, _ptr(self.ws), _ptr(positions), _ptr(slots),
                                    _ptr(block_table), _ptr(seq_lens), _ptr(inv_freq), float(mscale), float(eps),
                                    float(scale), inv_freq.numel() * 2, self.H, self.F, self.n_q, self.n_kv, self.D,
                                    self.block_size, self.n_sm, _ptr(self.trace), _st()), "decode_mega")
        _count()
        return logits

    def arrivals_us(self) -> torch.Tensor:
        """With the trace on: ``[n_ctas, 2 + 5 * n_layers]`` microseconds (relative to the earliest stamp) at which each
        CTA started and then finished each phase of the last step (per layer: QKV, attention, O, gate/up, down; last
        the vocabulary projection)."""
        t = self.trace.view(148, 1024).cpu()[: min(148, self.n_sm), : 2 + 5 * self.n_layers].double()
        return (t - t.min()) / 1e3

    def cycles(self) -> torch.Tensor:
        """With the trace on: ``[3, n_ctas, 2 + 5 * n_layers]`` cumulative SM cycles that one warp of each CTA had spent
        waiting for weight stages, computing, and waiting at the block barrier by the end of each phase."""
        t = self.trace.view(148, 4, 256).cpu()[: min(148, self.n_sm), 1:, : 2 + 5 * self.n_layers].double()
        return t.permute(1, 0, 2)


_sample_ws: dict[int, tuple[int, torch.Tensor]] = {}      # device index -> zero-initialised scratch of the multi-CTA sampler
use_fast_sampler = os.environ.get("EXO_DISABLE_FAST_SAMPLER") != "1"


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    """Filtered sampling, one token per row: three multi-CTA passes (histogram, boundary bin, draw) plus the single-CTA
    bisection kernel for rows whose distribution is too flat for the histogram to resolve."""
    rows, V = logits.shape
    lib = load()
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if not use_fast_sampler:
        _chk(lib.exo_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                            _ptr(out), rows, V, logits.stride(0), _dt(logits), _st()), "sample")
        _count()
        return out
    dev = logits.device.index or 0
    cap, ws = _sample_ws.get(dev, (0, None))
    if rows > cap:
        # grown outside any stream capture in practice: the executor's warm-up steps run before it captures
        cap = max(64, 1 << (rows - 1).bit_length())
        ws = torch.zeros(int(lib.exo_sample_workspace(cap)), dtype=torch.uint8, device=logits.device)
        _sample_ws[dev] = (cap, ws)
    _chk(lib.exo_sample_fast(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                             _ptr(out), _ptr(ws), cap, rows, V, logits.stride(0), _dt(logits), _st()), "sample")
    _count(4)
    return out


# ---- multi-head latent attention (DeepSeek-V2/V3, Kimi): absorbed form over the latent cache ----------------------
MLA_SMALL_T = 64      # up to this many tokens the absorbed projections run as CUDA-core kernels (weights read once)
use_mla_kernels = os.environ.get("EXO_DISABLE_MLA_KERNELS") != "1"


def _mla_dims_ok(kv_lora, rope_dim, dtype) -> bool:
    return use_mla_kernels and kv_lora == 512 and rope_dim == 64 and dtype == torch.bfloat16


def mla_kv_append(kva, norm_w, eps, positions, inv_freq, mscale, cache, slots, kv_lora):
    """Cache rows of the new tokens: ``[RMSNorm(kva[:, :kv_lora]) * norm_w | RoPE(kva[:, kv_lora:])]`` (adjacent-pair rope)."""
    rope_dim = kva.shape[1] - kv_lora
    if not (_mla_dims_ok(kv_lora, rope_dim, kva.dtype) and cache.dtype == torch.bfloat16):
        return ref.mla_kv_append(kva, norm_w, eps, positions, inv_freq, mscale, cache, slots, kv_lora)
    kva = kva.contiguous()
    _chk(load().exo_mla_kv_append(_ptr(kva), _ptr(norm_w), float(eps), _ptr(positions), _ptr(inv_freq), float(mscale),
                                  _ptr(cache), _ptr(slots), kva.shape[0], kv_lora, rope_dim, _st()), "mla_kv_append")
    _count()


def _heads_gemm(x_htk, w_hnk):
    """``out[h] = x[h] @ w[h].T`` for every head with the tcgen05 GEMM: ``[H, T, K] x [H, N, K] -> [H, T, N]``."""
    H, T, _ = x_htk.shape
    out = torch.empty(H, T, w_hnk.shape[1], dtype=x_htk.dtype, device=x_htk.device)
    for h in range(H):
        gemm_bf16(x_htk[h], w_hnk[h], out=out[h])
    return out


def mla_q_absorb(q, w_uk, positions, inv_freq, mscale, nope, kv_lora, w_uk_t=None):
    """Queries in cache space: ``[T, H, nope + rope] -> [T, H, kv_lora + rope]`` with ``q_nope . W_UK`` in front and
    the rotated rope sub-vector behind.  ``w_uk [H, nope, kv_lora]``; ``w_uk_t [H, kv_lora, nope]`` serves prefill."""
    T, H, qd = q.shape
    rope_dim = qd - nope
    if not (_mla_dims_ok(kv_lora, rope_dim, q.dtype) and nope == 128 and w_uk.dtype == torch.bfloat16):
        return ref.mla_q_absorb(q, w_uk, positions, inv_freq, mscale, nope)
    q = q.contiguous()
    out = torch.empty(T, H, kv_lora + rope_dim, dtype=q.dtype, device=q.device)
    small = T <= MLA_SMALL_T or gemm_impl is None
    _chk(load().exo_mla_q_absorb(_ptr(q), _ptr(w_uk), _ptr(positions), _ptr(inv_freq), float(mscale), _ptr(out), T, H, nope,
                                 kv_lora, rope_dim, int(not small), _st()), "mla_q_absorb")
    _count()
    if not small:
        ensure_gemm_init(q.device)
        wt = w_uk_t if w_uk_t is not None else w_uk.transpose(1, 2).contiguous()
        lat = _heads_gemm(q[..., :nope].transpose(0, 1).contiguous(), wt)          # [H, T, kv_lora]
        out[..., :kv_lora] = lat.transpose(0, 1)
        _count(H)
    return out


def mla_o_absorb(o_lat, w_uv):
    """Attention output back to head space: ``[T, H, kv_lora] x w_uv [H, v, kv_lora] -> [T, H * v]``."""
    T, H, L = o_lat.shape
    V = w_uv.shape[1]
    if not (use_mla_kernels and L == 512 and V == 128 and o_lat.dtype == torch.bfloat16 and w_uv.dtype == torch.bfloat16):
        return ref.mla_o_absorb(o_lat, w_uv)
    o_lat = o_lat.contiguous()
    if T <= MLA_SMALL_T or gemm_impl is None:
        out = torch.empty(T, H * V, dtype=o_lat.dtype, device=o_lat.device)
        _chk(load().exo_mla_o_absorb(_ptr(o_lat), _ptr(w_uv), _ptr(out), T, H, V, L, _st()), "mla_o_absorb")
        _count()
        return out
    ensure_gemm_init(o_lat.device)
    o = _heads_gemm(o_lat.transpose(0, 1).contiguous(), w_uv)                        # [H, T, V]
    _count(H)
    return o.transpose(0, 1).reshape(T, H * V)


def mla_paged_attention(q_full, ckv, block_tables, seq_lens, cu_q, scale, kv_lora, max_q_len=None):
    """Absorbed MLA attention: ``q_full [T, H, kv_lora + rope]`` (see :func:`mla_q_absorb`) over the paged latent cache
    ``ckv [n_blocks, block, kv_lora + rope]``; returns ``o_lat [T, H, kv_lora]``."""
    T, H, qd = q_full.shape
    rope_dim = qd - kv_lora
    nblk, bs, _ = ckv.shape
    B = seq_lens.numel()
    ok = _mla_dims_ok(kv_lora, rope_dim, q_full.dtype) and ckv.dtype == torch.bfloat16 and bs == 16 and (H % 16 == 0 or H in (1, 2, 4, 8))
    if not ok:
        return ref.mla_paged_attention(q_full[..., :kv_lora], q_full[..., kv_lora:], ckv, block_tables, seq_lens, cu_q, scale,
                                       kv_lora)
    lib = load()
    ensure_gemm_init(q_full.device)
    q_full = q_full.contiguous()
    out = torch.empty(T, H, kv_lora, dtype=q_full.dtype, device=q_full.device)
    decode = max_q_len == 1 and T == B
    groups = max(1, H // 16)
    max_blocks = block_tables.shape[1]
    tok_seq = None
    if decode:
        ns = lib.exo_mla_attn_splits(T * groups, max_blocks * bs)
    else:
        ns = 1
        tok_seq = torch.empty(T, dtype=torch.int32, device=q_full.device)
        _chk(lib.exo_token_seq(_ptr(cu_q), _ptr(tok_seq), B, _st()), "token_seq")
        _count()
    ws = _workspace(q_full.device, lib.exo_mla_attn_workspace(T, H, ns)) if ns > 1 else None
    _chk(lib.exo_mla_attn_tc(_ptr(q_full), _ptr(ckv), _ptr(block_tables), _ptr(seq_lens), None if decode else _ptr(cu_q),
                             _ptr(tok_seq), _ptr(out), _ptr(ws), float(scale), T, H, kv_lora, rope_dim, nblk,
                             max_blocks, bs, ns, _st()), "mla_attn_tc")
    _count(2 if ns > 1 else 1)
    return out


MOE_GEMV_MAX_TOKENS = 4    # up to this many tokens the experts run as grouped GEMVs (no sort, two launches)
use_moe_kernels = os.environ.get("EXO_DISABLE_MOE_KERNELS") != "1"
use_moe_gemv_fp8 = os.environ.get("EXO_DISABLE_MOE_GEMV_FP8") != "1"    # off: small batches of fp8 experts take the grouped GEMM


def moe_route(logits, top_k, kind, norm_topk, bias, n_group, topk_group, scaling):
    T, E = logits.shape
    if (not use_moe_kernels or E > 512 or top_k > 16 or n_group > 32 or logits.dtype not in _DT
            or (bias is not None and bias.dtype not in _DT)):
        return ref.moe_route(logits, top_k, kind, norm_topk, bias, n_group, topk_group, scaling)
    logits = logits.contiguous()
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    sig = kind != "softmax"
    _chk(load().exo_moe_route(_ptr(logits), _ptr(bias) if sig else None, _ptr(w), _ptr(ids), T, E, top_k,
                              n_group if sig else 1, topk_group if sig else 1, _dt(logits),
                              _dt(bias) if (sig and bias is not None) else BF16, int(sig), int(bool(norm_topk)),
                              float(scaling), _st()), "moe_route")
    _count()
    return w, ids


MOE_ACTS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}


def moe_experts(x, w_gate_up, w_down, weights, ids, expert_offset=0, n_experts_total=None, act="silu", limit=0.0):
    """``act``: ``silu`` / ``gelu_tanh`` (gated: ``w_gate_up [E, 2F, H]``) or ``relu2`` (not gated: ``w_gate_up [E, F, H]``).
    ``limit`` > 0 (with ``silu``): the activated gate is capped at ``limit`` and the up projection clamped to ``+-limit``."""
    T, H = x.shape
    E, F2, _ = w_gate_up.shape
    F, k = (F2 if act == "relu2" else F2 // 2), ids.shape[1]
    fp8 = isinstance(w_gate_up, Fp8Weight)
    if fp8 and act != "silu":
        raise KernelError("block-scaled fp8 experts are built for SwiGLU only")
    ok = (use_moe_kernels and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and H % 8 == 0 and F % 8 == 0
          and H >= 64 and F >= 64 and E <= 1024)
    if fp8:
        ok = ok and isinstance(w_down, Fp8Weight) and H % 64 == 0 and F % 128 == 0
    if not ok:
        return ref.moe_experts(x, w_gate_up, w_down, weights, ids, expert_offset, act, limit)
    x, ids = x.contiguous(), ids.contiguous().to(torch.int32)
    weights = weights.contiguous().float()
    out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    P = T * k
    lib = load()
    if not fp8 and T <= MOE_GEMV_MAX_TOKENS and H * 2 <= 200 * 1024 and k * F * 2 <= 200 * 1024:
        hs = torch.empty(P, F, dtype=x.dtype, device=x.device)
        _chk(lib.exo_moe_experts_gemv(_ptr(x), _ptr(w_gate_up), _ptr(w_down), _ptr(weights), _ptr(ids), _ptr(out), _ptr(hs),
                                      T, k, H, F, E, expert_offset, MOE_ACTS[act], float(limit), _st()), "moe_experts_gemv")
        _count(2)
        return out
    if (fp8 and use_moe_gemv_fp8 and not limit and T <= MOE_GEMV_MAX_TOKENS and -(-H // 64) * 128 <= 200 * 1024
            and k * -(-F // 64) * 128 <= 200 * 1024):
        # a handful of tokens: stream the chosen experts' fp8 tiles on CUDA cores over all SMs (two launches) instead of
        # the grouped tensor-core GEMM, which keeps one CTA per 128 features of a pair busy and the rest of the GPU idle
        hs = torch.empty(P, F, dtype=x.dtype, device=x.device)
        kind = 1 if w_gate_up.kind == "mxfp8" else 2
        _chk(lib.exo_moe_experts_gemv_fp8(_ptr(x), _ptr(w_gate_up.to_tiled().tiles), _ptr(w_down.to_tiled().tiles), _ptr(weights),
                                          _ptr(ids), _ptr(out), _ptr(hs), T, k, H, F, E, expert_offset, kind, _st()),
             "moe_experts_gemv_fp8")
        _count(2)
        return out
    ensure_gemm_init(x.device)
    # under expert parallelism only E / n_experts_total of the pairs are expected here: size the tiles for those
    bn = lib.exo_moe_tile_rows(max(1, P * E // max(E, n_experts_total or E)), E)
    scratch = torch.empty(lib.exo_moe_plan_ints(E, lib.exo_moe_max_tiles(P, E, bn)), dtype=torch.int32, device=x.device)
    pos = torch.empty(P, dtype=torch.int32, device=x.device)
    xs = torch.empty(P, H, dtype=x.dtype, device=x.device)
    hs = torch.empty(P, F, dtype=x.dtype, device=x.device)
    ys = torch.empty(P, H, dtype=x.dtype, device=x.device)
    if fp8:
        kind = 1 if w_gate_up.kind == "mxfp8" else 2
        wgu, wd = w_gate_up.to_tiled().tiles, w_down.to_tiled().tiles
    else:
        kind, wgu, wd = 0, w_gate_up.contiguous(), w_down.contiguous()
    _chk(lib.exo_moe_experts_grouped(_ptr(x), _ptr(wgu), _ptr(wd), _ptr(weights), _ptr(ids), _ptr(out),
                                     _ptr(scratch), _ptr(pos), _ptr(xs), _ptr(hs), _ptr(ys), T, k, H, F, E, expert_offset,
                                     kind, bn, int(fp8_f16_operands), MOE_ACTS[act], float(limit), _st()), "moe_experts_grouped")
    _count(7)
    return out
