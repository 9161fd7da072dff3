"""Micro-benchmarks of the individual sm_100a kernels against the measured roofline.

    python -m exo_b200.utils.bench_kernels [--only gemv,gemm,fp8,moe,attn,mla,prefill,gdn,misc] [--peaks MEASURED_PEAKS.json]

Every case is timed with CUDA events after warm-up; a 256 MB buffer is overwritten between
iterations so that no operand survives in the 126 MB L2.  Output: achieved GB/s or TFLOP/s and
the fraction of the measured copy bandwidth / cuBLAS bf16 throughput.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from ..ops import cuda as K
from ..ops import reference as ref


def timeit(fn, iters: int = 10, warm: int = 3) -> float:
    # L2 flush = write 256 MB, then read another 256 MB: the read sweep forces the write-back of the
    # dirty lines, so the timed kernel starts on a cold but CLEAN L2 (dirty lines would be written
    # back during the timed reads and charge it with DRAM traffic that is not its own)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    sweep = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        flush.fill_(1)
        sweep.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best  # ms


def timeit_rot(fns, reps: int = 0, iters: int = 5) -> float:
    """Per-call time of a list of equivalent calls on DIFFERENT operands run back to back.

    The operands together exceed the L2 several times over, so each call streams from HBM, and
    the event pair brackets many calls, so its own microseconds do not bias short kernels.
    """
    reps = reps or max(len(fns), 8)
    for i in range(len(fns)):
        fns[i]()
    torch.cuda.synchronize()
    # the calls are captured in a CUDA graph: a Python-driven launch costs ~10 us of host time,
    # more than most of these kernels run, and would turn the measurement into a launch benchmark
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for i in range(reps):
            fns[i % len(fns)]()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    return best


def small_cases(only: set[str]) -> None:
    """One case per section, a few hundred MB on the device, three eager launches each."""
    from ..ops import quant
    K.load()
    g = torch.Generator(device="cuda").manual_seed(0)

    def rnd(*s):
        return (torch.randn(*s, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    calls = []
    if "fp8" in only:
        x, w = rnd(32, 4096), quant.quantize(rnd(28672, 4096), "mxfp8")
        calls.append(lambda: K.linear(x, w))
        x2 = rnd(2048, 4096)
        calls.append(lambda: K.linear(x2, w))
    if "gemm" in only:
        xg, wg = rnd(2048, 4096), rnd(28672, 4096)
        calls.append(lambda: K.gemm_bf16(xg, wg))
    if "moe" in only:
        E_all, E, k, H, F = 128, 16, 8, 4096, 1536
        wgu, wd = rnd(E, 2 * F, H), rnd(E, H, F)
        for T in (32, 4096):
            xm = rnd(T, H)
            wt, ids = K.moe_route(torch.randn(T, E_all, device="cuda", generator=g), k, "softmax", True, None, 1, 1, 1.0)
            calls.append(lambda xm=xm, wt=wt, ids=ids: K.moe_experts(xm, wgu, wd, wt, ids, 0, E_all))
    if "attn" in only:
        Hq, Hkv, D, bs, B, ctx = 32, 8, 128, 16, 32, 2048
        nb = B * (ctx // bs + 1) + 1
        bt = (torch.arange(B * (ctx // bs + 1), device="cuda", dtype=torch.int32) + 1).view(B, -1)
        sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
        q, kc, vc = rnd(B, Hq, D), rnd(nb, bs, Hkv, D), rnd(nb, bs, Hkv, D)
        calls.append(lambda: K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=1))
    if "mla" in only:
        H, kvl, rope, bs, B, ctx = 16, 512, 64, 16, 16, 8192
        nbk = B * (ctx // bs) + 1
        btm = (torch.arange(B * (ctx // bs), device="cuda", dtype=torch.int32) + 1).view(B, -1)
        slm = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        cum = torch.arange(B + 1, device="cuda", dtype=torch.int32)
        qm, ckv = rnd(B, H, kvl + rope), rnd(nbk, bs, kvl + rope)
        calls.append(lambda: K.mla_paged_attention(qm, ckv, btm, slm, cum, (128 + rope) ** -0.5, kvl, max_q_len=1))
    if "misc" in only:
        lg = rnd(32, 128256) * 40
        lg[:, ::3001] += 14.0
        t = torch.full((32,), 0.7, device="cuda")
        tk = torch.full((32,), 20, device="cuda", dtype=torch.int32)
        tp, mp, u = torch.full((32,), 0.9, device="cuda"), torch.full((32,), 0.05, device="cuda"), torch.rand(32, device="cuda")
        calls.append(lambda: K.sample(lg, t, tk, tp, mp, u))
    if "comm" in only:
        # the reduce + residual + RMSNorm kernel of a two-rank group on ONE GPU: the peer is a second local arena whose
        # partial and arrival flag the host writes (no kernel waits on another kernel)
        import ctypes as C

        from ..parallel.fused import arena_layout, bind
        lib = bind(K.load())
        K.ensure_gemm_init(torch.device("cuda", 0))
        rows, cols = 256, 4096
        L = arena_layout(lib, 2, rows, cols, 64, 8)
        arenas = [torch.zeros(L["total"], dtype=torch.uint8, device="cuda") for _ in range(2)]
        arr = (C.c_void_p * 2)(*[a.data_ptr() for a in arenas])
        assert lib.exo_comm_init(arr, None, 2, 0, L["slot"], L["gather_off"], L["x_off"], L["x_bytes"], L["h_off"], L["n_off"],
                                 L["ll_off"], L["ll_slot"]) == 0
        res, w = rnd(rows, cols), rnd(cols)
        hh, xx = torch.empty_like(res), torch.empty_like(res)
        state = {"it": 0}

        def reduce_once():
            parity = state["it"] & 1
            state["it"] += 1
            arenas[0][:4096].view(torch.int32)[2048 // 4 + parity * 8 + 1] = 1        # the peer's "partial ready"
            lib.exo_reduce_norm_bf16(res.data_ptr(), w.data_ptr(), 1e-5, hh.data_ptr(), xx.data_ptr(), rows, cols, parity, 0, 1,
                                     torch.cuda.current_stream().cuda_stream)
        calls.append(reduce_once)
    for _ in range(3):
        for c in calls:
            c()
    torch.cuda.synchronize()
    if "comm" in only:
        K.check_status()
        lib.exo_comm_reset()
    K.gemm_check()
    print("small cases done:", len(calls))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="gemv,gemm,fp8,moe,attn,mla,prefill,misc")
    ap.add_argument("--peaks", default=str(Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"))
    ap.add_argument("--small", action="store_true",
                    help="one modest case per section, launched eagerly three times (the form to run under a profiler)")
    a = ap.parse_args()
    if a.small:
        small_cases(set(a.only.split(",")))
        return
    hbm, tf, basis = 6650.0, 1590.0, "fallback"
    try:
        p = json.loads(Path(a.peaks).read_text())
        hbm, tf, basis = p["hbm_gbs"], p["bf16_tflops"], "measured"
    except (OSError, KeyError, ValueError):
        pass
    only = set(a.only.split(","))
    K.load()
    g = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16

    def rnd(*s):
        return (torch.randn(*s, device="cuda", generator=g) * 0.05).to(bf)

    print(f"roofline basis: HBM {hbm:.0f} GB/s, bf16 {tf:.0f} TFLOP/s ({basis})")
    if "gemv" in only:
        for M in (1, 4, 8):
            for N, Kd in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (16032, 4096), (4096, 512)):
                x, nw = rnd(M, Kd), rnd(Kd)
                copies = max(2, -(-(400 << 20) // (N * Kd * 2)))
                ws = [rnd(N, Kd) for _ in range(copies)]
                ms = timeit_rot([(lambda w=w: K.linear(x, w, None, None, nw, 1e-5)) for w in ws])
                gb = N * Kd * 2 / 1e9
                print(f"gemv M={M} N={N} K={Kd}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s  "
                      f"{gb / ms * 1e3 / hbm:5.2f} of {basis} HBM")
    if "gemm" in only:
        for M in (16, 32, 64, 128, 256, 2048, 4096):
            for N, Kd in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
                x = rnd(M, Kd)
                copies = max(2, -(-(400 << 20) // (N * Kd * 2)))
                ws = [rnd(N, Kd) for _ in range(copies)]
                ms = timeit_rot([(lambda w=w: K.gemm_bf16(x, w)) for w in ws])
                gb = (N * Kd + M * Kd + M * N) * 2 / 1e9
                fl = 2.0 * M * N * Kd / 1e12
                print(f"gemm M={M} N={N} K={Kd}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s ({gb / ms * 1e3 / hbm:4.2f})  "
                      f"{fl / ms * 1e3:7.1f} TFLOP/s ({fl / ms * 1e3 / tf:4.2f}) of {basis}")
        K.gemm_check()
    if "fp8" in only:
        # block-scaled fp8 weights (1 byte per weight + 1/32 byte of scale): the roofline is the bytes read
        from ..ops import quant
        for M in (1, 32, 64, 2048):
            for N, Kd in ((6144, 4096), (28672, 4096), (4096, 14336)):
                x = rnd(M, Kd)
                copies = max(2, -(-(400 << 20) // (N * Kd)))
                ws = [quant.quantize(rnd(N, Kd), "mxfp8") for _ in range(copies)]
                ms = timeit_rot([(lambda w=w: K.linear(x, w)) for w in ws])
                gb = (N * Kd * (1 + 1 / 32) + (M * Kd + M * N) * 2) / 1e9
                fl = 2.0 * M * N * Kd / 1e12
                print(f"gemm-fp8w M={M} N={N} K={Kd}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s ({gb / ms * 1e3 / hbm:4.2f})  "
                      f"{fl / ms * 1e3:7.1f} TFLOP/s ({fl / ms * 1e3 / tf:4.2f}) of {basis}")
        K.gemm_check()
    if "moe" in only:
        # one rank's share of a Qwen3-235B-A22B layer under EP8: 16 local experts of 128, top-8, H 4096, F 1536
        E_all, E, k, H, F = 128, 16, 8, 4096, 1536
        for T in (1, 4, 32, 256, 4096):
            x = rnd(T, H)
            logits = torch.randn(T, E_all, device="cuda", generator=g)
            w, ids = K.moe_route(logits, k, "softmax", True, None, 1, 1, 1.0)
            copies = max(2, -(-(400 << 20) // (E * 3 * F * H * 2)))
            ex = [(rnd(E, 2 * F, H), rnd(E, H, F)) for _ in range(copies)]
            ms = timeit_rot([(lambda a=a, b=b: K.moe_experts(x, a, b, w, ids, 0, E_all)) for a, b in ex])
            local = (ids < E)
            active = int(torch.unique(ids[local]).numel())
            pairs = int(local.sum())
            gb = active * 3 * F * H * 2 / 1e9
            fl = 2.0 * pairs * 3 * F * H / 1e12
            print(f"moe-experts T={T} ({pairs} local pairs, {active}/{E} experts): {ms * 1e3:8.1f} us  "
                  f"{gb / ms * 1e3:7.0f} GB/s ({gb / ms * 1e3 / hbm:4.2f})  {fl / ms * 1e3:7.1f} TFLOP/s ({fl / ms * 1e3 / tf:4.2f}) of {basis}")
            if True:        # the same experts as block-scaled fp8
                from ..ops import quant
                exq = [(quant.quantize(a, "mxfp8"), quant.quantize(b, "mxfp8")) for a, b in ex]
                gbq = gb / 2 * (1 + 1 / 32)
                for gemv in ((True, False) if T <= K.MOE_GEMV_MAX_TOKENS else (False,)):
                    K.use_moe_gemv_fp8 = gemv
                    ms = timeit_rot([(lambda a=a, b=b: K.moe_experts(x, a, b, w, ids, 0, E_all)) for a, b in exq])
                    print(f"moe-experts-fp8 T={T} ({'streaming GEMV' if gemv else 'grouped GEMM'}): {ms * 1e3:8.1f} us  "
                          f"{gbq / ms * 1e3:7.0f} GB/s ({gbq / ms * 1e3 / hbm:4.2f})  "
                          f"{fl / ms * 1e3:7.1f} TFLOP/s ({fl / ms * 1e3 / tf:4.2f}) of {basis}")
                K.use_moe_gemv_fp8 = True
                del exq
            ms = timeit_rot([(lambda: K.moe_route(logits, k, "softmax", True, None, 1, 1, 1.0)) for _ in range(4)])
            print(f"moe-route T={T} E={E_all} k={k}: {ms * 1e3:8.1f} us")
        K.gemm_check()
    if "moegemv" in only:
        # decode-sized batches of block-scaled fp8 experts with every chosen expert local (the streaming GEMV pair alone):
        # a Qwen3-235B rank (H 4096, F 1536) and a DeepSeek-V3 rank (H 7168, F 2048), one token, eight experts
        from ..ops import quant
        for name, E, k, H, F, kind in (("qwen3-235b", 16, 8, 4096, 1536, "mxfp8"), ("deepseek-v3", 32, 8, 7168, 2048, "dsfp8")):
            x = rnd(1, H)
            w = torch.full((1, k), 1.0 / k, device="cuda")
            exq = [(quant.quantize(rnd(E, 2 * F, H), kind), quant.quantize(rnd(E, H, F), kind)) for _ in range(4)]
            for n_local in (k, 2, 1):       # the rest of the token's experts live on other ranks
                ids = torch.randperm(E, device="cuda")[:k].to(torch.int32).view(1, k)
                ids[0, n_local:] += 10000
                gbq = n_local * 3 * F * H * (1 + 1 / 32) / 1e9
                for gemv in (True, False):
                    K.use_moe_gemv_fp8 = gemv
                    ms = timeit_rot([(lambda a=a, b=b: K.moe_experts(x, a, b, w, ids, 0, E)) for a, b in exq], reps=16)
                    print(f"moe-experts-fp8 {name} T=1, {n_local} of {k} pairs local ({'streaming GEMV' if gemv else 'grouped GEMM'}): "
                          f"{ms * 1e3:8.1f} us  {gbq / ms * 1e3:7.0f} GB/s ({gbq / ms * 1e3 / hbm:4.2f} of {basis} HBM)")
            K.use_moe_gemv_fp8 = True
            del exq
    if "attn" in only:
        Hq, Hkv, D, bs = 32, 8, 128, 16
        for B, ctx in ((1, 2048), (1, 8192), (32, 2048), (64, 4096)):
            nb = B * (ctx // bs + 1) + 1
            bt = (torch.arange(B * (ctx // bs + 1), device="cuda", dtype=torch.int32) + 1).view(B, -1)
            sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
            cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
            q = rnd(B, Hq, D)
            gb = B * ctx * Hkv * D * 2 * 2 / 1e9
            copies = max(2, int(0.4 / gb) + 1)
            caches = [(rnd(nb, bs, Hkv, D), rnd(nb, bs, Hkv, D)) for _ in range(copies)]
            ms = timeit_rot([(lambda kc=kc, vc=vc: K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=1))
                             for kc, vc in caches])
            print(f"decode-attn B={B} ctx={ctx}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s  "
                  f"{gb / ms * 1e3 / hbm:5.2f} of {basis} HBM")
    if "mla" in only:
        # DeepSeek-V3 attention of one rank under TP8: 16 heads over the shared latent cache (576 values per token)
        H, L, R, bs = 16, 512, 64, 16
        for B, ctx in ((1, 8192), (16, 8192), (64, 4096)):
            per = ctx // bs + 1
            bt = (torch.arange(B * per, device="cuda", dtype=torch.int32) + 1).view(B, -1)
            sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
            cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
            q = rnd(B, H, L + R)
            gb = B * ctx * (L + R) * 2 / 1e9
            copies = max(2, int(0.4 / gb) + 1)
            caches = [rnd(B * per + 1, bs, L + R) for _ in range(copies)]
            ms = timeit_rot([(lambda c=c: K.mla_paged_attention(q, c, bt, sl, cu, 192 ** -0.5, L, 1)) for c in caches])
            print(f"mla-decode-attn B={B} ctx={ctx} heads={H}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s  "
                  f"{gb / ms * 1e3 / hbm:5.2f} of {basis} HBM")
        T = 2048
        per = T // bs + 1
        c = rnd(per + 1, bs, L + R)
        bt = (torch.arange(per, device="cuda", dtype=torch.int32) + 1).view(1, -1)
        sl = torch.tensor([T], device="cuda", dtype=torch.int32)
        cu = torch.tensor([0, T], device="cuda", dtype=torch.int32)
        q = rnd(T, H, L + R)
        ms = timeit(lambda: K.mla_paged_attention(q, c, bt, sl, cu, 192 ** -0.5, L, T), iters=5)
        fl = 2.0 * T * T / 2 * H * (2 * L + R) / 1e12
        print(f"mla-prefill-attn T={T} heads={H}: {ms * 1e3:8.1f} us  {fl / ms * 1e3:7.1f} TFLOP/s (causal)  "
              f"{fl / ms * 1e3 / tf:5.2f} of {basis} bf16")
        K.check_status()
    if "prefill" in only:
        Hq, Hkv, D, bs = 32, 8, 128, 16
        for T in (512, 2048, 4096):
            nb = T // bs + 2
            kc, vc = rnd(nb, bs, Hkv, D), rnd(nb, bs, Hkv, D)
            bt = (torch.arange(nb - 1, device="cuda", dtype=torch.int32) + 1).view(1, -1)
            sl = torch.tensor([T], device="cuda", dtype=torch.int32)
            cu = torch.tensor([0, T], device="cuda", dtype=torch.int32)
            q = rnd(T, Hq, D)
            ms = timeit(lambda: K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=T), iters=5)
            fl = 4.0 * T * T * Hq * D / 2 / 1e12
            print(f"prefill-attn T={T}: {ms * 1e3:8.1f} us  {fl / ms * 1e3:7.1f} TFLOP/s (causal)  "
                  f"{fl / ms * 1e3 / tf:5.2f} of {basis} bf16")
    if "gdn" in only:
        # Qwen3-Next linear-attention layer between its projections: 16 key heads, 32 value heads, 128 x 128 state per head
        hk, hv, dk, dv, taps = 16, 32, 128, 128, 4
        C = 2 * hk * dk + hv * dv
        W = C + hv * dv + 2 * hv
        conv_w = torch.randn(C, taps, device="cuda") * 0.3
        a_log, dt_b, nw = torch.randn(hv, device="cuda") * 0.3, torch.randn(hv, device="cuda") * 0.3, rnd(dv)
        for B, L in ((1, 1), (32, 1), (128, 1), (1, 2048), (4, 2048)):
            T = B * L
            n_state = min(64, max(2, int(0.3e9 / (B * hv * dk * dv * 4)) + 1))          # rotate over more state than the L2 holds
            recs = [torch.zeros(B + 1, hv, dk, dv, device="cuda") for _ in range(n_state)]
            conv = torch.zeros(B + 1, C, taps - 1, device="cuda", dtype=torch.bfloat16)
            seats = torch.arange(1, B + 1, device="cuda", dtype=torch.int32)
            cu = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * L)
            pos = (torch.arange(L, device="cuda", dtype=torch.int32) + 7).repeat(B)
            proj = rnd(T, W)
            ms = timeit_rot([(lambda r=r: K.gated_delta(proj, conv_w, a_log, dt_b, nw, 1e-6, conv, r, seats, cu, pos, hk, hv, dk, dv))
                             for r in recs])
            gb = (2 * B * hv * dk * dv * 4 + T * (W + C + hv * dv) * 2) / 1e9
            print(f"gated-delta B={B} L={L}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s ({gb / ms * 1e3 / hbm:4.2f} of {basis} HBM)  "
                  f"{ms * 1e3 / L:6.2f} us per token of a sequence")
        # full-attention layers of the same model: 16 query heads over 2 KV heads of 256 dims
        Hq, Hkv, D, bs = 16, 2, 256, 16
        for B, ctx in ((1, 2048), (32, 2048), (32, 8192)):
            nb = B * (ctx // bs + 1) + 1
            bt = (torch.arange(B * (ctx // bs + 1), device="cuda", dtype=torch.int32) + 1).view(B, -1)
            sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
            cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
            q = rnd(B, Hq, D)
            gb = B * ctx * Hkv * D * 2 * 2 / 1e9
            copies = max(2, int(0.4 / gb) + 1)
            caches = [(rnd(nb, bs, Hkv, D), rnd(nb, bs, Hkv, D)) for _ in range(copies)]
            ms = timeit_rot([(lambda kc=kc, vc=vc: K.paged_attention(q, kc, vc, bt, sl, cu, D ** -0.5, max_q_len=1))
                             for kc, vc in caches])
            print(f"decode-attn D=256 B={B} ctx={ctx}: {ms * 1e3:8.1f} us  {gb / ms * 1e3:7.0f} GB/s  "
                  f"{gb / ms * 1e3 / hbm:5.2f} of {basis} HBM")
    if "misc" in only:
        logits = rnd(32, 128256)
        print(f"argmax 32x128256: {timeit(lambda: K.argmax(logits)) * 1e3:.1f} us")
        one = rnd(1, 128256)
        print(f"argmax 1x128256: {timeit(lambda: K.argmax(one)) * 1e3:.1f} us")
        t = torch.full((32,), 0.7, device="cuda")
        tk = torch.zeros(32, device="cuda", dtype=torch.int32)
        tp = torch.full((32,), 0.9, device="cuda")
        mp = torch.full((32,), 0.05, device="cuda")
        u = torch.rand(32, device="cuda")
        print(f"sample 32x128256: {timeit(lambda: K.sample(logits, t, tk, tp, mp, u)) * 1e3:.1f} us")
        # the sampler on the three kinds of rows it meets, each over distinct logits back to back inside a graph
        peaked = [rnd(32, 128256) * 2 for _ in range(8)]
        for lg in peaked:
            lg[:, ::3001] += 14.0
        flat = [rnd(32, 128256) * 0.05 for _ in range(8)]
        settings = {"temp 0.7, min_p 0.05 (the API default)": (0, 1.0, 0.05), "top_k 40": (40, 1.0, 0.0),
                    "top_p 0.95": (0, 0.95, 0.0), "top_k 20, top_p 0.9, min_p 0.05": (20, 0.9, 0.05)}
        for label, (k_, p_, m_) in settings.items():
            tk_, tp_, mp_ = torch.full_like(tk, k_), torch.full_like(tp, p_), torch.full_like(mp, m_)
            for kind, rows in (("peaked", peaked), ("flat", flat)):
                for fast in (True, False):
                    K.use_fast_sampler = fast
                    dt = timeit_rot([lambda lg=lg: K.sample(lg, t, tk_, tp_, mp_, u) for lg in rows])
                    print(f"sample 32x128256 {kind:6s} {label:42s} {'multi-CTA' if fast else 'bisection'}: {dt * 1e3:.1f} us")
        K.use_fast_sampler = True
        x, w = rnd(32, 4096), rnd(4096)
        print(f"rmsnorm 32x4096: {timeit(lambda: K.rmsnorm(x, w, 1e-5, x)) * 1e3:.1f} us")


if __name__ == "__main__":
    main()
