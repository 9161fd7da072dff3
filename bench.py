#!/usr/bin/env python
"""Headline benchmark: decode tokens/s (batch 1 and 32) and TTFT for Llama-3.1-8B bf16 under
tensor parallelism on N B200s of one node (synthetic prompts, random-init weights).

    python bench.py --gpus N --steps K --warmup W            # N=1 runs in-process
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   # N>1

Two timed regions of exactly K decode steps each, both bracketed by barrier + synchronize and
timed with CUDA events, max over ranks:
  * device: pre-built step plans replayed back to back (input tokens taken from the previous
    step's samples on device) → ``value``;
  * end to end: the public ``Engine.step()`` call, which every step copies the packed plan from
    pinned host memory to the device and reads the sampled ids back → ``e2e``.
Measurement follows the reference's definition of generation throughput (tokens after the
first divided by the time between first and last token, ``bench/METHODOLOGY.md:37-63`` in the
reference) with EOS ignored so that exactly the requested number of tokens is produced.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np


def parse() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--batch", type=int, default=1, help="decode batch of the headline value")
    ap.add_argument("--also-batch", type=int, default=32, help="second decode batch reported under 'also'")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"])
    ap.add_argument("--no-also", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="pre-flight only: run the first N layers of the model (the JSON line then says so and is not a result)")
    return ap.parse_args()


REFERENCE_UNAVAILABLE = ("reference (exo 0.3.70) cannot be installed offline: build backend uv_build and its "
                         "mlx / mlx-cuda / mlx-lm git-fork dependencies and the Rust exo_rs crate are not in the image")


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.proc, self.rows = index, None, []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return

    import faulthandler
    # a stuck collective must end the run with a stack dump, not sit until an outer limit kills it
    faulthandler.dump_traceback_later(int(os.environ.get("EXO_BENCH_WATCHDOG_S", "900")), exit=True)

    import torch
    import torch.distributed as dist

    def note(msg: str) -> None:
        if os.environ.get("EXO_BENCH_VERBOSE"):
            print(f"[bench r{os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from exo_b200.models.config import preset
    from exo_b200.models.weights import ShardSpec, fast_random_weights
    from exo_b200.engine.engine import Engine
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.engine.plan import StepPlan, FLAG_ALL_GREEDY, FLAG_TOKENS_FROM_PREV
    from exo_b200.ops import cuda as K

    cfg = preset(args.model)
    if args.layers:
        from dataclasses import replace
        cfg = replace(cfg, n_layers=min(args.layers, cfg.n_layers))
    spec = ShardSpec(tp_rank=rank, tp_size=world)
    comm = None
    comm_name = "none"
    if world > 1:
        want = args.comm
        if want in ("auto", "fused"):
            try:
                from exo_b200.parallel.fused import FusedComm
                comm = FusedComm(dev, max_rows=max(args.prompt, 256), hidden=cfg.hidden,
                                 vocab_shard=-(-cfg.vocab // world))
                comm_name = "fused-p2p"
            except Exception as e:  # noqa: BLE001
                if want == "fused":
                    raise
                if rank == 0:
                    print(f"[bench] fused comm unavailable ({e!r}); using NCCL", file=sys.stderr)
        if comm is None:
            from exo_b200.parallel.comm import NcclComm
            comm = NcclComm()
            comm_name = "nccl"

    note(f"comm={comm_name}; building weights")
    weights = fast_random_weights(cfg, spec, dev, seed=0)
    torch.cuda.synchronize()
    note("weights ready")
    max_b = max(args.batch, 1 if args.no_also else args.also_batch)
    per_seq_blocks = -(-(args.prompt + 2 * args.warmup + 4 * args.steps + 64) // 16)
    n_blocks = max_b * per_seq_blocks + 64

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def make_engine() -> Engine:
        return Engine(cfg, weights, spec, comm, n_blocks=n_blocks, max_seqs=max(max_b, 8), prefill_chunk=4096,
                      max_blocks_per_seq=per_seq_blocks, device=dev, seed=0)

    eng = make_engine()
    rng = np.random.default_rng(1234)
    greedy = dict(temperature=0.0, ignore_eos=True)

    # ---------------- TTFT (one 2048-token prompt, admission -> first sampled token) ----------------
    def ttft_once() -> float:
        prompt = rng.integers(0, cfg.vocab, args.prompt).tolist()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rid = eng.submit(prompt, SamplingParams(max_tokens=1, **greedy), use_prefix_cache=False)
        got = False
        while not got:
            for o in eng.step():
                got |= o.req_id == rid and o.token is not None
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1))

    note("ttft warm-up")
    ttft_once()  # warm-up (kernel loading, descriptor caches)
    note("ttft timed")
    ttfts = [ttft_once() for _ in range(3)]
    note(f"ttft {ttfts}")
    ttft_ms = min(ttfts)
    K.gemm_check()

    # ---------------- decode ----------------
    def decode_bench(B: int, steps: int, warm: int) -> dict:
        for s in list(eng.seqs):
            eng.cancel(s)
        rids = [eng.submit(rng.integers(0, cfg.vocab, args.prompt).tolist(),
                           SamplingParams(max_tokens=10 ** 6, **greedy), use_prefix_cache=False) for _ in range(B)]
        while any(eng.seqs[r].in_prefill or not eng.seqs[r].output for r in rids):
            eng.step()
        note(f"decode B={B}: prefill done, warming up")
        for _ in range(max(warm, 3)):
            eng.step()
        note("e2e timed loop")
        # --- end to end: public API, H2D of the plan and D2H of the ids every step ---
        h0, d0 = eng.exe.h2d_bytes, eng.exe.d2h_bytes
        sampler = ClockSampler(local)
        barrier()
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng.step()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1))
        h2d = (eng.exe.h2d_bytes - h0) // steps
        d2h = (eng.exe.d2h_bytes - d0) // steps
        # --- device: pre-built plans, tokens chained on device ---
        seqs = [eng.seqs[r] for r in rids]
        bs = eng.alloc.block_size
        for s in seqs:
            assert eng.sched._ensure_blocks(s, s.n_tokens + steps + warm + 8)
        mb = max(len(s.blocks) for s in seqs)
        bt = np.zeros((B, mb), np.int32)
        for b, s in enumerate(seqs):
            bt[b, :len(s.blocks)] = s.blocks
        base = np.array([s.n_tokens - 1 for s in seqs], np.int32)
        rows = np.arange(B, dtype=np.int32)

        def plan_at(i: int) -> StepPlan:
            pos = base + i
            return StepPlan(n_tokens=B, n_seqs=B, max_q_len=1, flags=FLAG_ALL_GREEDY | FLAG_TOKENS_FROM_PREV,
                            tokens=np.zeros(B, np.int32), positions=pos, slots=bt[rows, pos // bs] * bs + pos % bs,
                            cu_q=np.arange(B + 1, dtype=np.int32), seq_lens=pos + 1, logit_rows=rows,
                            top_k=np.zeros(B, np.int32), temperature=np.zeros(B, np.float32),
                            top_p=np.ones(B, np.float32), min_p=np.zeros(B, np.float32),
                            uniform=np.zeros(B, np.float32), prev_rows=rows, block_tables=bt)
        note("device timed loop")
        plans = [plan_at(i) for i in range(steps + max(warm, 3))]
        for i in range(max(warm, 3)):
            eng.exe.run(plans[i])
        launches_before = K.launch_count
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            eng.exe.run(plans[max(warm, 3) + i])
        e1.record()
        barrier()
        clocks = sampler.stop() if rank == 0 else {}
        dev_ms = max_over_ranks(e0.elapsed_time(e1))
        key = (eng.exe.graphs and next(iter(eng.exe.graphs))) or None
        K.gemm_check()
        return {"B": B, "dev_ms_per_step": dev_ms / steps, "e2e_ms_per_step": e2e_ms / steps,
                "dev_tok_s": B * steps / (dev_ms / 1e3), "e2e_tok_s": B * steps / (e2e_ms / 1e3),
                "h2d": int(h2d), "d2h": int(d2h), "clocks": clocks, "eager_launches": K.launch_count - launches_before}

    # kernels per decode step = launches recorded while the step's graph was captured
    main_res = decode_bench(args.batch, args.steps, args.warmup)
    per_step_launches = getattr(eng.exe, "launches_per_graph", {}).get(
        __import__("exo_b200.engine.plan", fromlist=["bucket"]).bucket(args.batch, (1, 2, 4, 8, 16, 32, 64, 128, 256)), 0)
    also = None
    if not args.no_also and args.also_batch != args.batch:
        also = decode_bench(args.also_batch, max(16, args.steps // 2), args.warmup)

    if rank == 0:
        out = {
            "metric": f"decode_tok_s_bs{args.batch}", "value": round(main_res["dev_tok_s"], 2), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(main_res["dev_ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"model": cfg.name + (f" (REDUCED to {cfg.n_layers} layers: pre-flight, not a result)" if args.layers else ""),
                       "weights": cfg.quant if cfg.quant != "none" else "bf16",
                       "global_batch": args.batch, "seq_len": args.prompt,
                       "decode_context": f"{args.prompt}+", "parallelism": f"tp{world}", "comm": comm_name,
                       "l2": "per-step inputs (weights + KV) exceed the 126 MB L2; no explicit flush",
                       "kv": "paged, block 16"},
            "clocks": main_res["clocks"],
            "e2e": {"value": round(main_res["e2e_tok_s"], 2), "unit": "tokens/s",
                    "h2d_bytes_per_step": main_res["h2d"], "d2h_bytes_per_step": main_res["d2h"]},
            "gpu_launches": int(per_step_launches * args.steps) if per_step_launches else int(main_res["eager_launches"]),
            "ttft_ms": round(ttft_ms, 3), "prefill_tok_s": round(args.prompt / (ttft_ms / 1e3), 1),
        }
        if also is not None:
            out["also"] = {f"decode_tok_s_bs{also['B']}": round(also["dev_tok_s"], 1),
                           f"e2e_tok_s_bs{also['B']}": round(also["e2e_tok_s"], 1),
                           "ms_per_step": round(also["dev_ms_per_step"], 4)}
        print(json.dumps(out), flush=True)
    faulthandler.cancel_dump_traceback_later()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator whose collectives were captured
        # in still-alive CUDA graphs blocked for minutes (both ranks sat in destroy_process_group).
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
