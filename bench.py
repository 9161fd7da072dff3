#!/usr/bin/env python
"""Headline benchmark: decode tokens/s (batch 1 and 32) and TTFT for Llama-3.1-8B bf16 under
tensor parallelism on N B200s of one node (synthetic prompts, random-init weights).

    python bench.py --gpus N --steps K --warmup W            # N=1 runs in-process
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   # N>1

Two timed regions of exactly K decode steps each, both bracketed by barrier + synchronize and
timed with CUDA events, max over ranks, each repeated until about a second has been timed (the
median repeat is reported):
  * device: pre-built step plans replayed back to back (input tokens taken from the previous
    step's samples on device) → ``value``;
  * end to end: the public ``Engine.step()`` call, which every step copies the packed plan from
    pinned host memory to the device and reads the sampled ids back → ``e2e``.
On N > 1 GPUs the ranks are arranged as in serving: rank 0 owns the scheduler and publishes every
step's plan through the shared-memory plan channel, the other ranks execute the plans they receive.
The same decode loop is then repeated with the NCCL communicator (projection, ``ncclAllReduce``,
separate residual add and norm) and ``vs_baseline`` is the ratio of the two.
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
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL-communicator arm behind vs_baseline")
    ap.add_argument("--min-timed-s", type=float, default=1.0, help="repeat each K-step region until this much is timed")
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (the N GPUs become PP stages x N/PP tensor-parallel lanes)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="pre-flight only, one GPU: hold rank 0's shard of an N-way tensor-parallel split with identity "
                         "collectives (kernel shapes and launch counts of one rank; the tokens mean nothing)")
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
    chan = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from exo_b200.models.config import preset
    from exo_b200.models.weights import ShardSpec, fast_random_weights
    from exo_b200.engine.engine import Engine
    from exo_b200.engine.executor import Executor
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.engine.plan import StepPlan, FLAG_ALL_GREEDY, FLAG_TOKENS_FROM_PREV, bucket
    from exo_b200.ops import cuda as K

    if world > 1:
        from exo_b200.worker.engines.b200.bringup import PlanChannel
        chan = PlanChannel(dist.new_group(backend="gloo"), rank, world)

    cfg = preset(args.model)
    if args.layers:
        from dataclasses import replace
        cfg = replace(cfg, n_layers=min(args.layers, cfg.n_layers))
    pp = max(1, args.pp)
    if world % pp or cfg.n_layers < pp:
        raise SystemExit(f"--pp {pp} does not divide {world} GPUs / {cfg.n_layers} layers")
    tp = world // pp
    pp_rank, tp_rank = divmod(rank, tp)
    per_stage = cfg.n_layers // pp
    spec = ShardSpec(tp_rank=tp_rank, tp_size=tp, pp_rank=pp_rank, pp_size=pp, layer_start=pp_rank * per_stage,
                     layer_end=cfg.n_layers if pp_rank == pp - 1 else (pp_rank + 1) * per_stage)
    if args.shard_of > 1 and world == 1:
        spec = ShardSpec(tp_rank=0, tp_size=args.shard_of)
    pipe, stage_group = None, None
    if pp > 1:
        # every rank creates every group, in the same order: the lanes' stage-to-stage links and the stages' TP groups
        from exo_b200.parallel.comm import PipeComm
        stage_groups = [dist.new_group([s * tp + t for t in range(tp)]) for s in range(pp)]
        lane_groups = [dist.new_group([s * tp + t for s in range(pp)]) for t in range(tp)]
        stage_group = stage_groups[pp_rank]
        pipe = PipeComm(pp_rank, pp, tp_rank, tp, lane_groups[tp_rank])

    def make_comm(kind: str):
        if tp == 1:
            return None, "none"
        if kind == "fused":
            from exo_b200.models.weights import vocab_shard
            from exo_b200.parallel.fused import FusedComm
            c = FusedComm(dev, max_rows=max(min(args.prompt, 4096), 256), hidden=cfg.hidden, vocab_shard=vocab_shard(cfg.vocab, tp),
                          **({"group": stage_group} if stage_group is not None else {}))
            return c, f"fused ({c.transport})"
        from exo_b200.parallel.comm import NcclComm
        return (NcclComm(stage_group) if stage_group is not None else NcclComm()), "nccl"

    want = "nccl" if args.comm == "nccl" else "fused"
    try:
        comm, comm_name = make_comm(want)
    except Exception as e:  # noqa: BLE001
        if args.comm == "fused":
            raise
        if rank == 0:
            print(f"[bench] fused comm unavailable ({e!r}); using NCCL", file=sys.stderr)
        comm, comm_name = make_comm("nccl")

    note(f"comm={comm_name}; building weights")
    # router weights: N(0, 1) for softmax routers (widely spread logits, no two alike); sigmoid routers get N(0, 1/H) so
    # that the LOGITS are N(0, 1): larger ones saturate the sigmoid, every score ties at 1.0 and the top-k then picks
    # the lowest expert ids for every token, i.e. all of one rank's experts and none of the others'
    router_std = None if not cfg.n_experts else (cfg.hidden ** -0.5 if cfg.router == "sigmoid" else 1.0)
    weights = fast_random_weights(cfg, spec, dev, seed=0, router_std=router_std)
    torch.cuda.synchronize()
    note("weights ready")
    max_b = max(args.batch, 1 if args.no_also else args.also_batch)
    MAX_REPEATS = max(1, 2048 // max(1, args.steps))        # bounds the KV each sequence may grow into
    decode_room = 2 * MAX_REPEATS * args.steps + 2 * args.steps + 4 * max(args.warmup, 3) + 64
    per_seq_blocks = -(-(args.prompt + decode_room) // 16)
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

    def agree(v: int) -> int:
        """Rank 0's value on every rank (repeat counts are decided by the leader's clock)."""
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.int64)
        dist.broadcast(t, 0)
        return int(t.item())

    class Rank:
        """This rank's part in the serving topology: the leader schedules and publishes plans, followers execute them."""

        def __init__(self, the_comm):
            self.leader = rank == 0
            if self.leader:
                self.eng = Engine(cfg, weights, spec, the_comm, n_blocks=n_blocks, max_seqs=max(max_b, 8), prefill_chunk=4096,
                                  max_blocks_per_seq=per_seq_blocks, device=dev, seed=0,
                                  plan_sink=(lambda p: chan.send(p, [])) if chan is not None else None, pipe=pipe)
                self.exe = self.eng.exe
            else:
                self.eng = None
                self.exe = Executor(cfg, weights, spec, the_comm, n_blocks=n_blocks, max_blocks_per_seq=per_seq_blocks,
                                    max_tokens_per_step=4096, max_seqs=max(max_b, 8), device=dev, pipe=pipe)

        def run(self, marker: str, fn=None) -> None:
            """Leader: do ``fn`` (which steps the engine / publishes plans), then publish ``marker``.
            Follower: execute published plans until ``marker`` arrives."""
            if self.leader:
                if fn is not None:
                    fn()
                if chan is not None:
                    chan.send(None, [marker])
                return
            while True:
                plan, fin, _stop = chan.recv()
                if plan is not None:
                    self.exe.run(plan)
                if marker in fin:
                    return

    me = Rank(comm)
    rng = np.random.default_rng(1234)
    greedy = dict(temperature=0.0, ignore_eos=True)

    # ---------------- TTFT (one prompt, admission -> first sampled token) ----------------
    def ttft_once(r: "Rank") -> float:
        def go():
            prompt = rng.integers(0, cfg.vocab, args.prompt).tolist()
            rid = r.eng.submit(prompt, SamplingParams(max_tokens=1, **greedy), use_prefix_cache=False)
            got = False
            while not got:
                for o in r.eng.step():
                    got |= o.req_id == rid and o.token is not None
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.run("ttft", go)
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1))

    note("ttft warm-up")
    ttft_once(me)  # warm-up (kernel loading, descriptor caches)
    note("ttft timed")
    ttfts = [ttft_once(me) for _ in range(3)]
    note(f"ttft {ttfts}")
    ttft_ms = min(ttfts)
    K.check_status()

    # ---------------- decode ----------------
    def decode_bench(r: "Rank", B: int, steps: int, warm: int, e2e: bool = True) -> dict:
        warm = max(warm, 3)
        rids: list[str] = []

        def prefill():
            for s in list(r.eng.seqs):
                r.eng.cancel(s)
            rids.extend(r.eng.submit(rng.integers(0, cfg.vocab, args.prompt).tolist(),
                                     SamplingParams(max_tokens=10 ** 6, **greedy), use_prefix_cache=False) for _ in range(B))
            while any(r.eng.seqs[x].in_prefill or not r.eng.seqs[x].output for x in rids):
                r.eng.step()
            for _ in range(warm):
                r.eng.step()
        r.run("prefilled", prefill)
        # estimate the step time on the leader to size the repeats
        barrier()
        t0 = time.perf_counter()
        r.run("probe", lambda: [r.eng.step() for _ in range(3)])
        barrier()
        est_ms = (time.perf_counter() - t0) * 1e3 / 3
        repeats = agree(int(min(MAX_REPEATS, max(1, -(-args.min_timed_s * 1e3 // (est_ms * steps))))))
        note(f"decode B={B}: step ~{est_ms:.2f} ms, {repeats} repeat(s) of {steps} steps")
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # --- end to end: public API, H2D of the plan and D2H of the ids every step ---
        e2e_ms: list[float] = []
        h2d = d2h = 0
        if e2e:
            for _ in range(repeats):
                h0, d0 = r.exe.h2d_bytes, r.exe.d2h_bytes
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r.run("e2e", lambda: [r.eng.step() for _ in range(steps)])
                e1.record()
                barrier()
                e2e_ms.append(max_over_ranks(e0.elapsed_time(e1)))
                h2d, d2h = (r.exe.h2d_bytes - h0) // steps, (r.exe.d2h_bytes - d0) // steps
        # --- device: pre-built plans, tokens chained on device ---
        plans: list[StepPlan] = []
        if r.leader:
            seqs = [r.eng.seqs[x] for x in rids]
            bs = r.eng.alloc.block_size
            total = warm + repeats * steps
            for s in seqs:
                assert r.eng.sched._ensure_blocks(s, s.n_tokens + total + 8)
            mb = max(len(s.blocks) for s in seqs)
            bt = np.zeros((B, mb), np.int32)
            for b, s in enumerate(seqs):
                bt[b, :len(s.blocks)] = s.blocks
            base = np.array([s.n_tokens - 1 for s in seqs], np.int32)
            rows = np.arange(B, dtype=np.int32)
            for i in range(total):
                pos = base + i
                plans.append(StepPlan(n_tokens=B, n_seqs=B, max_q_len=1, flags=FLAG_ALL_GREEDY | FLAG_TOKENS_FROM_PREV,
                                      tokens=np.zeros(B, np.int32), positions=pos, slots=bt[rows, pos // bs] * bs + pos % bs,
                                      cu_q=np.arange(B + 1, dtype=np.int32), seq_lens=pos + 1, logit_rows=rows,
                                      top_k=np.zeros(B, np.int32), temperature=np.zeros(B, np.float32),
                                      top_p=np.ones(B, np.float32), min_p=np.zeros(B, np.float32),
                                      uniform=np.zeros(B, np.float32), prev_rows=rows, block_tables=bt))

        def replay(lo: int, hi: int):
            def go():
                for i in range(lo, hi):
                    if chan is not None:
                        chan.send(plans[i], [])
                    r.exe.run(plans[i])
            return go
        r.run("dev-warm", replay(0, warm))
        launches_before = K.launch_count
        dev_ms: list[float] = []
        for k in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r.run("dev", replay(warm + k * steps, warm + (k + 1) * steps))
            e1.record()
            barrier()
            dev_ms.append(max_over_ranks(e0.elapsed_time(e1)))
        clocks = sampler.stop() if rank == 0 else {}
        K.check_status()
        if r.leader:
            # the device holds the state of the last plan: nothing ran ahead of, or tore, the staged plans
            L = r.exe.last_layout
            got = r.exe.dev[L.seq_lens:L.seq_lens + B].cpu().numpy()
            assert (got == plans[-1].seq_lens).all(), "device-side plan state does not match the last plan"
        d_ms = statistics.median(dev_ms) / steps
        e_ms = statistics.median(e2e_ms) / steps if e2e_ms else float("nan")
        return {"B": B, "dev_ms_per_step": d_ms, "e2e_ms_per_step": e_ms, "dev_tok_s": B / (d_ms / 1e3),
                "e2e_tok_s": B / (e_ms / 1e3) if e2e_ms else None, "h2d": int(h2d), "d2h": int(d2h), "clocks": clocks,
                "repeats": repeats, "timed_s": round(sum(dev_ms) / 1e3, 3),
                "eager_launches": K.launch_count - launches_before}

    main_res = decode_bench(me, args.batch, args.steps, args.warmup)
    # kernels per decode step = launches recorded while the step's graph was captured
    per_step_launches = getattr(me.exe, "launches_per_graph", {}).get(bucket(args.batch, (1, 2, 4, 8, 16, 32, 64, 128, 256)), 0)
    also = None
    if not args.no_also and args.also_batch != args.batch:
        also = decode_bench(me, args.also_batch, max(16, args.steps // 2), args.warmup)

    # ---------------- the same decode loop on the NCCL communicator: the baseline behind vs_baseline ----------------
    base_res = None
    if world > 1 and want == "fused" and not args.no_baseline and comm_name.startswith("fused"):
        note("baseline arm (NCCL communicator)")
        for s in (list(me.eng.seqs) if me.leader else []):
            me.eng.cancel(s)
        me_fused, me = me, None
        me_fused.exe.graphs.clear()
        del me_fused
        torch.cuda.empty_cache()
        nccl_comm, _ = make_comm("nccl")
        base = Rank(nccl_comm)
        base_res = decode_bench(base, args.batch, args.steps, args.warmup, e2e=False)

    if rank == 0:
        out = {
            "metric": f"decode_tok_s_bs{args.batch}", "value": round(main_res["dev_tok_s"], 2), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(main_res["dev_ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(main_res["dev_tok_s"] / base_res["dev_tok_s"], 3) if base_res else None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"model": cfg.name + (f" (REDUCED to {cfg.n_layers} layers: pre-flight, not a result)" if args.layers else "")
                       + (f" (ONE RANK'S SHARD of a {args.shard_of}-way split, no collectives: pre-flight, not a result)" if args.shard_of > 1 and world == 1 else ""),
                       "weights": cfg.quant if cfg.quant != "none" else "bf16",
                       "global_batch": args.batch, "seq_len": args.prompt,
                       "decode_context": f"{args.prompt}+", "parallelism": f"tp{world}" if pp == 1 else f"pp{pp}xtp{tp}", "comm": comm_name,
                       "topology": "rank 0 schedules and publishes each step's plan over shared memory; the other ranks execute it"
                                   if world > 1 else "single process",
                       "l2": "per-step inputs (weights + KV) exceed the 126 MB L2; no explicit flush",
                       "kv": "paged, block 16",
                       "timing": f"median of {main_res['repeats']} repeat(s) of {args.steps} steps ({main_res['timed_s']} s timed)",
                       "baseline": ("same decode loop on the NCCL communicator (projection, ncclAllReduce, residual add, norm): "
                                    f"{base_res['dev_tok_s']:.1f} tok/s" if base_res else
                                    "none at one GPU (no published Llama-3.1-8B number; the baseline arm needs a collective)")},
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
        # Unmap the symmetric arena in order (every rank idle, multicast binding first), then leave without tearing
        # NCCL down: destroying a communicator whose collectives were captured in still-alive CUDA graphs blocked for
        # minutes (both ranks sat in destroy_process_group).
        dist.barrier()
        torch.cuda.synchronize()
        if comm is not None and hasattr(comm, "close"):
            try:
                comm.close()
            except Exception as e:  # noqa: BLE001
                print(f"[bench r{rank}] arena teardown: {e!r}", file=sys.stderr)
        if chan is not None:
            chan.close()
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
