"""Run a few decode (or prefill) steps eagerly inside an NVTX range, for kernel profilers.

    python -m exo_b200.utils.profile_step --model llama-3.1-8b --batch 1 --context 2048 --steps 2
    ncu --nvtx --nvtx-include "exo_step/" --metrics gpu__time_duration.sum --clock-control none \
        python -m exo_b200.utils.profile_step --batch 32 --steps 1

The KV cache is filled with random values instead of running a real prefill, and CUDA graphs
are off so that every kernel shows up as its own launch.  ``--layers`` shrinks the model for
multi-pass captures (``--set full``) that must stay small.  The range also prints per-step
device time measured with CUDA events when no profiler is attached.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from ..engine.executor import Executor
from ..engine.plan import FLAG_ALL_GREEDY, StepPlan
from ..models.config import preset
from ..models.weights import ShardSpec, fast_random_weights


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"])
    ap.add_argument("--graphs", action="store_true")
    ap.add_argument("--tp-shard", type=int, default=1,
                    help="run ONE rank's share of an N-way tensor-parallel model on this GPU (heads, FFN and vocabulary "
                         "divided by N, no communication): every kernel then has the shape it has under TP-N")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = preset(a.model)
    if a.layers:
        cfg.n_layers = a.layers
    if a.tp_shard > 1:
        n = a.tp_shard
        cfg.n_heads //= n
        cfg.n_kv_heads = max(1, cfg.n_kv_heads // n)
        cfg.ffn //= n
        cfg.vocab = -(-cfg.vocab // n)
    w = fast_random_weights(cfg, ShardSpec(), dev)
    bs = 16
    B = a.batch if a.mode == "decode" else 1
    per = -(-(a.context + a.steps + a.warmup + 32) // bs)
    exe = Executor(cfg, w, n_blocks=B * per + 8, max_blocks_per_seq=per, max_tokens_per_step=max(a.context, 256),
                   max_seqs=max(B, 8), device=dev, use_graphs=a.graphs)
    for kc, vc in exe.kv.layers.values():
        kc.normal_(0, 0.5)
        if vc is not None:
            vc.normal_(0, 0.5)
    bt = (np.arange(B * per, dtype=np.int32).reshape(B, per) + 1)
    rng = np.random.default_rng(0)

    def plan(i: int) -> StepPlan:
        if a.mode == "decode":
            pos = np.full(B, a.context + i, np.int32)
            rows = np.arange(B, dtype=np.int32)
            return StepPlan(B, B, 1, FLAG_ALL_GREEDY, rng.integers(0, cfg.vocab, B).astype(np.int32), pos,
                            bt[rows, pos // bs] * bs + pos % bs, np.arange(B + 1, dtype=np.int32), pos + 1, rows,
                            np.zeros(B, np.int32), np.zeros(B, np.float32), np.ones(B, np.float32),
                            np.zeros(B, np.float32), np.zeros(B, np.float32), np.full(B, -1, np.int32), bt)
        T = a.context
        pos = np.arange(T, dtype=np.int32)
        return StepPlan(T, 1, T, FLAG_ALL_GREEDY, rng.integers(0, cfg.vocab, T).astype(np.int32), pos,
                        bt[0, pos // bs] * bs + pos % bs, np.array([0, T], np.int32), np.array([T], np.int32),
                        np.array([T - 1], np.int32), np.zeros(1, np.int32), np.zeros(1, np.float32),
                        np.ones(1, np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32),
                        np.full(1, -1, np.int32), bt[:1])

    for i in range(a.warmup):
        exe.run(plan(i))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.nvtx.range_push("exo_step")
    e0.record()
    for i in range(a.steps):
        exe.run(plan(a.warmup + i))
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    print(f"{a.mode} batch={B} context={a.context} layers={cfg.n_layers} tp-shard={a.tp_shard}: "
          f"{e0.elapsed_time(e1) / a.steps:.3f} ms/step (eager={not a.graphs})")


if __name__ == "__main__":
    main()
