"""Micro-benchmark of the tensor-parallel collectives: peer-memory all-reduce against NCCL, and the
row-parallel projection with the hand-over against projection + all-reduce.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m exo_b200.utils.bench_comm

Every case is captured in a CUDA graph of ``reps`` back-to-back calls, timed with CUDA events on
every rank, and the maximum over ranks is reported.  For an all-reduce of S bytes over N GPUs the
roofline is the two-shot traffic ``2 (N-1)/N * S`` per GPU and direction over the measured peer-copy
bandwidth (770 GB/s); at decode sizes the number that matters is the latency.  A multi-rank program
cannot be run under ncu on this kind of box, so these event timings are the evidence for the
collectives.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def timed(fn, reps: int, iters: int = 5) -> float:
    """ms per call: graph of ``reps`` calls, best of ``iters`` replays, max over ranks."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    t = torch.tensor([best], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import cuda as K
    from ..parallel.comm import NcclComm
    from ..parallel.fused import FusedComm, Reduction
    K.load()
    H = a.hidden
    fused = FusedComm(dev, max_rows=4096, hidden=H, vocab_shard=1024)
    nccl = NcclComm()
    g = torch.Generator(device="cuda").manual_seed(rank)

    def say(msg: str) -> None:
        if rank == 0:
            print(msg, flush=True)

    say(f"ranks {world}; transport {fused.transport}; link basis {LINK_GBS:.0f} GB/s per direction (measured peer copy)")
    from .. import ops
    nw = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    for rows in (4, 32, 256, 2048, 4096):
        x = (torch.randn(rows, H, device="cuda", generator=g) * 0.1).bfloat16()
        res = torch.zeros_like(x)
        S = rows * H * 2
        reps = 64 if rows <= 256 else 8

        def ours():
            # what the model does after a row-parallel projection: the partial sits in the arena, one kernel forms
            # residual + sum over ranks and the RMSNorm of it
            buf, parity = fused.partial_out(rows, H)
            buf.copy_(x)
            return Reduction(fused, parity, res, rows, H).norm(nw, 1e-5)

        def base():
            return ops.rmsnorm(nccl.all_reduce(x, res), nw, 1e-5)[0]
        t_f = timed(ours, reps)
        t_c = timed(lambda: fused.region(0, 0, rows, H).copy_(x), reps)        # the staging copy alone (a GEMM writes there directly)
        t_n = timed(base, reps)
        two = fused.two_shot(rows, H)
        wire = (2 * (world - 1) / world * S) if two else ((world - 1) * S)      # bytes leaving each GPU
        ideal_ms = wire / (LINK_GBS * 1e9) * 1e3
        say(f"sum over ranks + residual + RMSNorm [{rows} x {H}] bf16 ({S >> 10} KiB, {'two' if two else 'one'}-shot): "
            f"fused kernel {(t_f - t_c) * 1e3:8.1f} us (+{t_c * 1e3:.1f} us staging copy)   NCCL all-reduce + norm kernel "
            f"{t_n * 1e3:8.1f} us   link time {ideal_ms * 1e3:7.1f} us -> {ideal_ms / max(t_f - t_c, 1e-9):4.2f} of the link roofline")
    # row-parallel down projection of a decode step: hand-over (no collective kernel; the sum is formed by the consumer)
    # against projection + all-reduce.  The consumer here is the next layer's RMSNorm + qkv projection.
    Kd = a.ffn // world
    w_down = (torch.randn(H, Kd, device="cuda", generator=g) * 0.02).bfloat16()
    w_qkv = (torch.randn(H + 2 * (H // 4), H, device="cuda", generator=g) * 0.02).bfloat16()
    for rows in (1, 2):
        x = (torch.randn(rows, Kd, device="cuda", generator=g) * 0.1).bfloat16()
        res = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)

        def pair(comm):
            h = comm.row_linear(x, w_down, res)
            return ops.norm_linear(h, nw, 1e-5, w_qkv)
        fused.use_handover = True
        t_h = timed(lambda: pair(fused), 64)
        fused.use_handover = False
        t_a = timed(lambda: pair(fused), 64)
        t_n = timed(lambda: pair(nccl), 64)
        fused.use_handover = True
        say(f"down-proj [{rows} x {Kd}]x[{Kd} x {H}] + all-reduce + RMSNorm + qkv: hand-over {t_h * 1e3:7.1f} us   "
            f"peer-memory all-reduce kernel {t_a * 1e3:7.1f} us   NCCL {t_n * 1e3:7.1f} us")
    fused.check()
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
