"""Tensor-parallel communicators behind one interface (``row_linear`` / ``all_reduce`` /
``gather_vocab`` / ``send`` / ``recv``).

* ``NcclComm``  – the baseline: local GEMM, then ``ncclAllReduce`` through ``torch.distributed``.
  It mirrors what the reference does with ``mx.distributed.all_sum`` after every row-parallel
  projection (``src/exo/worker/engines/mlx/auto_parallel.py:465-469``, ``:641``, ``:647``).
* ``FusedComm`` (``exo_b200.parallel.fused``) – the product: the projection, the exchange over
  NVLink peer memory and the reduction (+ residual add) run as one kernel sequence on
  symmetric buffers, no NCCL on the hot path.
* ``GlooComm``  – CPU ranks for host-side tests (``gloo`` backend, world size > 1).

Pipeline-parallel activation hops stay on NCCL/gloo point-to-point (``send`` / ``recv``), as
in the reference's ``PipelineFirstLayer`` / ``PipelineLastLayer`` (``auto_parallel.py:132-194``).
"""
from __future__ import annotations

from collections import deque

import torch
import torch.distributed as dist

from .. import ops


class DistComm:
    """Collectives through a ``torch.distributed`` process group (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_collectives = 0

    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype == torch.bfloat16 and x.device.type == "cpu":
            y = x.float()
            dist.all_reduce(y, group=self.group)
            x = y.to(torch.bfloat16)
        else:
            x = x.contiguous()
            dist.all_reduce(x, group=self.group)
        self.n_collectives += 1
        return x if residual is None else x + residual

    def all_reduce_stat(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        return x

    def row_linear(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.all_reduce(ops.linear(x, w), residual)

    def row_sum(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.all_reduce(x, residual)

    def gather_vocab(self, logits_local: torch.Tensor) -> torch.Tensor:
        logits_local = logits_local.contiguous()
        parts = [torch.empty_like(logits_local) for _ in range(self.size)]
        dist.all_gather(parts, logits_local, group=self.group)
        self.n_collectives += 1
        return torch.cat(parts, dim=-1)

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x.contiguous(), dst, group=self.group)

    def recv(self, x: torch.Tensor, src: int) -> None:
        dist.recv(x, src, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)


NcclComm = DistComm
GlooComm = DistComm


class PipeComm:
    """Pipeline-stage links of one tensor-parallel lane: activations hop stage to stage, the ids
    sampled on the last stage go back to every stage (the first needs them as next-step input,
    global rank 0 for the scheduler).  World layout: ``rank = pp_rank * tp_size + tp_rank``.

    The reference moves the hidden state with ``send`` / ``recv_like`` between
    ``PipelineLastLayer`` and ``PipelineFirstLayer`` and then all-gathers the final stage's output
    so that every rank can sample (``auto_parallel.py:132-194``); here only the sampled ids
    (4 bytes per sequence) travel back.
    """

    RX_SLOTS = 3

    def __init__(self, pp_rank: int, pp_size: int, tp_rank: int, tp_size: int, lane_group=None):
        self.pp_rank, self.pp_size = pp_rank, pp_size
        self.lane_group = lane_group          # the pp_size ranks that share this tp_rank
        g = lambda stage: stage * tp_size + tp_rank
        self.prev = g(pp_rank - 1) if pp_rank > 0 else None
        self.next = g(pp_rank + 1) if pp_rank < pp_size - 1 else None
        self.last = g(pp_size - 1)
        self.n_hops = 0
        # CUDA: hops run beside the compute stream.  Receives land in a ring of buffers this object owns (memory the
        # caching allocator may hand out again is not safe to fill from another stream), each reusable once the step
        # that read it has been enqueued and its event has passed; sends are started when the stage's output is ready
        # and the compute stream goes on without waiting for the peer to take them.
        self.stream = None
        self.rx: list[torch.Tensor] = []
        self.rx_done: list = [None] * self.RX_SLOTS
        self.rx_last = -1
        self.sends: deque = deque()

    def _ring(self, T: int, hidden: int, dtype, device) -> torch.Tensor:
        if self.stream is None:
            self.stream = torch.cuda.Stream(device=device)
        if not self.rx or self.rx[0].shape[0] < T or self.rx[0].dtype != dtype:
            rows = max(T, self.rx[0].shape[0] if self.rx else 0)
            torch.cuda.current_stream(device).synchronize()      # rare: the first step, or a larger chunk than any before
            self.stream.synchronize()
            self.rx = [torch.empty(rows, hidden, dtype=dtype, device=device) for _ in range(self.RX_SLOTS)]
            self.rx_done = [None] * self.RX_SLOTS
        self.rx_last = (self.rx_last + 1) % self.RX_SLOTS
        return self.rx[self.rx_last][:T]

    def recv_hidden(self, T: int, hidden: int, dtype, device) -> torch.Tensor:
        """The residual stream ``[T, hidden]`` of this step from the previous stage."""
        device = torch.device(device)
        self.n_hops += 1
        if device.type != "cuda":
            buf = torch.empty(T, hidden, dtype=torch.float32 if dtype == torch.bfloat16 else dtype)   # gloo has no bf16
            dist.recv(buf, self.prev)
            return buf.to(dtype)
        buf = self._ring(T, hidden, dtype, device)
        done = self.rx_done[self.rx_last]
        if done is not None:
            self.stream.wait_event(done)
        with torch.cuda.stream(self.stream):
            work = dist.irecv(buf, self.prev)
        work.wait()                          # the compute stream waits for the data, the host does not
        return buf

    def consumed(self) -> None:
        """The step that read the last received buffer has been enqueued on the current stream."""
        if self.stream is not None and self.rx_last >= 0 and self.rx:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.rx[0].device))
            self.rx_done[self.rx_last] = ev

    def send_hidden(self, h: torch.Tensor) -> None:
        self.n_hops += 1
        if h.device.type != "cuda":
            dist.send((h.float() if h.dtype == torch.bfloat16 else h).contiguous(), self.next)
            return
        if self.stream is None:
            self.stream = torch.cuda.Stream(device=h.device)
        h = h.contiguous()
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(h.device))
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            work = dist.isend(h, self.next)
        h.record_stream(self.stream)
        self.sends.append((work, h))         # the tensor stays referenced until the transfer is known to be over
        while len(self.sends) > 4:
            old, _ = self.sends.popleft()
            old.wait()

    def share_ids(self, ids: torch.Tensor) -> torch.Tensor:
        dist.broadcast(ids, src=self.last, group=self.lane_group)
        return ids
