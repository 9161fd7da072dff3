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

    def __init__(self, pp_rank: int, pp_size: int, tp_rank: int, tp_size: int, lane_group=None):
        self.pp_rank, self.pp_size = pp_rank, pp_size
        self.lane_group = lane_group          # the pp_size ranks that share this tp_rank
        g = lambda stage: stage * tp_size + tp_rank
        self.prev = g(pp_rank - 1) if pp_rank > 0 else None
        self.next = g(pp_rank + 1) if pp_rank < pp_size - 1 else None
        self.last = g(pp_size - 1)
        self.n_hops = 0

    def recv_hidden(self, like: torch.Tensor) -> torch.Tensor:
        buf = like.float() if (like.device.type == "cpu" and like.dtype == torch.bfloat16) else like
        dist.recv(buf, self.prev)
        self.n_hops += 1
        return buf.to(like.dtype)

    def send_hidden(self, h: torch.Tensor) -> None:
        if h.device.type == "cpu" and h.dtype == torch.bfloat16:
            h = h.float()
        dist.send(h.contiguous(), self.next)
        self.n_hops += 1

    def share_ids(self, ids: torch.Tensor) -> torch.Tensor:
        dist.broadcast(ids, src=self.last, group=self.lane_group)
        return ids
