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
