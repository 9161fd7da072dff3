"""Tensor-parallel communicator on NVLink peer memory: the product path.

Each rank allocates one arena, exports it with CUDA IPC, and maps every peer's arena
(handles travel once through ``torch.distributed.all_gather_object``).  From then on the
collectives of the decode / prefill hot path are our own kernels storing into peer HBM through
NVSwitch — no NCCL call per layer.  This replaces the ``mx.distributed.all_sum`` the reference
issues after every row-parallel projection (``src/exo/worker/engines/mlx/auto_parallel.py:465-469``
and its ``ring`` / ``jaccl`` transports, ``src/exo/worker/engines/mlx/utils_mlx.py:104-143``).

Device-side waits are bounded (2 s): a rank whose peer never signals records an error code that
``check()`` turns into ``CollectiveTimeout`` on the host; nothing spins forever.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import ops
from ..ops import cuda as K


class CollectiveTimeout(RuntimeError):
    pass


class _RawBuffer:
    """Wraps a raw device pointer so that ``torch.as_tensor`` can view it (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class FusedComm:
    def __init__(self, device: torch.device, max_rows: int, hidden: int, vocab_shard: int, group=None,
                 max_gather_rows: int = 256):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        lib = K.load()
        for name, (res, args) in {
            "exo_symm_alloc": (C.c_void_p, [C.c_size_t]), "exo_symm_free": (C.c_int, [C.c_void_p]),
            "exo_symm_handle": (C.c_int, [C.c_void_p, C.c_void_p]), "exo_symm_open": (C.c_void_p, [C.c_void_p]),
            "exo_symm_close": (C.c_int, [C.c_void_p]), "exo_comm_header_bytes": (C.c_size_t, []),
            "exo_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_size_t]),
            "exo_comm_status": (C.c_int, []),
            "exo_allreduce_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p]),
            "exo_allgather_cols_bf16": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
        }.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        self.lib = lib
        n = self.size
        hdr = lib.exo_comm_header_bytes()
        one_shot = 512 << 10
        two_shot = 2 * (max_rows * hidden * 2 + n - 1) // n
        self.slot_bytes = (max(one_shot, two_shot) + 4095) // 4096 * 4096
        self.max_elems = max_rows * hidden
        self.vocab_shard = vocab_shard
        self.max_gather_rows = max_gather_rows
        self.gather_off = hdr + 2 * n * self.slot_bytes
        gather_bytes = max_gather_rows * n * vocab_shard * 2
        self.arena_bytes = self.gather_off + gather_bytes
        torch.cuda.set_device(device)
        self.local = lib.exo_symm_alloc(self.arena_bytes)
        if not self.local:
            raise RuntimeError(f"cannot allocate {self.arena_bytes >> 20} MiB symmetric arena")
        handle = C.create_string_buffer(64)
        K._chk(lib.exo_symm_handle(self.local, handle), "ipc handle")
        handles: list[bytes | None] = [None] * n
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peers: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peers.append(self.local)
            else:
                p = lib.exo_symm_open(C.create_string_buffer(h, 64))
                if not p:
                    raise RuntimeError(f"rank {self.rank}: cannot map arena of rank {r} (no peer access?)")
                self.peers.append(p)
        arr = (C.c_void_p * n)(*self.peers)
        K._chk(lib.exo_comm_init(arr, n, self.rank, self.slot_bytes, self.gather_off), "comm init")
        dist.barrier(group=group)
        raw = torch.as_tensor(_RawBuffer(self.local + self.gather_off, gather_bytes), device=device)
        self.gather_buf = raw.view(torch.bfloat16)
        self._ar = 0
        self.n_collectives = 0

    # ---- collectives ----
    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual + sum over ranks of x`` (bf16), identical bits on every rank."""
        x = x.contiguous()
        if x.dtype != torch.bfloat16 or x.numel() % 8:
            raise K.KernelError("fused all-reduce takes bf16 tensors whose size is a multiple of 8")
        if x.numel() > self.max_elems:
            # larger than one arena slot (a long prefill chunk): reduce it in row blocks that fit
            if x.dim() != 2 or x.shape[1] > self.max_elems:
                raise K.KernelError(f"tensor of {x.numel()} elements exceeds the arena slot ({self.max_elems})")
            rows = max(8, (self.max_elems // x.shape[1]) // 8 * 8)
            parts = [self.all_reduce(x[r:r + rows], None if residual is None else residual[r:r + rows])
                     for r in range(0, x.shape[0], rows)]
            return torch.cat(parts, dim=0)
        out = torch.empty_like(x)
        parity = self._ar & 1
        self._ar += 1
        K._chk(self.lib.exo_allreduce_bf16(x.data_ptr(), None if residual is None else residual.data_ptr(),
                                           out.data_ptr(), x.numel(), parity, K._st()), "allreduce")
        K._count()
        self.n_collectives += 1
        return out

    def row_linear(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.all_reduce(ops.linear(x, w), residual)

    def gather_vocab(self, logits_local: torch.Tensor) -> torch.Tensor:
        rows, cols = logits_local.shape
        if cols != self.vocab_shard or rows > self.max_gather_rows:
            raise K.KernelError("gather shape does not match the arena")
        logits_local = logits_local.contiguous()
        K._chk(self.lib.exo_allgather_cols_bf16(logits_local.data_ptr(), rows, cols, 2, K._st()), "allgather")
        K._count()
        self.n_collectives += 1
        return self.gather_buf[:rows * self.size * cols].view(rows, self.size * cols)

    def check(self) -> None:
        code = self.lib.exo_comm_status()
        if code:
            raise CollectiveTimeout(f"rank {self.rank}: device-side wait on a peer timed out (code {code})")

    # ---- point to point (pipeline stages) stays on NCCL ----
    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x.contiguous(), dst, group=self.group)

    def recv(self, x: torch.Tensor, src: int) -> None:
        dist.recv(x, src, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for r, p in enumerate(self.peers):
            if r != self.rank and p:
                self.lib.exo_symm_close(p)
        dist.barrier(group=self.group)
        self.lib.exo_symm_free(self.local)
        self.peers = []
