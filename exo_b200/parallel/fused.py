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
import os

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


HANDOVER_ROWS = 256           # rows of the residual stream one hand-over slot holds (decode batches)


class Handover:
    """The not-yet-reduced output of a row-parallel projection: partials of all ranks sit in this rank's
    staging slots.  ``norm_linear`` consumes it inside the next projection; ``value()`` gives the tensor
    (running the stand-alone finish kernel if nobody consumed it)."""

    def __init__(self, comm: "FusedComm", parity: int, residual: torch.Tensor | None, rows: int, cols: int):
        self.comm, self.parity, self.residual, self.shape = comm, parity, residual, (rows, cols)
        ref = residual if residual is not None else None
        self.out = torch.empty(rows, cols, dtype=torch.bfloat16, device=comm.device) if ref is None else torch.empty_like(ref)
        self.done = False

    def norm_linear(self, norm_w, eps, w, bias=None, swiglu=False):
        M, Kd = self.shape
        N = w.shape[0]
        lib = self.comm.lib
        if not self.done and os.environ.get("EXO_TP_HANDOVER_CONSUME") == "0":
            return K.linear(self.value(), w, bias, None, norm_w, eps, swiglu)      # measurement aid: stand-alone finish kernel
        if not self.done and M > 2 and Kd % 8 == 0:
            # batched decode: one kernel finishes the reduction, leaves the residual stream and the normalised rows
            xn = torch.empty_like(self.out)
            K._chk(lib.exo_tp_handover_rmsnorm(K._ptr(self.residual), norm_w.data_ptr(), eps, self.out.data_ptr(), xn.data_ptr(),
                                               M, Kd, self.parity, K._st()), "handover rmsnorm")
            K._count()
            self.done = True
            return K.linear(xn, w, bias, None, None, 0.0, swiglu)
        if self.done or not isinstance(w, torch.Tensor) or not lib.exo_gemv_stream_supported(M, N, Kd, int(swiglu)):
            return K.linear(self.value(), w, bias, None, norm_w, eps, swiglu)
        y = torch.empty(M, N // 2 if swiglu else N, dtype=torch.bfloat16, device=self.out.device)
        K._chk(lib.exo_gemv_stream_tp(None, w.data_ptr(), K._ptr(bias), y.data_ptr(), K._ptr(norm_w), eps, M, N, Kd, int(swiglu),
                                      2, self.parity, K._ptr(self.residual), self.out.data_ptr(), K._st()), "gemv_stream_tp consume")
        K._count()
        self.done = True
        return y

    def value(self) -> torch.Tensor:
        if not self.done:
            n = self.shape[0] * self.shape[1]
            K._chk(self.comm.lib.exo_tp_handover_finish(K._ptr(self.residual), self.out.data_ptr(), n, self.parity, K._st()),
                   "handover finish")
            K._count()
            self.done = True
        return self.out


def resolve(h):
    """A tensor for ``h``: hand-overs are finished, tensors pass through."""
    return h.value() if isinstance(h, Handover) else h


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
            "exo_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t]),
            "exo_comm_handover_bytes": (C.c_size_t, [C.c_int, C.c_size_t]),
            "exo_tp_handover_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                  C.c_int, C.c_void_p]),
            "exo_gemm_bf16_tp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_void_p]),
            "exo_tp_handover_finish": (C.c_int, [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p]),
            "exo_gemv_stream_tp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int,
                                             C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
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
        self.handover_off = (self.gather_off + gather_bytes + 4095) // 4096 * 4096
        self.handover_slot = (HANDOVER_ROWS * hidden * 2 + 4095) // 4096 * 4096
        self.arena_bytes = self.handover_off + lib.exo_comm_handover_bytes(n, self.handover_slot)
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
        K._chk(lib.exo_comm_init(arr, n, self.rank, self.slot_bytes, self.gather_off, self.handover_off,
                                 self.handover_slot), "comm init")
        dist.barrier(group=group)
        raw = torch.as_tensor(_RawBuffer(self.local + self.gather_off, gather_bytes), device=device)
        self.gather_buf = raw.view(torch.bfloat16)
        self._ar = 0
        self._ho = 0             # hand-overs issued so far (parity = low bit)
        self.n_collectives = 0
        self.n_handovers = 0
        self.use_handover = os.environ.get("EXO_DISABLE_TP_HANDOVER") != "1"
        # the GEMM-epilogue variant (batches > 2) measured slower than GEMM + all-reduce kernel: off unless asked for
        self.handover_gemm = os.environ.get("EXO_TP_HANDOVER_GEMM") == "1"

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

    def row_linear(self, x: torch.Tensor, w: torch.Tensor, residual=None):
        """``residual + all-reduce(x @ w.T)``.  At decode batch sizes the projection itself stores its rows
        into every rank's staging slot and a :class:`Handover` is returned: the next ``norm_linear`` (or
        ``resolve``) forms the sum, so no collective kernel is launched."""
        residual = resolve(residual)
        M, Kd = x.shape
        N = w.shape[0]
        fits = (self.use_handover and x.dtype == torch.bfloat16 and 0 < M and M * N * 2 <= self.handover_slot
                and isinstance(w, torch.Tensor))       # block-scaled fp8 weights take the GEMM + all-reduce path
        if fits and M <= 2 and K.use_stream_gemv and self.lib.exo_gemv_stream_supported(M, N, Kd, 0):
            K.ensure_stream_init(x.device)
            parity = self._ho & 1
            self._ho += 1
            x = x.contiguous()
            y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)      # this rank's partial (pushed by the kernel's last CTA)
            K._chk(self.lib.exo_gemv_stream_tp(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), None, 0.0, M, N, Kd, 0, 1, parity,
                                               None, None, K._st()), "gemv_stream_tp push")
            K._count()
            self.n_handovers += 1
            return Handover(self, parity, residual, M, N)
        if (fits and self.handover_gemm and M > K.SMALL_M and K.gemm_impl is not None and Kd >= 64 and Kd % 8 == 0
                and N % 8 == 0):
            # batched decode: the tcgen05 GEMM's epilogue does the peer stores
            K.ensure_gemm_init(x.device)
            parity = self._ho & 1
            self._ho += 1
            x = x.contiguous()
            splits = self.lib.exo_gemm_splits(M, N, Kd)
            while splits > 1 and splits * M * N > K.GEMM_PARTIAL_FLOATS:
                splits -= 1
            K._chk(self.lib.exo_gemm_bf16_tp(x.data_ptr(), w.data_ptr(), None, M, N, Kd, splits, parity, K._st()), "gemm_tp push")
            K._count()
            self.n_handovers += 1
            return Handover(self, parity, residual, M, N)
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
