"""Tensor-parallel communicator on NVLink symmetric memory: the product path.

Each rank owns one arena.  Where the driver allows it the arena is a virtual-memory allocation whose
file descriptor travels to the peers over a Unix socket, every rank maps every arena, and all of
them are bound to one NVLink multicast object, so that a kernel can read the SUM of a buffer over all
ranks with one ``multimem.ld_reduce`` (NVSwitch forms it) or write all ranks with one ``multimem.st``.
Otherwise the arena is a ``cudaMalloc`` block shared through CUDA IPC and the same kernels use plain
peer loads and stores.  From then on the collectives of the decode / prefill hot path are our own
kernels — no NCCL call per layer.  This replaces the ``mx.distributed.all_sum`` the reference issues
after every row-parallel projection (``src/exo/worker/engines/mlx/auto_parallel.py:465-469``) and its
``ring`` / ``jaccl`` transports (``src/exo/worker/engines/mlx/utils_mlx.py:104-143``).

Three forms of "row-parallel projection, then sum over ranks":

* decode batches up to 64 rows: the projection kernel itself (streaming GEMV, or the GEMM's epilogue) sends its
  rows to every rank as flag-in-data words, one ``multimem.st`` per 8 bytes; the consumer polls the words it
  needs (:class:`Handover`).  One one-way trip per collective, no flag, no fence; for one or two rows the
  consumer is the next RMSNorm + GEMV's prologue, so no collective kernel runs at all;
* larger batches: the GEMM writes its partial into this rank's own arena and ONE kernel forms
  ``residual + sum`` and the RMSNorm of it, reading the sum through the switch (:class:`Reduction`);
* prefill chunks: the same kernel in its two-shot form (each rank reduces and normalises 1/N of the
  rows and broadcasts them).

Device-side waits are bounded (``EXO_COLLECTIVE_TIMEOUT_US``): a rank whose peer never signals
records a code in a host-mapped status word that ``check()`` turns into ``CollectiveTimeout``.
"""
from __future__ import annotations

import ctypes as C
import os
import socket
import uuid

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


LL_ROWS = 64                  # largest decode batch handed over with flag-in-data words (one one-way trip per collective)
ONE_SHOT_MAX_BYTES = 4 << 20  # (n - 1) * tensor bytes above which the reduction goes two-shot

_SIGS = {
    "exo_symm_alloc": (C.c_void_p, [C.c_size_t]), "exo_symm_free": (C.c_int, [C.c_void_p]),
    "exo_symm_handle": (C.c_int, [C.c_void_p, C.c_void_p]), "exo_symm_open": (C.c_void_p, [C.c_void_p]),
    "exo_symm_close": (C.c_int, [C.c_void_p]), "exo_comm_header_bytes": (C.c_size_t, []),
    "exo_comm_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int] + [C.c_size_t] * 8),
    "exo_comm_reset": (C.c_int, []),
    "exo_gemm_bf16_tp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_void_p]),
    "exo_gemm_fp8w_tp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_void_p]),
    "exo_tp_ll_finish": (C.c_int, [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p]),
    "exo_tp_ll_push": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "exo_tp_ll_reduce_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p]),
    "exo_gemv_stream_tp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int,
                                     C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "exo_comm_status": (C.c_int, []),
    "exo_allreduce_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_void_p]),
    "exo_allgather_cols_bf16": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "exo_reduce_norm_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_void_p]),
    "exo_gather_rows_bf16": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "exo_comm_region": (C.c_void_p, [C.c_int, C.c_int]),
    "exo_comm_has_multicast": (C.c_int, []),
    "exo_vmm_supported": (C.c_int, []), "exo_vmm_granularity": (C.c_size_t, [C.c_int, C.c_int]),
    "exo_vmm_alloc": (C.c_void_p, [C.c_size_t, C.POINTER(C.c_int)]), "exo_vmm_import": (C.c_void_p, [C.c_int, C.c_size_t]),
    "exo_mc_create": (C.c_ulonglong, [C.c_size_t, C.c_int, C.POINTER(C.c_int)]), "exo_mc_import": (C.c_ulonglong, [C.c_int]),
    "exo_mc_add_device": (C.c_int, [C.c_ulonglong]),
    "exo_mc_bind_and_map": (C.c_void_p, [C.c_ulonglong, C.c_void_p, C.c_size_t]),
    "exo_vmm_unmap": (C.c_int, [C.c_void_p]),
    "exo_set_collective_timeout_us": (C.c_int, [C.c_long]),
}


def bind(lib: C.CDLL) -> C.CDLL:
    """Declare the signatures of the communicator's entry points on the loaded kernel library."""
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def arena_layout(lib, n: int, max_rows: int, hidden: int, vocab_shard: int, max_gather_rows: int) -> dict:
    """Byte offsets of the arena's regions (identical on every rank)."""
    hdr = lib.exo_comm_header_bytes()
    one_shot = 512 << 10
    two_shot = 2 * (max_rows * hidden * 2 + n - 1) // n
    slot = (max(one_shot, two_shot) + 4095) // 4096 * 4096
    gather_off = hdr + 2 * n * slot
    gather_bytes = max_gather_rows * n * vocab_shard * 2
    x_off = (gather_off + gather_bytes + 4095) // 4096 * 4096
    x_bytes = (max_rows * hidden * 2 + 4095) // 4096 * 4096
    h_off = x_off + 2 * x_bytes
    n_off = h_off + 2 * x_bytes
    ll_off = n_off + 2 * x_bytes
    ll_slot = (LL_ROWS * hidden * 4 + 4095) // 4096 * 4096      # 8-byte words of two bf16 values + sequence number
    return dict(slot=slot, gather_off=gather_off, gather_bytes=gather_bytes, x_off=x_off, x_bytes=x_bytes, h_off=h_off, n_off=n_off,
                ll_off=ll_off, ll_slot=ll_slot, total=ll_off + 2 * n * ll_slot)


class Handover:
    """The not-yet-reduced output of a row-parallel projection of a decode step: every rank's rows sit in this
    rank's slots as flag-in-data words (two bf16 values and the hand-over's sequence number per 8-byte store), sent
    by the projection kernel itself.  ``norm_linear`` consumes them: for one or two rows inside the next streaming
    projection's prologue (no kernel in between), for larger batches in one reduce + RMSNorm kernel.  ``value()``
    gives the reduced tensor (running the stand-alone kernel if nobody consumed the hand-over)."""

    def __init__(self, comm: "FusedComm", parity: int, residual: torch.Tensor | None, rows: int, cols: int):
        self.comm, self.parity, self.residual, self.shape = comm, parity, residual, (rows, cols)
        ref = residual if residual is not None else None
        self.out = torch.empty(rows, cols, dtype=torch.bfloat16, device=comm.device) if ref is None else torch.empty_like(ref)
        self.done = False

    def norm(self, norm_w, eps) -> torch.Tensor:
        """RMSNorm of the reduced residual stream (which ``value()`` then returns), one kernel."""
        if self.done:
            return K.rmsnorm(self.out, norm_w, eps)[0]
        M, Kd = self.shape
        xn = torch.empty_like(self.out)
        K._chk(self.comm.lib.exo_tp_ll_reduce_norm(K._ptr(self.residual), norm_w.data_ptr(), float(eps), self.out.data_ptr(),
                                                  xn.data_ptr(), M, Kd, self.parity, K._st()), "ll reduce norm")
        K._count()
        self.done = True
        return xn

    def norm_linear(self, norm_w, eps, w, bias=None, swiglu=False):
        M, Kd = self.shape
        N = w.shape[0]
        lib = self.comm.lib
        if self.done:
            return K.linear(self.out, w, bias, None, norm_w, eps, swiglu)
        if M > 2 or not isinstance(w, torch.Tensor) or not lib.exo_gemv_stream_supported(M, N, Kd, int(swiglu)):
            return K.linear(self.norm(norm_w, eps), w, bias, None, None, 0.0, swiglu)
        y = torch.empty(M, N // 2 if swiglu else N, dtype=torch.bfloat16, device=self.out.device)
        K._chk(lib.exo_gemv_stream_tp(None, w.data_ptr(), K._ptr(bias), y.data_ptr(), K._ptr(norm_w), eps, M, N, Kd, int(swiglu),
                                      2, self.parity, K._ptr(self.residual), self.out.data_ptr(), K._st()), "gemv_stream_tp consume")
        K._count()
        self.done = True
        return y

    def value(self) -> torch.Tensor:
        if not self.done:
            n = self.shape[0] * self.shape[1]
            K._chk(self.comm.lib.exo_tp_ll_finish(K._ptr(self.residual), self.out.data_ptr(), n, self.parity, K._st()),
                   "handover finish")
            K._count()
            self.done = True
        return self.out


class Reduction:
    """A row-parallel projection's partial sitting in this rank's arena, not yet summed over the ranks.

    The first consumer decides the kernel: ``norm_linear`` / ``norm`` run the fused ``residual + sum`` + RMSNorm
    kernel, ``value()`` alone runs it without the norm.  In the two-shot form (prefill chunks) each rank reduces
    and normalises 1/N of the rows; the normalised rows are broadcast, while the residual stream stays SHARDED by
    rows (``local_rows``) when a norm was asked for: the next reduction of the same shape needs exactly this rank's
    rows as its residual, so the full stream is only gathered if somebody asks for it with ``value()``.  Results
    that are views of the arena stay valid until the collective after next."""

    def __init__(self, comm: "FusedComm", parity: int, residual, rows: int, cols: int):
        self.comm, self.parity, self.residual, self.shape = comm, parity, residual, (rows, cols)
        self.out: torch.Tensor | None = None           # the full reduced residual stream
        self.local_rows: torch.Tensor | None = None    # [rows, cols] with only this rank's rows valid (sharded form)
        self.xn: torch.Tensor | None = None

    def _run(self, norm_w, eps: float, defer_wait: bool = False) -> None:
        comm = self.comm
        M, H = self.shape
        two = comm.two_shot(M, H)
        sharded = two and norm_w is not None
        defer_wait = defer_wait and sharded
        res = comm.residual_for(self.residual, M, H, two)
        xn = None
        if two:
            h_buf = torch.empty(M, H, dtype=torch.bfloat16, device=comm.device) if sharded else comm.region(1, self.parity, M, H)
            xn = comm.region(2, self.parity, M, H) if norm_w is not None else None
        else:
            h_buf = torch.empty(M, H, dtype=torch.bfloat16, device=comm.device)
            xn = torch.empty_like(h_buf) if norm_w is not None else None
        K._chk(comm.lib.exo_reduce_norm_bf16(K._ptr(res), K._ptr(norm_w), float(eps), h_buf.data_ptr(), K._ptr(xn), M, H,
                                             self.parity, int(two), int(not sharded) | (2 if defer_wait else 0), K._st()),
               "reduce_norm")
        K._count()
        comm.n_collectives += 1
        self.xn = xn
        if sharded:
            self.local_rows = h_buf
        else:
            self.out = h_buf

    @property
    def pending(self) -> bool:
        return self.out is None and self.local_rows is None

    def norm(self, norm_w, eps) -> torch.Tensor:
        if self.pending:
            self._run(norm_w, eps)
            return self.xn
        return K.rmsnorm(self.value(), norm_w, eps)[0]

    def norm_linear(self, norm_w, eps, w, bias=None, swiglu=False):
        if self.pending:
            M, H = self.shape
            comm = self.comm
            if (comm.use_gated_gemm and comm.two_shot(M, H) and isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16
                    and K.gated_gemm_ok(M, w.shape[0], H, swiglu) and (bias is None or not swiglu)):
                # all-gather -> GEMM: the reduction kernel does not wait for the other ranks' normalised rows; the
                # projection's CTAs wait for the owner of their rows, starting with this rank's own
                self._run(norm_w, eps, defer_wait=True)
                return K.gemm_bf16(self.xn, w, bias, None, swiglu, gate_parity=self.parity)
            return K.linear(self.norm(norm_w, eps), w, bias, None, None, 0.0, swiglu)
        return K.linear(self.value(), w, bias, None, norm_w, eps, swiglu)

    def value(self) -> torch.Tensor:
        if self.pending:
            self._run(None, 0.0)
        if self.out is None:
            # the stream was left sharded by rows: gather every rank's rows (one more collective, off the layer loop)
            M, H = self.shape
            comm = self.comm
            K._chk(comm.lib.exo_gather_rows_bf16(self.local_rows.data_ptr(), M, H, self.parity, K._st()), "gather_rows")
            K._count()
            comm.n_collectives += 1
            self.out = comm.region(1, self.parity, M, H)
        return self.out


def resolve(h):
    """A tensor for ``h``: pending reductions are finished, tensors pass through."""
    return h.value() if isinstance(h, (Handover, Reduction)) else h


def _exchange_fds(rank: int, n: int, mine: list[int], group) -> dict[int, list[int]]:
    """Every rank sends ``mine`` (file descriptors) to every other rank over Unix sockets (SCM_RIGHTS)."""
    name = f"\0exo-symm-{os.getpid()}-{uuid.uuid4().hex[:12]}"      # abstract namespace: nothing to unlink
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(n)
    names: list[str | None] = [None] * n
    dist.all_gather_object(names, name, group=group)
    outs = []
    for r in range(n):
        if r == rank:
            continue
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.connect(names[r])
        socket.send_fds(s, [rank.to_bytes(4, "little")], mine)
        outs.append(s)
    got: dict[int, list[int]] = {}
    srv.settimeout(120)
    for _ in range(n - 1):
        c, _addr = srv.accept()
        c.settimeout(120)
        msg, fds, _flags, _a = socket.recv_fds(c, 4, 8)
        got[int.from_bytes(msg[:4], "little")] = list(fds)
        c.close()
    dist.barrier(group=group)
    for s in outs:
        s.close()
    srv.close()
    return got


class FusedComm:
    def __init__(self, device: torch.device, max_rows: int, hidden: int, vocab_shard: int, group=None,
                 max_gather_rows: int = 256):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.lib = lib = bind(K.load())
        n = self.size
        torch.cuda.set_device(device)
        from ..shared import constants
        lib.exo_set_collective_timeout_us(int(constants.EXO_COLLECTIVE_TIMEOUT_US))
        L = arena_layout(lib, n, max_rows, hidden, vocab_shard, max_gather_rows)
        self.layout = L
        self.slot_bytes = L["slot"]
        self.max_elems = max_rows * hidden
        self.max_rows, self.hidden = max_rows, hidden
        self.vocab_shard = vocab_shard
        self.max_gather_rows = max_gather_rows
        self.gather_off = L["gather_off"]
        self.mc_ptr = 0
        self.transport = "ipc"
        self.peers: list[int] = []
        # every rank must take the same transport: agree on the weakest capability
        cap = lib.exo_vmm_supported() if os.environ.get("EXO_COMM_TRANSPORT", "vmm") != "ipc" else 0
        if os.environ.get("EXO_COMM_MULTICAST", "1") == "0":
            cap = min(cap, 1)
        caps: list[int | None] = [None] * n
        dist.all_gather_object(caps, cap, group=group)
        cap = min(int(c) for c in caps)
        if cap >= 1:
            self._open_vmm(L["total"], cap >= 2)
        else:
            self._open_ipc(L["total"])
        arr = (C.c_void_p * n)(*self.peers)
        K._chk(lib.exo_comm_init(arr, self.mc_ptr or None, n, self.rank, L["slot"], L["gather_off"], L["x_off"], L["x_bytes"],
                                 L["h_off"], L["n_off"], L["ll_off"], L["ll_slot"]), "comm init")
        dist.barrier(group=group)
        raw = torch.as_tensor(_RawBuffer(self.local + self.gather_off, L["gather_bytes"]), device=device)
        self.gather_buf = raw.view(torch.bfloat16)
        self._views: dict[tuple[int, int], torch.Tensor] = {}
        for which in (0, 1, 2):
            for parity in (0, 1):
                p = lib.exo_comm_region(which, parity)
                self._views[(which, parity)] = torch.as_tensor(_RawBuffer(p, L["x_bytes"]), device=device).view(torch.bfloat16)
        self._ar = 0
        self._ll = 0             # flag-in-data hand-overs issued so far (parity = low bit)
        self._rn = 0             # reduce + norm collectives issued so far
        self.n_collectives = 0
        self.n_handovers = 0
        self.use_handover = os.environ.get("EXO_DISABLE_TP_HANDOVER") != "1"
        self.use_reduce_norm = os.environ.get("EXO_DISABLE_REDUCE_NORM") != "1"
        self.use_gated_gemm = os.environ.get("EXO_DISABLE_GATED_GEMM") != "1"      # A/B: two-shot with its own trailing wait

    # ---- arena set-up ----
    def _open_ipc(self, total: int) -> None:
        lib, n = self.lib, self.size
        self.arena_bytes = total
        self.local = lib.exo_symm_alloc(total)
        if not self.local:
            raise RuntimeError(f"cannot allocate {total >> 20} MiB symmetric arena")
        handle = C.create_string_buffer(64)
        K._chk(lib.exo_symm_handle(self.local, handle), "ipc handle")
        handles: list[bytes | None] = [None] * n
        dist.all_gather_object(handles, handle.raw, group=self.group)
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peers.append(self.local)
            else:
                p = lib.exo_symm_open(C.create_string_buffer(h, 64))
                if not p:
                    raise RuntimeError(f"rank {self.rank}: cannot map arena of rank {r} (no peer access?)")
                self.peers.append(p)

    def _open_vmm(self, total: int, multicast: bool) -> None:
        lib, n, rank = self.lib, self.size, self.rank
        gran = lib.exo_vmm_granularity(n, int(multicast)) or (2 << 20)
        total = (total + gran - 1) // gran * gran
        self.arena_bytes = total
        fd = C.c_int(-1)
        self.local = lib.exo_vmm_alloc(total, C.byref(fd))
        ok = bool(self.local)
        mc_handle, mc_fd = 0, C.c_int(-1)
        if ok and multicast and rank == 0:
            mc_handle = lib.exo_mc_create(total, n, C.byref(mc_fd))
        flags: list[tuple | None] = [None] * n
        dist.all_gather_object(flags, (ok, bool(mc_handle) if rank == 0 else None), group=self.group)
        if not all(f[0] for f in flags):
            raise RuntimeError(f"rank {rank}: cannot allocate a {total >> 20} MiB virtual-memory arena")
        multicast = multicast and bool(flags[0][1])
        mine = [fd.value] + ([mc_fd.value] if (rank == 0 and multicast) else [])
        got = _exchange_fds(rank, n, mine, self.group)
        for r in range(n):
            if r == rank:
                self.peers.append(self.local)
                continue
            p = lib.exo_vmm_import(got[r][0], total)
            if not p:
                raise RuntimeError(f"rank {rank}: cannot map the arena of rank {r}")
            self.peers.append(p)
        if multicast:
            if rank != 0:
                mc_handle = lib.exo_mc_import(got[0][1])
            added = bool(mc_handle) and lib.exo_mc_add_device(mc_handle) == 0
            oks: list[bool | None] = [None] * n
            dist.all_gather_object(oks, added, group=self.group)        # also: every device is added before anyone binds
            if all(oks):
                self.mc_ptr = lib.exo_mc_bind_and_map(mc_handle, self.local, total) or 0
            oks = [None] * n
            dist.all_gather_object(oks, bool(self.mc_ptr), group=self.group)
            if not all(oks):                                             # all or nobody: the kernels of all ranks must agree
                if self.mc_ptr:
                    lib.exo_vmm_unmap(self.mc_ptr)
                self.mc_ptr = 0
        for fds in got.values():
            for f in fds:
                os.close(f)
        for f in mine:
            os.close(f)
        self.transport = "vmm+multicast" if self.mc_ptr else "vmm"

    # ---- regions of the reduce + norm kernels ----
    def region(self, which: int, parity: int, rows: int, cols: int) -> torch.Tensor:
        """``[rows, cols]`` bf16 view of region ``which`` (0 partial, 1 residual stream, 2 normalised rows)."""
        return self._views[(which, parity)][:rows * cols].view(rows, cols)

    def two_shot(self, rows: int, cols: int) -> bool:
        return rows >= 2 * self.size and (self.size - 1) * rows * cols * 2 > ONE_SHOT_MAX_BYTES

    def fits(self, rows: int, cols: int) -> bool:
        return (self.use_reduce_norm and 0 < rows and rows * cols * 2 <= self.layout["x_bytes"] and cols % 8 == 0
                and cols <= 8192)

    def residual_for(self, residual, rows: int, cols: int, two_shot: bool):
        """The tensor a reduction of ``[rows, cols]`` adds: a residual stream that the previous two-shot reduction left
        sharded by rows is used as it is when this reduction is two-shot over the same shape (same row ownership)."""
        if isinstance(residual, Reduction) and not residual.pending and residual.out is None:
            if two_shot and residual.shape == (rows, cols):
                return residual.local_rows
        return resolve(residual)

    def partial_out(self, rows: int, cols: int) -> tuple[torch.Tensor, int]:
        """Buffer for the next reduction's partial (write the projection output here) and its parity."""
        parity = self._rn & 1
        self._rn += 1
        return self.region(0, parity, rows, cols), parity

    # ---- collectives ----
    def row_sum(self, x: torch.Tensor, residual=None):
        """``residual + sum over ranks of x`` as a pending :class:`Handover` / :class:`Reduction` (or a tensor when
        the shape takes neither): the consumer's norm is then fused into the same kernel.  ``x`` was computed by some
        other kernel (the combined expert outputs of a MoE layer); decode batches go out as flag-in-data words."""
        if x.dtype != torch.bfloat16 or x.numel() % 8:
            raise K.KernelError("fused all-reduce takes bf16 tensors whose size is a multiple of 8")
        if x.dim() == 2:
            M, N = x.shape
            if (self.use_handover and 0 < M <= LL_ROWS and N % 8 == 0 and N <= 8192
                    and ((M + 1) & ~1) * N * 4 <= self.layout["ll_slot"]):
                x = x.contiguous()
                parity = self._ll & 1
                self._ll += 1
                K._chk(self.lib.exo_tp_ll_push(x.data_ptr(), M, N, parity, K._st()), "ll push")
                K._count()
                self.n_handovers += 1
                return Handover(self, parity, resolve(residual), M, N)
            if self.fits(M, N):
                buf, parity = self.partial_out(M, N)
                buf.copy_(x)
                return Reduction(self, parity, residual, M, N)
        return self._all_reduce_slots(x, residual)

    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual + sum over ranks of x`` (bf16)."""
        return resolve(self.row_sum(x, residual))

    def _all_reduce_slots(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        """Shapes the hand-over and the reduce + norm kernels do not take: the push-style kernels over staging slots."""
        residual = resolve(residual)
        x = x.contiguous()
        if x.numel() > self.max_elems:
            # larger than one arena slot (a long prefill chunk): reduce it in row blocks that fit
            if x.dim() != 2 or x.shape[1] > self.max_elems:
                raise K.KernelError(f"tensor of {x.numel()} elements exceeds the arena slot ({self.max_elems})")
            rows = max(8, (self.max_elems // x.shape[1]) // 8 * 8)
            parts = [self._all_reduce_slots(x[r:r + rows], None if residual is None else residual[r:r + rows])
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
        """``residual + all-reduce(x @ w.T)``, returned as a pending :class:`Handover` / :class:`Reduction`
        where the shapes allow it: the next ``norm_linear`` (or ``resolve``) then forms the sum."""
        M, Kd = x.shape
        N = w.shape[0]
        fp8 = isinstance(w, K.Fp8Weight)
        fits = (self.use_handover and x.dtype == torch.bfloat16 and 0 < M <= LL_ROWS and N % 8 == 0
                and ((M + 1) & ~1) * N * 4 <= self.layout["ll_slot"] and (fp8 or isinstance(w, torch.Tensor)))
        if fits and fp8 and Kd % 8 == 0 and Kd >= 64:
            # block-scaled fp8 weights: the fp8-weight GEMM's epilogue sends the words (every decode batch size)
            K.ensure_gemm_init(x.device)
            parity = self._ll & 1
            self._ll += 1
            x = x.contiguous()
            splits = self.lib.exo_gemm_splits(M, N, Kd)
            while splits > 1 and splits * M * N > K.GEMM_PARTIAL_FLOATS:
                splits -= 1
            kind = 1 if w.kind == "mxfp8" else 2
            f16 = K.fp8_f16_operands and N * Kd >= K.FP8_F16_MIN_WEIGHTS
            if f16:
                x16 = torch.empty(M, Kd, dtype=torch.float16, device=x.device)
                K._chk(self.lib.exo_bf16_to_f16(K._ptr(x), K._ptr(x16), M * Kd, K._st()), "bf16_to_f16")
                K._count()
                x = x16
            K._chk(self.lib.exo_gemm_fp8w_tp(x.data_ptr(), K._ptr(w.to_tiled().tiles), kind, None, M, N, Kd, splits, parity,
                                             int(f16), K._st()), "gemm_fp8w_tp push")
            K._count()
            self.n_handovers += 1
            return Handover(self, parity, resolve(residual), M, N)
        fits = fits and not fp8
        if fits and M <= 2 and K.use_stream_gemv and self.lib.exo_gemv_stream_supported(M, N, Kd, 1):
            # (1: rows leave in pairs, like the gate/up form)
            K.ensure_stream_init(x.device)
            parity = self._ll & 1
            self._ll += 1
            x = x.contiguous()
            K._chk(self.lib.exo_gemv_stream_tp(x.data_ptr(), w.data_ptr(), None, None, None, 0.0, M, N, Kd, 0, 1, parity,
                                               None, None, K._st()), "gemv_stream_tp push")
            K._count()
            self.n_handovers += 1
            return Handover(self, parity, resolve(residual), M, N)
        if fits and K.gemm_impl is not None and Kd >= 64 and Kd % 8 == 0:
            # decode batch: the tcgen05 GEMM's epilogue sends the words
            K.ensure_gemm_init(x.device)
            parity = self._ll & 1
            self._ll += 1
            x = x.contiguous()
            splits = self.lib.exo_gemm_splits(M, N, Kd)
            while splits > 1 and splits * M * N > K.GEMM_PARTIAL_FLOATS:
                splits -= 1
            K._chk(self.lib.exo_gemm_bf16_tp(x.data_ptr(), w.data_ptr(), None, M, N, Kd, splits, parity, K._st()), "gemm_tp push")
            K._count()
            self.n_handovers += 1
            return Handover(self, parity, resolve(residual), M, N)
        if x.dtype == torch.bfloat16 and self.fits(M, N):
            buf, parity = self.partial_out(M, N)
            K.linear(x, w, out=buf)                      # the projection writes straight into this rank's arena
            return Reduction(self, parity, residual, M, N)
        residual = resolve(residual)
        if x.dtype == torch.bfloat16 and M > 0 and N % 8 == 0 and N <= 8192 and self.use_reduce_norm:
            # longer than the arena region: row blocks that fit, each reduced by its own collective
            rows = max(8, (self.layout["x_bytes"] // (N * 2)) // 8 * 8)
            parts = [resolve(self.row_linear(x[r:r + rows], w, None if residual is None else residual[r:r + rows])).clone()
                     for r in range(0, M, rows)]
            return torch.cat(parts, dim=0)
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

    def all_reduce_stat(self, x: torch.Tensor) -> torch.Tensor:
        """A few fp32 numbers per token (normalisation statistics): the process group's all-reduce, which is
        stream-ordered and capturable; the arenas carry bf16 rows."""
        x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        return x

    def close(self) -> None:
        """Ordered teardown: every rank is idle before any mapping goes away (the multicast binding first)."""
        if not self.peers:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._views.clear()
        self.lib.exo_comm_reset()
        if self.transport == "ipc":
            for r, p in enumerate(self.peers):
                if r != self.rank and p:
                    self.lib.exo_symm_close(p)
            dist.barrier(group=self.group)
            self.lib.exo_symm_free(self.local)
        else:
            if self.mc_ptr:
                self.lib.exo_vmm_unmap(self.mc_ptr)
                self.mc_ptr = 0
            dist.barrier(group=self.group)
            for r, p in enumerate(self.peers):
                if r != self.rank and p:
                    self.lib.exo_vmm_unmap(p)
            dist.barrier(group=self.group)
            self.lib.exo_vmm_unmap(self.local)
        self.peers = []
