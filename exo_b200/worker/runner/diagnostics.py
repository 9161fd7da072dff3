"""Classification of a dying runner's stderr into known failure kinds.

The supervisor keeps the tail of the child's stderr; these patterns turn it into structured
``KnownRunnerDiagnostic`` items attached to ``RunnerFailed`` and to the ``ErrorChunk`` of each
in-flight request (reference ``src/exo/worker/runner/diagnostics.py:13-108``, whose taxonomy is
Metal time-outs and TCP-ring socket errors; the kinds here are the CUDA / NCCL / NVLink ones).
"""
from __future__ import annotations

import re
from collections import deque

from ...shared.wire import KnownRunnerDiagnostic

PATTERNS: tuple[tuple[str, str, re.Pattern[str]], ...] = (
    ("cuda_oom", "The GPU ran out of memory", re.compile(r"CUDA out of memory|cudaErrorMemoryAllocation|OutOfMemoryError", re.I)),
    ("cuda_fault", "A CUDA kernel faulted", re.compile(r"illegal memory access|an illegal instruction|misaligned address|Xid \d+|unspecified launch failure", re.I)),
    ("nccl_error", "An NCCL collective failed", re.compile(r"NCCL (WARN|error)|ncclUnhandledCudaError|ncclSystemError|ncclRemoteError", re.I)),
    ("collective_timeout", "A rank stopped answering inside a collective", re.compile(r"CollectiveTimeout|DeviceWaitTimeout|gave up waiting for a peer GPU|Watchdog caught collective operation timeout|device-side wait on a peer timed out", re.I)),
    ("kernel_timeout", "A kernel's internal pipeline wait ran out", re.compile(r"pipeline wait ran out|device-side timeout code", re.I)),
    ("peer_access", "GPU peer access is unavailable", re.compile(r"cannot map arena|peer access|cudaErrorPeerAccess", re.I)),
    ("kernel_missing", "The native kernel library is missing", re.compile(r"_kernels\.so is missing|KernelError: .* is missing", re.I)),
    ("checkpoint", "The model checkpoint is incomplete or unreadable", re.compile(r"no \*\.safetensors under|checkpoint shape .* != expected|safetensors", re.I)),
    ("host_oom", "The host ran out of memory", re.compile(r"MemoryError|Cannot allocate memory", re.I)),
)


class DiagnosticCollector:
    """Feed it stderr lines; ask for diagnostics when the process has died."""

    def __init__(self, context_lines: int = 4):
        self.context: deque[str] = deque(maxlen=context_lines)
        self.found: dict[str, KnownRunnerDiagnostic] = {}

    def feed(self, line: str) -> None:
        self.context.append(line)
        for kind, summary, rx in PATTERNS:
            if kind not in self.found and rx.search(line):
                self.found[kind] = KnownRunnerDiagnostic(kind=kind, summary=summary, evidence=list(self.context))

    def diagnostics(self) -> list[KnownRunnerDiagnostic]:
        return list(self.found.values())


def cause_from_exit(exitcode: int | None) -> str:
    if exitcode is None:
        return "runner is still running"
    if exitcode < 0:
        import signal
        try:
            return f"runner killed by {signal.Signals(-exitcode).name}"
        except ValueError:
            return f"runner killed by signal {-exitcode}"
    return "runner exited cleanly" if exitcode == 0 else f"runner exited with code {exitcode}"
