"""TCP endpoints of prefill/decode disaggregation: the prefill instance's server and the decode
instance's fetch.

The server (reference: ``src/exo/worker/disaggregated/server.py:42-105``) accepts one request per
connection on a thread per client, hands it to a ``resolve(job, stream) -> bool`` callback that
streams the answer, and reports protocol and resolver failures in-band as ``error`` messages
(400 bad request, 500 resolver exception, 503 nobody picked the job up).  The fetch side
(reference: ``engines/mlx/disaggregated/client.py``) collects the stream into per-layer lists of
chunks and raises on an ``error`` message or a stream that ends before ``done``.
"""
from __future__ import annotations

import socket
import socketserver
import threading
from collections.abc import Callable
from dataclasses import dataclass, field
from typing import BinaryIO, cast

from .protocol import (ArraysState, Done, ErrorMessage, Header, KVChunk, PrefillRequest, ProtocolError, read_header,
                       read_message, read_request, write_header, write_message, write_request)

ResolveHandler = Callable[[PrefillRequest, BinaryIO], bool]


def send_error(wfile: BinaryIO, code: int, message: str) -> None:
    try:
        write_header(wfile, Header(num_layers=0, dtype="float32"))
        write_message(wfile, ErrorMessage(code=code, message=message))
    except Exception:  # noqa: BLE001 - the peer may already be gone
        pass


class _Handler(socketserver.StreamRequestHandler):
    def setup(self) -> None:
        super().setup()
        sock = cast(socket.socket, self.request)
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        sock.setsockopt(socket.SOL_SOCKET, socket.SO_SNDBUF, 4 << 20)

    def handle(self) -> None:
        server = cast("PrefillServer", self.server)
        wfile = cast(BinaryIO, self.wfile)
        try:
            job = read_request(cast(BinaryIO, self.rfile))
        except ConnectionError:
            return
        except (ProtocolError, ValueError) as e:
            send_error(wfile, 400, f"Bad request: {e}")
            return
        try:
            picked_up = server.resolve(job, wfile)
        except Exception as e:  # noqa: BLE001 - reported to the client
            send_error(wfile, 500, str(e))
            return
        if not picked_up:
            send_error(wfile, 503, f"Prefill not picked up for request_id={job.request_id!r}")


class PrefillServer(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self, resolve: ResolveHandler, host: str = "0.0.0.0", port: int = 0):
        super().__init__((host, port), _Handler)
        self.resolve = resolve
        self.port = self.server_address[1]
        self._thread: threading.Thread | None = threading.Thread(target=self.serve_forever, name="prefill-server", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self.shutdown()
        self.server_close()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None


@dataclass
class PrefillResult:
    header: Header
    chunks: dict[int, list[KVChunk]] = field(default_factory=dict)       # layer -> chunks in token order
    states: dict[int, ArraysState] = field(default_factory=dict)
    total_tokens: int = 0


class RemotePrefillError(Exception):
    def __init__(self, code: int, message: str):
        super().__init__(f"remote prefill failed ({code}): {message}")
        self.code = code


def remote_prefill_fetch(endpoint: str, request: PrefillRequest, *, timeout: float = 300.0,
                         on_header: Callable[[Header], None] | None = None,
                         on_kv_chunk: Callable[[KVChunk, int], None] | None = None) -> PrefillResult:
    host, _, port = endpoint.rpartition(":")
    with socket.create_connection((host or "127.0.0.1", int(port)), timeout=timeout) as sock:
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        sock.setsockopt(socket.SOL_SOCKET, socket.SO_RCVBUF, 4 << 20)
        rfile, wfile = sock.makefile("rb"), sock.makefile("wb")
        write_request(cast(BinaryIO, wfile), request)
        header = read_header(cast(BinaryIO, rfile))
        if on_header is not None:
            on_header(header)
        res = PrefillResult(header)
        n = 0
        while True:
            msg = read_message(cast(BinaryIO, rfile))
            if msg is None:
                raise ConnectionError("prefill stream ended before 'done'")
            if isinstance(msg, ErrorMessage):
                raise RemotePrefillError(msg.code, msg.message)
            if isinstance(msg, Done):
                res.total_tokens = msg.total_tokens
                return res
            if isinstance(msg, KVChunk):
                res.chunks.setdefault(msg.layer_idx, []).append(msg)
                n += 1
                if on_kv_chunk is not None:
                    on_kv_chunk(msg, n)
            elif isinstance(msg, ArraysState):
                res.states[msg.layer_idx] = msg
