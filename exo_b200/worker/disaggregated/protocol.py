"""Wire protocol of prefill/decode disaggregation: a prefill instance streams the KV cache of a
prompt to the decode instance over TCP.

Frames and messages are the reference's (``src/exo/worker/disaggregated/protocol.py:1-152``,
``server.py:19-40``): every frame is a 4-byte big-endian length followed by a msgpack map; the
client sends one ``PrefillRequest{request_id, model_id, token_ids, start_pos}``; the server
answers with a ``Header{request_id, model_id, num_layers, dtype, start_pos}`` and then messages
tagged by ``type``: ``kv_chunk`` (one layer, a run of tokens, keys/values as raw
``[num_tokens, n_heads, head_dim]`` bytes), ``arrays_state`` (per-layer state tensors of
non-attention layers), ``done{total_tokens}`` or ``error{code, message}``.  Encoded with the
``msgpack`` package; maps keyed by field name decode on either implementation.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, BinaryIO, Literal

import msgpack

DType = Literal["bfloat16", "float16", "float32"]
MAX_FRAME = 1 << 31


class ProtocolError(Exception):
    pass


@dataclass
class PrefillRequest:
    request_id: str = ""
    model_id: str = ""
    token_ids: list[int] = field(default_factory=list)
    start_pos: int = 0


@dataclass
class Header:
    request_id: str = ""
    model_id: str = ""
    num_layers: int = 0
    dtype: DType = "bfloat16"
    start_pos: int = 0


@dataclass
class KVChunk:
    layer_idx: int
    num_tokens: int
    n_heads: int
    head_dim: int
    dtype: DType
    keys: bytes
    values: bytes
    type: str = "kv_chunk"

    @property
    def shape(self) -> tuple[int, int, int]:
        return (self.num_tokens, self.n_heads, self.head_dim)


@dataclass
class TensorBlob:
    dtype: DType
    shape: tuple[int, ...]
    data: bytes


@dataclass
class ArraysState:
    layer_idx: int
    arrays: list[TensorBlob] = field(default_factory=list)
    type: str = "arrays_state"


@dataclass
class Done:
    total_tokens: int
    type: str = "done"


@dataclass
class ErrorMessage:
    code: int
    message: str
    type: str = "error"


Message = KVChunk | ArraysState | Done | ErrorMessage
_BY_TAG = {"kv_chunk": KVChunk, "arrays_state": ArraysState, "done": Done, "error": ErrorMessage}


def _read_exactly(stream: BinaryIO, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = stream.read(n - len(buf))
        if not chunk:
            if not buf:
                return b""
            raise ConnectionError(f"Connection closed after {len(buf)}/{n} bytes")
        buf.extend(chunk)
    return bytes(buf)


def write_frame(stream: BinaryIO, payload: bytes) -> None:
    stream.write(len(payload).to_bytes(4, "big"))
    stream.write(payload)
    stream.flush()


def read_frame(stream: BinaryIO) -> bytes:
    raw = _read_exactly(stream, 4)
    if not raw:
        return b""
    n = int.from_bytes(raw, "big")
    if n > MAX_FRAME:
        raise ProtocolError(f"frame of {n} bytes exceeds the limit")
    return _read_exactly(stream, n)


def _pack(obj: Any) -> bytes:
    return msgpack.packb(asdict(obj), use_bin_type=True)


def _unpack(payload: bytes, what: str) -> dict[str, Any]:
    try:
        d = msgpack.unpackb(payload, raw=False)
    except Exception as e:  # noqa: BLE001 - msgpack raises several unrelated types
        raise ProtocolError(f"Bad {what}: {e}") from e
    if not isinstance(d, dict):
        raise ProtocolError(f"Bad {what}: expected a map")
    return d


def write_request(stream: BinaryIO, req: PrefillRequest) -> None:
    write_frame(stream, _pack(req))


def read_request(stream: BinaryIO) -> PrefillRequest:
    payload = read_frame(stream)
    if not payload:
        raise ConnectionError("No request received")
    d = _unpack(payload, "request")
    try:
        return PrefillRequest(request_id=str(d.get("request_id", "")), model_id=str(d.get("model_id", "")),
                              token_ids=[int(t) for t in d.get("token_ids", [])], start_pos=int(d.get("start_pos", 0)))
    except (TypeError, ValueError) as e:
        raise ProtocolError(f"Bad request: {e}") from e


def write_header(stream: BinaryIO, header: Header) -> None:
    write_frame(stream, _pack(header))


def read_header(stream: BinaryIO) -> Header:
    payload = read_frame(stream)
    if not payload:
        raise ConnectionError("No header received")
    d = _unpack(payload, "header")
    known = {k: d[k] for k in ("request_id", "model_id", "num_layers", "dtype", "start_pos") if k in d}
    return Header(**known)


def write_message(stream: BinaryIO, msg: Message) -> None:
    write_frame(stream, _pack(msg))


def read_message(stream: BinaryIO) -> Message | None:
    payload = read_frame(stream)
    if not payload:
        return None
    d = _unpack(payload, "message")
    cls = _BY_TAG.get(d.get("type", ""))
    if cls is None:
        raise ProtocolError(f"Bad message: unknown type {d.get('type')!r}")
    try:
        if cls is ArraysState:
            return ArraysState(layer_idx=int(d["layer_idx"]),
                               arrays=[TensorBlob(a["dtype"], tuple(a["shape"]), a["data"]) for a in d.get("arrays", [])])
        return cls(**{k: v for k, v in d.items() if k != "type"})
    except (KeyError, TypeError) as e:
        raise ProtocolError(f"Bad message: {e}") from e
