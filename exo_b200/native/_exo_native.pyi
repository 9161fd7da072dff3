"""Typed stub of the native runtime module (``exo_b200/native/csrc``: message bus, pidfile, NVML topology).

The reference ships a generated stub for its PyO3 module (``rust/exo_rs/exo_rs.pyi``); this one is written by hand
next to the pybind11 module it describes.
"""
from typing import Literal

def namespace_hash(namespace: str) -> int:
    """8-byte tag of a cluster namespace (carried in the bus handshake and in discovery packets)."""

def valid_identity(identity: str) -> bool:
    """True for a node identity the bus accepts: hex digits, at most 32, no leading zero."""

ConnectionEvent = tuple[Literal["connection"], str, bool]        # ("connection", peer identity, connected)
DiscoveredEvent = tuple[Literal["discovered"], str, str]         # ("discovered", peer identity, "host:port")
MessageEvent = tuple[Literal["message"], str, bytes]             # ("message", topic, payload)

class Bus:
    """Topic pub/sub over TCP between the nodes of one namespace, with peer liveliness and LAN discovery."""

    def __init__(self, identity: str, namespace: str, listen_port: int = 0, discovery_port: int = 0) -> None: ...
    @property
    def listen_port(self) -> int:
        """TCP port the bus accepts peers on (the bound port when 0 was asked for)."""
    @property
    def event_fd(self) -> int:
        """File descriptor that is readable whenever ``try_recv`` has something: watch it from the event loop."""
    def try_recv(self) -> ConnectionEvent | DiscoveredEvent | MessageEvent | None:
        """Next queued event without blocking, or ``None``."""
    def connect(self, host: str, port: int) -> bool:
        """Connect to a peer explicitly (the GIL is released while connecting)."""
    def subscribe(self, topic: str) -> None: ...
    def unsubscribe(self, topic: str) -> None: ...
    def publish(self, topic: str, data: bytes) -> int:
        """Blocks (GIL released) until the frame is handed to every subscribed peer; returns how many got it."""
    def peers(self) -> list[str]:
        """Identities of the peers whose handshake has completed."""
    def close(self) -> None: ...

class NativeError(RuntimeError): ...

class Pidfile:
    """Locked PID file: raises ``NativeError("AlreadyRunning:<pid>")`` when another process holds it."""

    def __init__(self, path: str) -> None: ...
    def write(self) -> None:
        """Write the current pid (call after daemonising)."""
    def as_raw_fd(self) -> int: ...
    def close(self) -> None:
        """Unlock and remove the file."""

class GpuInfo:
    index: int
    name: str
    uuid: str
    mem_total: int
    mem_free: int
    power_mw: int
    temp_c: int
    util_pct: int
    sm_mhz: int
    nvlink_peers_links: list[int]
    p2p_ok: list[int]
    active_links: int

def nvml_enumerate() -> tuple[list[GpuInfo], str]:
    """Every GPU NVML shows and an error string (empty list and a message when there is no driver)."""
