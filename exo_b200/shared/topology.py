"""Cluster topology: a directed multigraph of nodes (one per GPU here) and links.

Same public surface as the reference's ``Topology`` (``src/exo/shared/topology.py:33-308``:
add/remove nodes and connections, cycles, RDMA-only cycles, leaf test, sub-graphs, snapshot
round-trip) without the rustworkx dependency — the graphs are tiny (≤ 8 GPUs per box), so simple
cycles are enumerated with a plain DFS.  ``SocketConnection`` / ``RDMAConnection`` keep their wire
shape; an ``NvlinkConnection`` edge carries the measured peer bandwidth the planner uses.
"""
from __future__ import annotations

import re
from collections.abc import Callable, Iterable, Iterator
from dataclasses import dataclass

from pydantic import BaseModel, ConfigDict, computed_field, field_validator

from .base import FrozenModel, NodeId


class Multiaddr(BaseModel):
    model_config = ConfigDict(frozen=True)
    address: str

    _RE = (r"^/ip4/(\d{1,3}(?:\.\d{1,3}){3})(/tcp/(\d{1,5}))?(/p2p/[A-Za-z0-9]+)?$",
           r"^/ip6/([0-9a-fA-F:]+)(/tcp/(\d{1,5}))?(/p2p/[A-Za-z0-9]+)?$",
           r"^/dns[46]?/([a-zA-Z0-9.-]+)(/tcp/(\d{1,5}))?(/p2p/[A-Za-z0-9]+)?$")

    @field_validator("address")
    @classmethod
    def _fmt(cls, v: str) -> str:
        if not any(re.match(p, v) for p in cls._RE):
            raise ValueError(f"Invalid multiaddr format: {v}")
        return v

    @computed_field
    @property
    def address_type(self) -> str:
        return self.address.split("/")[1]

    @computed_field
    @property
    def ip_address(self) -> str:
        return self.address.split("/")[2]

    @computed_field
    @property
    def port(self) -> int:
        m = re.search(r"/tcp/(\d{1,5})", self.address)
        if not m:
            raise ValueError(f"multiaddr without a tcp port: {self.address}")
        return int(m.group(1))

    def __str__(self) -> str:
        return self.address


class RDMAConnection(FrozenModel):
    source_rdma_iface: str
    sink_rdma_iface: str


class SocketConnection(FrozenModel):
    sink_multiaddr: Multiaddr

    def __hash__(self) -> int:
        return hash(self.sink_multiaddr.ip_address)


class NvlinkConnection(FrozenModel):
    """GPU↔GPU link through NVSwitch with its measured one-direction copy bandwidth."""
    source_gpu: int
    sink_gpu: int
    gbps: float = 0.0
    links: int = 0


Edge = RDMAConnection | SocketConnection | NvlinkConnection


class Connection(FrozenModel):
    source: NodeId
    sink: NodeId
    edge: Edge


@dataclass(frozen=True)
class Cycle:
    node_ids: list[NodeId]

    def __len__(self) -> int:
        return len(self.node_ids)

    def __iter__(self) -> Iterator[NodeId]:
        return iter(self.node_ids)


class TopologySnapshot(BaseModel):
    nodes: list[NodeId] = []
    connections: dict[NodeId, dict[NodeId, list[Edge]]] = {}


class Topology:
    def __init__(self) -> None:
        self._nodes: list[NodeId] = []
        self._out: dict[NodeId, dict[NodeId, list[Edge]]] = {}

    # ---- snapshot ----
    def to_snapshot(self) -> TopologySnapshot:
        return TopologySnapshot(nodes=list(self._nodes),
                                connections={s: {t: list(es) for t, es in d.items() if es} for s, d in self._out.items() if d})

    @classmethod
    def from_snapshot(cls, snap: TopologySnapshot) -> "Topology":
        t = cls()
        for n in snap.nodes:
            t.add_node(n)
        for s, d in snap.connections.items():
            for k, es in d.items():
                for e in es:
                    t.add_connection(Connection(source=s, sink=k, edge=e))
        return t

    def __eq__(self, o: object) -> bool:
        return isinstance(o, Topology) and self.to_snapshot() == o.to_snapshot()

    # ---- nodes ----
    def add_node(self, n: NodeId) -> None:
        if n not in self._out:
            self._nodes.append(n)
            self._out[n] = {}

    def contains_node(self, n: NodeId) -> bool:
        return n in self._out

    def list_nodes(self) -> Iterable[NodeId]:
        return list(self._nodes)

    def remove_node(self, n: NodeId) -> None:
        if n not in self._out:
            return
        self._nodes.remove(n)
        del self._out[n]
        for d in self._out.values():
            d.pop(n, None)

    def neighbours(self, n: NodeId) -> list[NodeId]:
        return [t for t, es in self._out.get(n, {}).items() if es]

    def node_is_leaf(self, n: NodeId) -> bool:
        return n in self._out and len(self.neighbours(n)) <= 1

    # ---- edges ----
    def add_connection(self, c: Connection) -> None:
        self.add_node(c.source)
        self.add_node(c.sink)
        es = self._out[c.source].setdefault(c.sink, [])
        if c.edge not in es:
            es.append(c.edge)

    def remove_connection(self, c: Connection) -> None:
        es = self._out.get(c.source, {}).get(c.sink)
        if es and c.edge in es:
            es.remove(c.edge)
            if not es:
                del self._out[c.source][c.sink]

    def out_edges(self, n: NodeId) -> Iterable[Connection]:
        return [Connection(source=n, sink=t, edge=e) for t, es in self._out.get(n, {}).items() for e in es]

    def get_all_connections_between(self, a: NodeId, b: NodeId) -> list[Edge]:
        return list(self._out.get(a, {}).get(b, []))

    def list_connections(self) -> list[Connection]:
        return [c for n in self._nodes for c in self.out_edges(n)]

    def map_connections(self) -> dict[NodeId, dict[NodeId, list[Edge]]]:
        return {s: {t: list(es) for t, es in d.items()} for s, d in self._out.items()}

    def replace_all_out_rdma_connections(self, n: NodeId, new: Iterable[Connection]) -> None:
        for es in self._out.get(n, {}).values():
            es[:] = [e for e in es if not isinstance(e, RDMAConnection)]
        self._out[n] = {t: es for t, es in self._out.get(n, {}).items() if es}
        for c in new:
            self.add_connection(c)

    def remove_all_rdma_connections_touching(self, n: NodeId) -> None:
        for s, d in self._out.items():
            for t in list(d):
                if s == n or t == n:
                    d[t] = [e for e in d[t] if not isinstance(e, RDMAConnection)]
                    if not d[t]:
                        del d[t]

    # ---- cycles ----
    def _simple_cycles(self, keep: Callable[[Edge], bool]) -> list[list[NodeId]]:
        adj = {s: [t for t, es in d.items() if any(keep(e) for e in es)] for s, d in self._out.items()}
        order = {n: i for i, n in enumerate(self._nodes)}
        found: list[list[NodeId]] = []

        def dfs(start: NodeId, cur: NodeId, path: list[NodeId], seen: set[NodeId]) -> None:
            for nxt in adj.get(cur, []):
                if nxt == start and len(path) >= 2:
                    found.append(list(path))
                elif nxt not in seen and order[nxt] > order[start]:
                    seen.add(nxt)
                    path.append(nxt)
                    dfs(start, nxt, path, seen)
                    path.pop()
                    seen.discard(nxt)

        for s in self._nodes:
            dfs(s, s, [s], {s})
        return found

    def get_cycles(self) -> list[Cycle]:
        """Every simple directed cycle of ≥ 2 nodes plus every single node."""
        return [Cycle(c) for c in self._simple_cycles(lambda e: True)] + [Cycle([n]) for n in self._nodes]

    def get_rdma_cycles(self) -> list[Cycle]:
        return [Cycle(c) for c in self._simple_cycles(lambda e: isinstance(e, (RDMAConnection, NvlinkConnection)))]

    def is_rdma_cycle(self, cycle: Cycle) -> bool:
        ids = list(cycle.node_ids)
        if len(ids) < 2:
            return False
        for a, b in zip(ids, ids[1:] + ids[:1]):
            if not any(isinstance(e, (RDMAConnection, NvlinkConnection)) for e in self.get_all_connections_between(a, b)):
                return False
        return True

    def get_subgraph_from_nodes(self, ids: list[NodeId]) -> "Topology":
        t = Topology()
        keep = set(ids)
        for n in self._nodes:
            if n in keep:
                t.add_node(n)
        for c in self.list_connections():
            if c.source in keep and c.sink in keep:
                t.add_connection(c)
        return t

    def min_nvlink_gbps(self, ids: list[NodeId]) -> float:
        """Slowest measured NVLink edge among a group of nodes (0 when some pair has none)."""
        worst = float("inf")
        for a in ids:
            for b in ids:
                if a == b:
                    continue
                bw = [e.gbps for e in self.get_all_connections_between(a, b) if isinstance(e, NvlinkConnection)]
                worst = min(worst, max(bw) if bw else 0.0)
        return 0.0 if worst == float("inf") else worst
