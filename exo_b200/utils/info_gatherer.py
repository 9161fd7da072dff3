"""Node telemetry: what this node (one GPU and its host) looks like, reported periodically.

Same role as the reference's ``InfoGatherer`` (``src/exo/utils/info_gatherer/info_gatherer.py:
388-644``: one task per kind of information, each with its own period, all writing
``GatheredInfo`` messages into one channel; ``system_info.py`` for interfaces and identity), with
the Mac probes (macmon, system_profiler, networksetup, rdma_ctl) replaced by what matters on a
B200 box: NVML for HBM, utilisation, power, temperature, and the NVLink peer table that the
placement planner turns into topology edges.  "Memory" of a GPU node is its HBM: a placement that
fits by this figure fits on the device.  The GPU probe is injected so the whole gatherer runs
against a fake NVML in tests.
"""
from __future__ import annotations

import os
import platform
import shutil
import socket
from collections.abc import Callable, Sequence
from dataclasses import dataclass, field

import anyio
import psutil

from ..shared import constants
from ..shared.base import Memory
from ..shared.cards import Backend
from ..shared.wire import (DiskUsage, GatheredInfo, MemoryUsage, MiscData, NetworkInterfaceInfo, NodeBackends,
                           NodeDiskUsage, NodeMemory, NodeNetworkInterfaces, NodeNvlink, NodeNvlinkInfo, NodePerformance,
                           NvlinkPeer, RdmaCtlStatus, StaticNodeInformation, SystemPerformanceProfile)
from .channels import ChannelClosed, Sender

NVLINK5_GBPS_PER_LINK = 50.0 * 8     # 50 GB/s per direction per link, in Gbit/s
NVSWITCH_DEFAULT_LINKS = 18


@dataclass
class GpuSample:
    """One reading of one GPU (the fields of the native ``nvml_enumerate`` rows)."""
    index: int
    name: str = "Unknown"
    uuid: str = ""
    mem_total: int = 0
    mem_free: int = 0
    power_mw: int = 0
    temp_c: int = 0
    util_pct: int = 0
    sm_mhz: int = 0
    nvlink_peers_links: Sequence[int] = field(default_factory=list)
    p2p_ok: Sequence[int] = field(default_factory=list)
    active_links: int = 0


GpuProbe = Callable[[], list[GpuSample]]


def nvml_probe() -> list[GpuSample]:
    """All GPUs NVML shows, through the native module; ``[]`` without a driver."""
    try:
        from ..native import _exo_native as nat
    except ImportError:
        return []
    rows, _err = nat.nvml_enumerate()
    return [GpuSample(index=r.index, name=r.name, uuid=r.uuid, mem_total=r.mem_total, mem_free=r.mem_free,
                      power_mw=r.power_mw, temp_c=r.temp_c, util_pct=r.util_pct, sm_mhz=r.sm_mhz,
                      nvlink_peers_links=list(r.nvlink_peers_links), p2p_ok=list(r.p2p_ok), active_links=r.active_links)
            for r in rows]


def node_gpu_index() -> int | None:
    v = os.environ.get("EXO_GPU_INDEX")
    return int(v) if v not in (None, "") else None


def classify_interface(name: str) -> str:
    n = name.lower()
    if n.startswith(("wl", "wifi")):
        return "wifi"
    if n.startswith(("en", "eth", "bond", "ib")):
        return "ethernet"
    if n.startswith(("veth", "docker", "br-", "tun", "tap")):
        return "maybe_ethernet"
    return "unknown"


def network_interfaces() -> list[NetworkInterfaceInfo]:
    out = []
    for name, addrs in psutil.net_if_addrs().items():
        for a in addrs:
            if a.family in (socket.AF_INET, socket.AF_INET6) and a.address:
                ip = a.address.split("%", 1)[0]
                if ip.startswith("fe80") or ip in ("127.0.0.1", "::1"):
                    continue
                out.append(NetworkInterfaceInfo(name=name, ip_address=ip, interface_type=classify_interface(name)))
    return out


def friendly_name(gpu: int | None) -> str:
    host = socket.gethostname() or "node"
    return host if gpu is None else f"{host}/gpu{gpu}"


def nvlink_info(me: GpuSample, n_gpus: int, measured: dict | None = None) -> NodeNvlinkInfo:
    """Peer table of one GPU.  Behind NVSwitch NVML reports no per-peer link count (links end at
    the switch), so a P2P-capable peer gets the GPU's whole active link budget.  ``measured`` is the link probe's
    result (``utils.link_probe``): where it has a figure for a peer, that figure replaces links x nominal."""
    peers = []
    got = (measured or {}).get("peers", {})
    for j in range(n_gpus):
        if j == me.index:
            continue
        ok = bool(me.p2p_ok[j]) if j < len(me.p2p_ok) else False
        direct = me.nvlink_peers_links[j] if j < len(me.nvlink_peers_links) else 0
        links = direct or (me.active_links or NVSWITCH_DEFAULT_LINKS if ok else 0)
        m = got.get(str(j)) or {}
        if ok and m.get("gbps"):
            peers.append(NvlinkPeer(peer_gpu=j, links=links, gbps=float(m["gbps"]), p2p=ok,
                                    latency_us=float(m.get("latency_us", 0.0)), measured=True))
        else:
            peers.append(NvlinkPeer(peer_gpu=j, links=links, gbps=links * NVLINK5_GBPS_PER_LINK, p2p=ok))
    return NodeNvlinkInfo(gpu_index=me.index, uuid=me.uuid, peers=peers, hbm_gbps=float((measured or {}).get("hbm_gbps", 0.0)))


def link_probe(gpu: int, peers: list[int], uuid: str) -> dict | None:
    """Measured copy bandwidths of this GPU (own HBM, each peer); tests replace this hook."""
    if os.environ.get("EXO_LINK_PROBE", "1") == "0" or not kernels_available():
        return None
    from .link_probe import measure
    return measure(gpu, peers, uuid)


def kernels_available() -> bool:
    from pathlib import Path
    return (Path(__file__).resolve().parent.parent / "ops" / "_kernels.so").exists()


class InfoGatherer:
    def __init__(self, sender: Sender[GatheredInfo], *, gpu_index: int | None = None, probe: GpuProbe | None = None,
                 memory_interval: float = 1.0, perf_interval: float = 1.0, disk_interval: float = 30.0,
                 network_interval: float = 10.0, misc_interval: float = 60.0, nvlink_interval: float = 30.0):
        self.sender, self.probe = sender, probe
        self.gpu_index = gpu_index if gpu_index is not None else node_gpu_index()
        self.iv = dict(memory=memory_interval, perf=perf_interval, disk=disk_interval, network=network_interval,
                       misc=misc_interval, nvlink=nvlink_interval)
        self._measured: dict | None = None
        self._probe_tried = False

    # ---- single readings (also used directly by tests and the power sampler) ----
    def _gpus(self) -> list[GpuSample]:
        try:
            return (self.probe or nvml_probe)()
        except Exception:  # a flaky driver call must not end telemetry
            return []

    def _mine(self, gpus: list[GpuSample]) -> GpuSample | None:
        if not gpus:
            return None
        idx = 0 if self.gpu_index is None else self.gpu_index
        return next((g for g in gpus if g.index == idx), None)

    def static_info(self) -> StaticNodeInformation:
        me = self._mine(self._gpus())
        return StaticNodeInformation(model=platform.node() or "Unknown", chip=me.name if me else (platform.processor() or platform.machine() or "Unknown"),
                                     os_version=f"{platform.system()} {platform.release()}", os_build_version=platform.version())

    def memory(self) -> NodeMemory:
        me = self._mine(self._gpus())
        sw = psutil.swap_memory()
        if me is not None and me.mem_total:
            return NodeMemory(memory=MemoryUsage.from_bytes(ram_total=me.mem_total, ram_available=me.mem_free,
                                                            swap_total=sw.total, swap_available=sw.free))
        vm = psutil.virtual_memory()
        override = os.environ.get("OVERRIDE_MEMORY_MB")
        avail = int(override) << 20 if override else vm.available
        return NodeMemory(memory=MemoryUsage.from_bytes(ram_total=vm.total, ram_available=avail, swap_total=sw.total,
                                                        swap_available=sw.free))

    def performance(self) -> NodePerformance:
        me = self._mine(self._gpus())
        cpu = psutil.cpu_percent(interval=None)
        if me is None:
            return NodePerformance(profile=SystemPerformanceProfile(pcpu_usage=cpu))
        return NodePerformance(profile=SystemPerformanceProfile(gpu_usage=me.util_pct / 100.0, temp=float(me.temp_c),
                                                                sys_power=me.power_mw / 1000.0, pcpu_usage=cpu))

    def disk(self) -> NodeDiskUsage:
        d = constants.EXO_DEFAULT_MODELS_DIR
        while not d.exists() and d != d.parent:
            d = d.parent
        u = shutil.disk_usage(d)
        return NodeDiskUsage(disk_usage=DiskUsage(total=Memory.from_bytes(u.total), available=Memory.from_bytes(u.free)))

    def backends(self) -> NodeBackends:
        me = self._mine(self._gpus())
        ok = me is not None and kernels_available()
        return NodeBackends(backends=[Backend.B200] if ok else [])

    def nvlink(self) -> NodeNvlink | None:
        gpus = self._gpus()
        me = self._mine(gpus)
        if me is None:
            return None
        if self._measured is None and not self._probe_tried and len(gpus) > 0:
            # once per node: the probe runs in a child process (tens of seconds the first time, cached afterwards)
            self._probe_tried = True
            peers = [j for j in range(len(gpus)) if j != me.index and j < len(me.p2p_ok) and me.p2p_ok[j]]
            try:
                self._measured = link_probe(me.index, peers, me.uuid)
            except Exception:  # noqa: BLE001 - telemetry must survive a failing probe
                self._measured = None
        return NodeNvlink(info=nvlink_info(me, len(gpus), self._measured))

    # ---- periodic tasks ----
    async def _every(self, seconds: float, read: Callable[[], GatheredInfo | None]) -> None:
        while True:
            info = await anyio.to_thread.run_sync(read)
            if info is not None:
                try:
                    await self.sender.send(info)
                except ChannelClosed:
                    return
            await anyio.sleep(seconds)

    async def run(self) -> None:
        try:
            await self.sender.send(self.static_info())
        except ChannelClosed:
            return
        async with anyio.create_task_group() as tg:
            tg.start_soon(self._every, self.iv["memory"], self.memory)
            tg.start_soon(self._every, self.iv["perf"], self.performance)
            tg.start_soon(self._every, self.iv["disk"], self.disk)
            tg.start_soon(self._every, self.iv["network"], lambda: NodeNetworkInterfaces(ifaces=network_interfaces()))
            tg.start_soon(self._every, self.iv["misc"], lambda: MiscData(friendly_name=friendly_name(self.gpu_index)))
            tg.start_soon(self._every, self.iv["misc"], self.backends)
            tg.start_soon(self._every, self.iv["misc"], lambda: RdmaCtlStatus(enabled=False))
            tg.start_soon(self._every, self.iv["nvlink"], self.nvlink)


async def check_reachable(candidates: dict[str, list[str]], api_port: int, timeout: float = 1.0):
    """Yield ``(ip, node_id)`` for every candidate address whose API answers ``/node_id`` with that id.

    The reference probes peers the same way (``src/exo/utils/info_gatherer/net_profile.py:14-127``):
    an HTTP GET per address, the answer must name the expected node.
    """
    import aiohttp

    async def one(session, node, ip, out):
        host = f"[{ip}]" if ":" in ip else ip
        try:
            async with session.get(f"http://{host}:{api_port}/node_id", timeout=aiohttp.ClientTimeout(total=timeout)) as r:
                if r.status == 200 and (await r.text()).strip().strip('"') == node:
                    out.append((ip, node))
        except Exception:
            pass

    found: list[tuple[str, str]] = []
    async with aiohttp.ClientSession() as session:
        async with anyio.create_task_group() as tg:
            for node, ips in candidates.items():
                for ip in ips:
                    tg.start_soon(one, session, node, ip, found)
    for item in found:
        yield item
