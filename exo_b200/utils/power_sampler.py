"""Power accounting for one request: samples every node's reported power while it runs.

Same contract as the reference's sampler (``src/exo/utils/power_sampler.py``): poll the cluster
state's per-node system profile at a fixed interval, split the samples at the moment prefill ends,
and report per-node and total average power and energy for the whole request and for the prefill
and generation phases.  On this engine the power figure of a node is its GPU's NVML board power.
"""
from __future__ import annotations

import time
from collections.abc import Callable, Mapping

import anyio

from ..api.types import NodePowerStats, PowerUsage
from ..shared.base import NodeId
from ..shared.wire import SystemPerformanceProfile


class PowerSampler:
    def __init__(self, get_node_system: Callable[[], Mapping[NodeId, SystemPerformanceProfile]], interval: float = 1.0):
        self.get, self.interval = get_node_system, interval
        self.samples: dict[NodeId, list[tuple[float, float]]] = {}
        self.t0 = time.perf_counter()
        self.t_prefill_done: float | None = None
        self.t_end: float | None = None

    def sample(self) -> None:
        now = time.perf_counter()
        for node, prof in self.get().items():
            self.samples.setdefault(node, []).append((now, prof.sys_power))

    def mark_prefill_done(self) -> None:
        if self.t_prefill_done is None:
            self.t_prefill_done = time.perf_counter()
            self.sample()

    async def run(self) -> None:
        self.sample()
        try:
            while True:
                await anyio.sleep(self.interval)
                self.sample()
        finally:
            self.sample()
            self.t_end = time.perf_counter()

    @staticmethod
    def _avg(xs: list[float]) -> float | None:
        return sum(xs) / len(xs) if xs else None

    def result(self) -> PowerUsage:
        end = self.t_end or time.perf_counter()
        elapsed = end - self.t0
        split = self.t_prefill_done
        pre_s = None if split is None else split - self.t0
        gen_s = None if split is None else end - split
        nodes: list[NodePowerStats] = []
        for node, ss in self.samples.items():
            allp = [p for _t, p in ss]
            pre = [p for t, p in ss if split is not None and t <= split]
            gen = [p for t, p in ss if split is not None and t >= split]
            pa, ga = self._avg(pre), self._avg(gen)
            nodes.append(NodePowerStats(
                node_id=node, samples=len(ss), avg_sys_power=self._avg(allp) or 0.0, prefill_avg_sys_power=pa,
                generation_avg_sys_power=ga, prefill_energy_joules=None if pa is None or pre_s is None else pa * pre_s,
                generation_energy_joules=None if ga is None or gen_s is None else ga * gen_s))
        total_w = sum(n.avg_sys_power for n in nodes)

        def tot(attr: str) -> float | None:
            vals = [getattr(n, attr) for n in nodes]
            return None if not vals or any(v is None for v in vals) else float(sum(vals))
        return PowerUsage(elapsed_seconds=elapsed, nodes=nodes, total_avg_sys_power_watts=total_w,
                          total_energy_joules=total_w * elapsed, prefill_seconds=pre_s, generation_seconds=gen_s,
                          prefill_energy_joules=tot("prefill_energy_joules"), generation_energy_joules=tot("generation_energy_joules"),
                          prefill_avg_sys_power_watts=tot("prefill_avg_sys_power"), generation_avg_sys_power_watts=tot("generation_avg_sys_power"))
