"""Cluster harness shared by the benchmark and evaluation tools: from "a model name and a shape" to "a ready instance".

Counterpart of the reference's ``tools/src/exo_tools/harness.py``.  One class, ``Harness``, over the HTTP client:

* ``resolve_model``   short or partial names → the hub id the cluster knows (``/models``), ambiguous names are an error;
* ``placements``      ``/instance/previews`` filtered by sharding, communication back-end and node count, polled with
                      back-off until the cluster has settled (nodes still joining give fewer previews at first);
* ``ensure_downloaded`` disk check on every node of the chosen placement (``/state`` ``nodeDisk``), optionally freeing
                      space by deleting that node's completed, writable downloads smallest first, then ``/download/start``
                      per node and a progress poll until every node has the shard or one reports a failure; returns
                      the download wall time when anything was fetched;
* ``launch`` / ``teardown`` / ``find_existing`` / ``snapshot`` (what the cluster looked like when a number was taken).

``add_instance_args`` gives every tool the same flags.
"""
from __future__ import annotations

import argparse
import time
from dataclasses import dataclass, field
from typing import Any, Callable

from .client import ApiError, ExoClient


def untag(v: dict[str, Any]) -> dict[str, Any]:
    """``{"Variant": {...}}`` → the inner record; bare records pass through."""
    if len(v) == 1:
        (inner,) = v.values()
        if isinstance(inner, dict):
            return inner
    return v


def tag_of(v: dict[str, Any]) -> str:
    return next(iter(v)) if len(v) == 1 else ""


def instance_nodes(instance: dict[str, Any]) -> list[str]:
    return list(untag(instance)["shardAssignments"]["nodeToRunner"])


def instance_runners(instance: dict[str, Any]) -> list[str]:
    return list(untag(instance)["shardAssignments"]["runnerToShard"])


def add_instance_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True, help="hub id, or any unambiguous part of one the cluster knows")
    ap.add_argument("--sharding", default="Tensor", choices=["Tensor", "Pipeline", "both"])
    ap.add_argument("--instance-meta", default="any", help="communication back-end of the placement (e.g. Nvlink, Ring), or any")
    ap.add_argument("--min-nodes", type=int, default=1)
    ap.add_argument("--max-nodes", type=int, default=0, help="0: no limit")
    ap.add_argument("--settle-timeout", type=float, default=60.0, help="seconds to wait for a placement to appear")
    ap.add_argument("--ready-timeout", type=float, default=1800.0)
    ap.add_argument("--danger-delete-downloads", action="store_true", help="free disk space by deleting other completed downloads")
    ap.add_argument("--keep-instance", action="store_true")
    ap.add_argument("--reuse-instance", action="store_true", help="use a running instance of the model if there is one")


@dataclass
class Harness:
    client: ExoClient
    log: Callable[[str], None] = print
    sleep: Callable[[float], None] = time.sleep
    created: list[str] = field(default_factory=list)

    # ---- models ----
    def resolve_model(self, name: str) -> str:
        data = (self.client.get("/models") or {}).get("data", [])
        ids = [m.get("hugging_face_id") or m.get("id") for m in data]
        ids = [i for i in ids if i]
        if name in ids:
            return name
        low = name.lower()
        hits = [i for i in ids if i.lower().endswith("/" + low)] or [i for i in ids if low in i.lower()]
        if len(hits) == 1:
            return hits[0]
        if not hits:
            return name                                   # not known yet: the API can add it from the hub
        raise ValueError(f"{name!r} matches several models: {', '.join(sorted(hits)[:6])}")

    def model_bytes(self, model_id: str) -> int:
        for m in (self.client.get("/models") or {}).get("data", []):
            if (m.get("hugging_face_id") or m.get("id")) == model_id:
                return int(m.get("storage_size_megabytes", 0)) << 20
        return 0

    # ---- placements ----
    def placements(self, model_id: str, sharding: str = "Tensor", instance_meta: str = "any", min_nodes: int = 1,
                   max_nodes: int = 0, settle_timeout: float = 60.0) -> list[dict[str, Any]]:
        """Valid previews of the wanted shape, fewest nodes first.  Polls with back-off until one exists."""
        deadline, nap = time.monotonic() + settle_timeout, 1.0
        while True:
            out = []
            for p in self.client.previews(model_id):
                if p.get("error") or not p.get("instance"):
                    continue
                n = len(instance_nodes(p["instance"]))
                if n < min_nodes or (max_nodes and n > max_nodes):
                    continue
                if sharding != "both" and str(p.get("sharding", "")).lower() != sharding.lower():
                    continue
                meta = str(p.get("instance_meta") or p.get("instanceMeta") or tag_of(p["instance"]))
                if instance_meta != "any" and instance_meta.lower() not in meta.lower():
                    continue
                out.append(p)
            if out or time.monotonic() >= deadline:
                return sorted(out, key=lambda p: len(instance_nodes(p["instance"])))
            self.log(f"no placement of {model_id} yet ({max(0.0, deadline - time.monotonic()):.0f}s left)")
            self.sleep(min(nap, max(0.0, deadline - time.monotonic())))
            nap = min(nap * 2, 8.0)

    # ---- downloads ----
    def _downloads(self, node_id: str) -> list[dict[str, Any]]:
        return list((self.client.state().get("downloads") or {}).get(node_id, []))

    @staticmethod
    def _of_model(entry: dict[str, Any], kind: str, model_id: str) -> dict[str, Any] | None:
        body = entry.get(kind)
        if body is None:
            return None
        card = untag(body.get("shardMetadata", {})).get("modelCard", {})
        return body if card.get("modelId") == model_id else None

    def ensure_downloaded(self, model_id: str, preview: dict[str, Any], danger_delete: bool = False,
                          poll_s: float = 5.0, timeout: float = 6 * 3600.0) -> float | None:
        inner = untag(preview["instance"])
        node_to_runner = inner["shardAssignments"]["nodeToRunner"]
        shards = inner["shardAssignments"]["runnerToShard"]
        need = self.model_bytes(model_id)
        missing = [n for n in node_to_runner
                   if not any(self._of_model(e, "DownloadCompleted", model_id) for e in self._downloads(n))]
        if not missing:
            return None
        disks = self.client.state().get("nodeDisk") or {}
        for node in missing:
            avail = int(((disks.get(node) or {}).get("available") or {}).get("inBytes", 0))
            if not need or not avail or avail >= need:
                continue
            if not danger_delete:
                raise RuntimeError(f"node {node}: {need >> 30} GiB needed, {avail >> 30} GiB free "
                                   f"(--danger-delete-downloads frees space)")
            done = [(untag(e["DownloadCompleted"]["shardMetadata"])["modelCard"]["modelId"], int(e["DownloadCompleted"]["total"]["inBytes"]))
                    for e in self._downloads(node) if "DownloadCompleted" in e and not e["DownloadCompleted"].get("readOnly")]
            for other, size in sorted(done, key=lambda t: t[1]):
                if other == model_id:
                    continue
                self.log(f"node {node}: deleting {other} ({size >> 20} MiB)")
                self.client.delete(f"/download/{node}/{other}")
                avail += size
                if avail >= need:
                    break
            if avail < need:
                raise RuntimeError(f"node {node}: could not free {need >> 30} GiB")
        t0 = time.perf_counter()
        for node in missing:
            self.client.post("/download/start", {"targetNodeId": node, "shardMetadata": shards[node_to_runner[node]]})
        deadline = time.monotonic() + timeout
        while missing:
            for node in list(missing):
                entries = self._downloads(node)
                failed = [b["errorMessage"] for e in entries if (b := self._of_model(e, "DownloadFailed", model_id))]
                if failed:
                    raise RuntimeError(f"download failed on {node}: {failed[0]}")
                if any(self._of_model(e, "DownloadCompleted", model_id) for e in entries):
                    missing.remove(node)
                    continue
                for e in entries:
                    b = self._of_model(e, "DownloadOngoing", model_id)
                    if b:
                        pr = b.get("downloadProgress", {})
                        got, tot = pr.get("downloaded", {}).get("inBytes", 0), pr.get("total", {}).get("inBytes", 0)
                        self.log(f"node {node}: {100 * got / tot if tot else 0:.1f}% at {pr.get('speed', 0) / 2**20:.1f} MiB/s, "
                                 f"{pr.get('completedFiles', 0)}/{pr.get('totalFiles', 0)} files")
            if missing:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"downloads still running on {missing}")
                self.sleep(poll_s)
        return time.perf_counter() - t0

    # ---- instances ----
    def find_existing(self, model_id: str) -> str | None:
        for iid, _inst in self.client.instances_of(model_id):
            return iid
        return None

    def launch(self, model_id: str, preview: dict[str, Any], ready_timeout: float = 1800.0) -> str:
        before = {iid for iid, _ in self.client.instances_of(model_id)}
        self.client.post("/instance", {"instance": preview["instance"]})
        deadline = time.monotonic() + ready_timeout
        while time.monotonic() < deadline:
            st = self.client.state()
            for iid, tagged in st["instances"].items():
                if iid in before or untag(tagged)["shardAssignments"]["modelId"] != model_id:
                    continue
                status = [tag_of(st["runners"].get(r, {"Missing": {}})) for r in instance_runners(tagged)]
                bad = [st["runners"][r] for r, s in zip(instance_runners(tagged), status) if s == "RunnerFailed"]
                if bad:
                    raise RuntimeError(f"instance {iid} failed: {untag(bad[0]).get('errorMessage') or bad[0]}")
                if status and all(s in ("RunnerReady", "RunnerRunning") for s in status):
                    self.created.append(iid)
                    return iid
            self.sleep(0.5)
        raise TimeoutError(f"{model_id}: no ready instance after {ready_timeout:.0f}s")

    def teardown(self) -> None:
        for iid in self.created:
            try:
                self.client.delete_instance(iid)
            except (ApiError, OSError):
                pass
        self.created.clear()

    def snapshot(self) -> dict[str, Any]:
        """What a result should be stored with: nodes, their memory, GPUs' links, running instances."""
        st = self.client.state()
        return {"nodes": sorted(st.get("nodeIdentities") or st.get("nodeMemory") or {}),
                "memory": st.get("nodeMemory"), "nvlink": st.get("nodeNvlink"),
                "instances": {iid: {"model": untag(t)["shardAssignments"]["modelId"], "kind": tag_of(t), "nodes": instance_nodes(t)}
                              for iid, t in (st.get("instances") or {}).items()}}

    # ---- the whole path ----
    def instance_for(self, a: argparse.Namespace) -> tuple[str, str, float | None]:
        """``(model id, instance id, download seconds or None)`` from the common flags."""
        model = self.resolve_model(a.model)
        if getattr(a, "reuse_instance", False):
            iid = self.find_existing(model)
            if iid:
                return model, iid, None
        cands = self.placements(model, a.sharding, a.instance_meta, a.min_nodes, a.max_nodes, a.settle_timeout)
        if not cands:
            raise RuntimeError(f"no placement of {model} with sharding={a.sharding}, nodes >= {a.min_nodes}")
        dl = self.ensure_downloaded(model, cands[0], a.danger_delete_downloads)
        return model, self.launch(model, cands[0], a.ready_timeout), dl
