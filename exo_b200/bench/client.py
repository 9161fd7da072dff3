"""Thin HTTP client for a running cluster: what the benchmark and evaluation tools share.

Counterpart of the reference's ``tools/src/exo_tools/{client,cluster}.py``: find or place an
instance of a model, wait until its runners are ready, tear it down again.
"""
from __future__ import annotations

import json
import time
import urllib.error
import urllib.parse
import urllib.request
from typing import Any


class ApiError(RuntimeError):
    def __init__(self, status: int, body: str):
        super().__init__(f"HTTP {status}: {body[:300]}")
        self.status, self.body = status, body


class ExoClient:
    def __init__(self, host: str = "127.0.0.1", port: int = 52415, timeout: float = 600.0):
        self.base, self.timeout = f"http://{host}:{port}", timeout

    def request(self, method: str, path: str, body: Any = None, params: dict[str, Any] | None = None, timeout: float | None = None) -> Any:
        url = self.base + path + ("?" + urllib.parse.urlencode(params, doseq=True) if params else "")
        data = None if body is None else json.dumps(body).encode()
        req = urllib.request.Request(url, data=data, method=method, headers={"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=timeout or self.timeout) as r:
                raw = r.read()
        except urllib.error.HTTPError as e:
            raise ApiError(e.code, e.read().decode(errors="replace")) from e
        return json.loads(raw) if raw else None

    def get(self, path: str, **params: Any) -> Any:
        return self.request("GET", path, params=params or None)

    def post(self, path: str, body: Any, timeout: float | None = None) -> Any:
        return self.request("POST", path, body, timeout=timeout)

    def delete(self, path: str) -> Any:
        return self.request("DELETE", path)

    # ---- cluster helpers ----
    def state(self) -> dict[str, Any]:
        return self.get("/state")

    def instances_of(self, model_id: str) -> list[tuple[str, dict[str, Any]]]:
        out = []
        for iid, tagged in self.state()["instances"].items():
            inst = next(iter(tagged.values()))
            if inst["shardAssignments"]["modelId"] == model_id:
                out.append((iid, inst))
        return out

    def previews(self, model_id: str) -> list[dict[str, Any]]:
        return self.get("/instance/previews", model_id=model_id)["previews"]

    def place(self, model_id: str, sharding: str = "Tensor", min_nodes: int = 1) -> None:
        self.post("/place_instance", {"model_id": model_id, "sharding": sharding, "min_nodes": min_nodes})

    def wait_ready(self, model_id: str, n_runners: int | None = None, timeout: float = 1800.0) -> str:
        """Block until an instance of the model exists and all of its runners report ``RunnerReady``."""
        deadline = time.time() + timeout
        while time.time() < deadline:
            st = self.state()
            for iid, tagged in st["instances"].items():
                inst = next(iter(tagged.values()))
                if inst["shardAssignments"]["modelId"] != model_id:
                    continue
                rids = list(inst["shardAssignments"]["runnerToShard"])
                statuses = [next(iter(st["runners"].get(r, {"Missing": {}}))) for r in rids]
                if any(s == "RunnerFailed" for s in statuses):
                    raise RuntimeError(f"instance {iid} failed: {[st['runners'].get(r) for r in rids]}")
                if all(s in ("RunnerReady", "RunnerRunning") for s in statuses) and (n_runners is None or len(rids) == n_runners):
                    return iid
            time.sleep(0.5)
        raise TimeoutError(f"no ready instance of {model_id} after {timeout:.0f}s")

    def delete_instance(self, instance_id: str, wait: float = 60.0) -> None:
        self.delete(f"/instance/{instance_id}")
        deadline = time.time() + wait
        while time.time() < deadline and instance_id in self.state()["instances"]:
            time.sleep(0.25)
