"""Pre-stage a model on every node of a running cluster through ``/download/start``.

Counterpart of the reference's ``scripts/download_model_to_cluster.py``: asks each node (or the
given ones) to download the whole model, then polls ``/state`` until every node reports it
completed (or one reports failure).

    python -m exo_b200.cli.download_model_to_cluster --model meta-llama/Llama-3.1-8B-Instruct
"""
from __future__ import annotations

import argparse
import sys
import time

from ..bench.client import ExoClient


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--nodes", default="", help="comma-separated node ids (default: every node in the topology)")
    ap.add_argument("--timeout", type=float, default=6 * 3600)
    a = ap.parse_args(argv)
    c = ExoClient(a.host, a.port)
    models = {m["id"]: m for m in c.get("/models")["data"]}
    if a.model not in models:
        added = c.post("/models/add", {"model_id": a.model})
        models[a.model] = added
    st = c.state()
    nodes = [n for n in a.nodes.split(",") if n] or list(st["topology"]["nodes"])
    previews = [p for p in c.previews(a.model) if p.get("instance")]
    if not previews:
        print("no placement preview available to take the model card from", file=sys.stderr)
        return 1
    inst = next(iter(previews[0]["instance"].values()))
    shard = next(iter(inst["shardAssignments"]["runnerToShard"].values()))
    kind, body = next(iter(shard.items()))
    full = {"PipelineShardMetadata": {**body, "deviceRank": 0, "worldSize": 1, "startLayer": 0, "endLayer": body["nLayers"],
                                      "tpSize": 1, "tpRank": 0, "ppSize": 1, "ppRank": 0}}
    for n in nodes:
        c.post("/download/start", {"targetNodeId": n, "shardMetadata": full})
    deadline = time.time() + a.timeout
    while time.time() < deadline:
        dl = c.state()["downloads"]
        status = {}
        for n in nodes:
            for d in dl.get(n, []):
                k, v = next(iter(d.items()))
                if next(iter(v["shardMetadata"].values()))["modelCard"]["modelId"] == a.model:
                    status[n] = (k, v)
        if any(k == "DownloadFailed" for k, _ in status.values()):
            print({n: v.get("errorMessage") for n, (k, v) in status.items() if k == "DownloadFailed"}, file=sys.stderr)
            return 1
        if len(status) == len(nodes) and all(k == "DownloadCompleted" for k, _ in status.values()):
            print(f"{a.model} is on {len(nodes)} node(s)")
            return 0
        done = sum(k == "DownloadCompleted" for k, _ in status.values())
        print(f"\r{done}/{len(nodes)} nodes complete", end="", flush=True)
        time.sleep(2)
    print("timed out", file=sys.stderr)
    return 1


if __name__ == "__main__":
    raise SystemExit(main())
