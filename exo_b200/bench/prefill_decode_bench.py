"""Prefill/decode disaggregation against a running cluster: is a request faster when one instance computes the prompt
and another decodes?

Counterpart of the reference's ``bench/prefill_decode_bench.py``.  Two phases over the same grid of prompt lengths
(``--pp``) and output lengths (``--tg``), each point repeated ``--repeat`` times with the prefix cache off:

1. *baseline*: one instance of the model serves the whole request;
2. *disaggregated*: a second instance is placed on other nodes, ``POST /v1/instance-links`` names the first as prefill
   source and the second as decode target, and the same requests are sent again.  The master routes them to the decode
   instance with the prefill endpoint attached; the worker fetches the prompt's KV from the prefill instance when the
   uncached part of the prompt is long enough to pay for the transfer.

The table printed at the end gives, per grid point, time to first token, prompt tokens/s, decode tokens/s and wall time
for both phases and their ratio.  ``--config file.toml`` supplies any flag (``[defaults]`` table, keys as flag names);
``--dry-run`` prints the plan (placements chosen, grid) and touches nothing.  Instances and the link this tool created
are removed at the end unless ``--keep`` is given.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
import tomllib
from typing import Any

from .client import ApiError, ExoClient
from .exo_bench import build_prompt, local_token_counter, one_request, server_token_counter


def ints(s: str) -> list[int]:
    return [int(x) for x in str(s).replace(" ", "").split(",") if x]


def untag(instance: dict[str, Any]) -> dict[str, Any]:
    """``{"NvlinkInstance": {...}}`` → the inner record (already-bare records pass through)."""
    return instance if "shardAssignments" in instance else next(iter(instance.values()))


def nodes_of(instance: dict[str, Any]) -> set[str]:
    return set(untag(instance)["shardAssignments"]["nodeToRunner"])


def pick_disjoint(previews: list[dict[str, Any]], sharding: str, n_nodes: int) -> tuple[dict[str, Any], dict[str, Any]] | None:
    """Two valid placements of the wanted shape that share no node."""
    def shape_ok(p: dict[str, Any]) -> bool:
        inst = p.get("instance")
        if p.get("error") or not inst:
            return False
        return p.get("sharding", sharding) == sharding and len(nodes_of(inst)) == n_nodes
    ok = [p for p in previews if shape_ok(p)]
    for i, a in enumerate(ok):
        for b in ok[i + 1:]:
            if not (nodes_of(a["instance"]) & nodes_of(b["instance"])):
                return a, b
    return None


def run_grid(client: ExoClient, model: str, prompts: dict[int, str], tgs: list[int], repeat: int, label: str) -> list[dict[str, Any]]:
    rows = []
    for pp, content in prompts.items():
        for tg in tgs:
            for k in range(repeat):
                r = one_request(client, model, content + f" #{label}{k}", tg, use_prefix_cache=False)
                r.update(phase=label, pp=pp, tg=tg, rep=k)
                if r.get("prompt_tps") and r.get("pp_tokens"):
                    r["ttft_s"] = r["pp_tokens"] / r["prompt_tps"]
                rows.append(r)
                print(f"[{label}] pp={pp} tg={tg} #{k}: prompt {r.get('prompt_tps') or 0:.0f} tok/s, decode "
                      f"{r.get('generation_tps') or 0:.1f} tok/s, wall {r['elapsed_s']:.2f}s", file=sys.stderr)
    return rows


def summarise(rows: list[dict[str, Any]]) -> dict[tuple[int, int], dict[str, float]]:
    out: dict[tuple[int, int], dict[str, float]] = {}
    for key in sorted({(r["pp"], r["tg"]) for r in rows}):
        pts = [r for r in rows if (r["pp"], r["tg"]) == key]
        med = lambda f: statistics.median([r[f] for r in pts if r.get(f) is not None] or [float("nan")])   # noqa: E731
        out[key] = {"ttft_s": med("ttft_s"), "prompt_tps": med("prompt_tps"), "generation_tps": med("generation_tps"),
                    "elapsed_s": med("elapsed_s")}
    return out


def diff_table(base: dict[tuple[int, int], dict[str, float]], dis: dict[tuple[int, int], dict[str, float]]) -> str:
    head = ("pp", "tg", "ttft base", "ttft disagg", "x", "decode base", "decode disagg", "x", "wall base", "wall disagg", "x")
    lines = [head]
    for key in sorted(base):
        b, d = base[key], dis.get(key)
        if d is None:
            continue
        ratio = lambda x, y: f"{x / y:.2f}" if y and y == y and x == x else "-"     # noqa: E731
        lines.append((str(key[0]), str(key[1]), f"{b['ttft_s']:.3f}s", f"{d['ttft_s']:.3f}s", ratio(b["ttft_s"], d["ttft_s"]),
                      f"{b['generation_tps']:.1f}", f"{d['generation_tps']:.1f}", ratio(d["generation_tps"], b["generation_tps"]),
                      f"{b['elapsed_s']:.2f}s", f"{d['elapsed_s']:.2f}s", ratio(b["elapsed_s"], d["elapsed_s"])))
    w = [max(len(ln[i]) for ln in lines) for i in range(len(head))]
    return "\n".join("  ".join(c.rjust(w[i]) for i, c in enumerate(ln)) for ln in lines)


def parse_args(argv: list[str] | None) -> argparse.Namespace:
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--config")
    known, _ = pre.parse_known_args(argv)
    defaults: dict[str, Any] = {}
    if known.config:
        with open(known.config, "rb") as f:
            cfg = tomllib.load(f)
        defaults = {k.replace("-", "_"): v for k, v in (cfg.get("defaults") or cfg).items() if not isinstance(v, dict)}
    ap = argparse.ArgumentParser(prog="prefill-decode-bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", help="TOML file with flag values")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required="model" not in defaults)
    ap.add_argument("--pp", default="2048,8192")
    ap.add_argument("--tg", default="128")
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--sharding", default="Tensor")
    ap.add_argument("--nodes-per-instance", type=int, default=1)
    ap.add_argument("--model-dir", default=None, help="tokenizer for exact prompt sizing (else the server is asked)")
    ap.add_argument("--skip-baseline", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--keep", action="store_true")
    ap.add_argument("--json-out", default=None)
    ap.set_defaults(**defaults)
    return ap.parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    a = parse_args(argv)
    client = ExoClient(a.host, a.port)
    pps, tgs = ints(a.pp), ints(a.tg)
    pair = pick_disjoint(client.previews(a.model), a.sharding, a.nodes_per_instance)
    if pair is None:
        print(f"need two placements of {a.model} ({a.sharding}, {a.nodes_per_instance} node(s) each) on disjoint nodes", file=sys.stderr)
        return 2
    plan = {"model": a.model, "grid": [[p, t] for p in pps for t in tgs], "repeat": a.repeat,
            "prefill_nodes": sorted(nodes_of(pair[0]["instance"])), "decode_nodes": sorted(nodes_of(pair[1]["instance"]))}
    if a.dry_run:
        print(json.dumps(plan, indent=1))
        return 0
    created: list[str] = []
    link_ids_before = {ln["linkId"] if "linkId" in ln else ln.get("link_id") for ln in client.get("/v1/instance-links")}
    rows: list[dict[str, Any]] = []
    try:
        before = {iid for iid, _ in client.instances_of(a.model)}
        client.post("/instance", {"instance": pair[0]["instance"]})
        first = client.wait_ready(a.model)
        created += [i for i, _ in client.instances_of(a.model) if i not in before]
        counter = local_token_counter(a.model_dir) or server_token_counter(client, a.model)
        prompts = {pp: build_prompt(counter, pp)[0] for pp in pps}
        if not a.skip_baseline:
            rows += run_grid(client, a.model, prompts, tgs, a.repeat, "baseline")
        have = {iid for iid, _ in client.instances_of(a.model)}
        client.post("/instance", {"instance": pair[1]["instance"]})
        deadline = time.time() + 1800
        second = None
        while time.time() < deadline and second is None:
            new = [i for i, _ in client.instances_of(a.model) if i not in have]
            if new:
                st = client.state()
                inst = untag(st["instances"][new[0]])
                rids = list(inst["shardAssignments"]["runnerToShard"])
                status = [next(iter(st["runners"].get(r, {"Missing": {}}))) for r in rids]
                if any(s == "RunnerFailed" for s in status):
                    raise RuntimeError(f"decode instance failed: {status}")
                if all(s in ("RunnerReady", "RunnerRunning") for s in status):
                    second = new[0]
            time.sleep(0.5)
        if second is None:
            raise TimeoutError("decode instance did not become ready")
        created.append(second)
        client.post("/v1/instance-links", {"prefill_instances": [first], "decode_instances": [second]})
        time.sleep(1.0)                                        # the link reaches every worker through the event log
        rows += run_grid(client, a.model, prompts, tgs, a.repeat, "disaggregated")
    except (ApiError, RuntimeError, TimeoutError) as e:
        print(f"stopped: {e}", file=sys.stderr)
        return 1
    finally:
        if not a.keep:
            for ln in client.get("/v1/instance-links"):
                lid = ln.get("linkId") or ln.get("link_id")
                if lid not in link_ids_before:
                    client.delete(f"/v1/instance-links/{lid}")
            for iid in created:
                try:
                    client.delete_instance(iid)
                except ApiError:
                    pass
    base = summarise([r for r in rows if r["phase"] == "baseline"])
    dis = summarise([r for r in rows if r["phase"] == "disaggregated"])
    if base and dis:
        print(diff_table(base, dis))
    if a.json_out:
        with open(a.json_out, "w") as f:
            json.dump({"plan": plan, "rows": rows}, f, indent=1)
    print(json.dumps({"model": a.model, "baseline": {f"{k[0]}x{k[1]}": v for k, v in base.items()},
                      "disaggregated": {f"{k[0]}x{k[1]}": v for k, v in dis.items()}}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
