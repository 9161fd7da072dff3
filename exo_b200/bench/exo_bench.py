"""Throughput benchmark of a running cluster through ``/bench/chat/completions``.

Method (the reference's, ``bench/METHODOLOGY.md`` and ``bench/exo_bench.py``): prompts of an exact
token length are built by binary search over a repeated atom string, measured with the model's own
tokenizer and chat template when they are available locally (otherwise with the server's reported
``prompt_tokens``); the bench endpoint runs with the prefix cache off (unless
``--use-prefix-cache``), EOS banned and output parsing bypassed; prefill and generation rates are
the server's per-task figures (``generation_tps = (tokens - 1) / (t_last - t_first)``); with
``--concurrency N`` the N requests are released together by a barrier and the aggregate is
``max(per-request tps) * N``.  ``--pp`` and ``--tg`` lists of equal length are run as pairs unless ``--all-combinations``;
``--stream`` reads the endpoint's server-sent events and adds client-side time to first token and inter-token gaps;
while requests are in flight a sampler thread reads the GPUs' utilisation, temperature, power and SM clock (NVML,
read-only) unless ``--no-system-metrics``; ``--dry-run`` lists the placements that would be used and the runs, and stops.
Results are one JSON object per (pp, tg, concurrency, repeat).

    python -m exo_b200.bench.exo_bench --model meta-llama/Llama-3.1-8B-Instruct --pp 512,2048 --tg 128 \
        --concurrency 1,8 --repeat 3 --place --sharding Tensor --min-nodes 2 --json-out results.jsonl
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import threading
import time
from collections.abc import Callable
from typing import Any

from .client import ApiError, ExoClient

ATOM = "a "


def build_prompt(count_tokens: Callable[[str], int], target: int, atom: str = ATOM) -> tuple[str, int]:
    """Content whose rendered prompt has exactly ``target`` tokens (or the closest reachable count)."""
    lo, hi = 0, max(8, target * 4)
    while count_tokens(atom * hi) < target and hi < (1 << 20):      # a counter that never grows must not loop forever
        hi *= 2
    best = (atom * hi, count_tokens(atom * hi))
    while lo <= hi:
        mid = (lo + hi) // 2
        n = count_tokens(atom * mid)
        if abs(n - target) < abs(best[1] - target):
            best = (atom * mid, n)
        if n == target:
            return atom * mid, n
        if n < target:
            lo = mid + 1
        else:
            hi = mid - 1
    return best


def local_token_counter(model_dir: str | None, vocab: int = 0) -> Callable[[str], int] | None:
    if not model_dir:
        return None
    from ..shared.messages import InputMessage, TextGenerationTaskParams
    from ..worker.engines.b200.tokenizer import load_tokenizer, render_prompt
    from pathlib import Path
    tok = load_tokenizer(Path(model_dir), vocab or 1 << 17)

    def count(content: str) -> int:
        p = TextGenerationTaskParams(model="m", input=[InputMessage(role="user", content=content)])
        text, _ = render_prompt(tok, p)
        return len(tok.encode(text, add_special_tokens=not getattr(tok, "chat_template", None)))
    return count


def server_token_counter(client: ExoClient, model: str) -> Callable[[str], int]:
    """No local tokenizer: ask the server (one-token bench request, read ``usage.prompt_tokens``)."""
    cache: dict[int, int] = {}

    def count(content: str) -> int:
        k = len(content)
        if k not in cache:
            r = client.post("/bench/chat/completions", {"model": model, "max_tokens": 2, "messages": [{"role": "user", "content": content}]})
            cache[k] = int(r["usage"]["prompt_tokens"])
        return cache[k]
    return count


def one_request(client: ExoClient, model: str, content: str, tg: int, use_prefix_cache: bool) -> dict[str, Any]:
    t0 = time.perf_counter()
    r = client.post("/bench/chat/completions", {"model": model, "max_tokens": tg, "temperature": 0.0, "use_prefix_cache": use_prefix_cache,
                                                "messages": [{"role": "user", "content": content}]})
    el = time.perf_counter() - t0
    gs = r.get("generation_stats") or {}
    return {"elapsed_s": el, "prompt_tps": gs.get("prompt_tps"), "generation_tps": gs.get("generation_tps"),
            "pp_tokens": gs.get("prompt_tokens") or (r.get("usage") or {}).get("prompt_tokens"),
            "tg_tokens": gs.get("generation_tokens") or (r.get("usage") or {}).get("completion_tokens"),
            "peak_memory_bytes": (gs.get("peak_memory_usage") or {}).get("inBytes") if isinstance(gs.get("peak_memory_usage"), dict) else None,
            "power": r.get("power_usage")}


def stream_request(client: ExoClient, model: str, content: str, tg: int, use_prefix_cache: bool) -> dict[str, Any]:
    """The same request with ``stream: true``: the server's statistics come in the last chunk; the time to the first token
    and the gaps between chunks are measured here."""
    import urllib.request
    body = json.dumps({"model": model, "max_tokens": tg, "temperature": 0.0, "use_prefix_cache": use_prefix_cache, "stream": True,
                       "messages": [{"role": "user", "content": content}]}).encode()
    req = urllib.request.Request(client.base + "/bench/chat/completions", data=body, method="POST", headers={"Content-Type": "application/json"})
    t0 = time.perf_counter()
    stamps: list[float] = []
    gs: dict[str, Any] = {}
    usage: dict[str, Any] = {}
    try:
        with urllib.request.urlopen(req, timeout=client.timeout) as r:
            for raw in r:
                line = raw.decode(errors="replace").strip()
                if line.startswith(": generation_stats "):          # the server's per-task figures ride in a comment line
                    gs = json.loads(line[len(": generation_stats "):])
                    continue
                if not line.startswith("data:") or line == "data: [DONE]":
                    continue
                ev = json.loads(line[5:])
                if ev.get("error"):
                    raise ApiError(500, json.dumps(ev["error"]))
                ch = (ev.get("choices") or [{}])[0]
                if (ch.get("delta") or {}).get("content") or (ch.get("delta") or {}).get("reasoning_content"):
                    stamps.append(time.perf_counter())
                gs = ev.get("generation_stats") or gs
                usage = ev.get("usage") or usage
    except OSError as e:
        raise ApiError(599, str(e)) from e
    gaps = [b - a for a, b in zip(stamps, stamps[1:])]
    return {"elapsed_s": time.perf_counter() - t0, "prompt_tps": gs.get("prompt_tps"), "generation_tps": gs.get("generation_tps"),
            "pp_tokens": gs.get("prompt_tokens") or usage.get("prompt_tokens"), "tg_tokens": gs.get("generation_tokens") or usage.get("completion_tokens"),
            "client_ttft_s": stamps[0] - t0 if stamps else None, "client_chunks": len(stamps),
            "client_gap_ms_p50": 1e3 * statistics.median(gaps) if gaps else None, "client_gap_ms_max": 1e3 * max(gaps) if gaps else None}


class SystemMetricsSampler:
    """Utilisation, temperature, power and SM clock of every visible GPU, sampled on a thread while requests run.  Reads only
    (NVML queries); without NVML or without a GPU it records nothing.  ``nvml`` may be any object with pynvml's functions."""

    def __init__(self, interval_s: float = 0.5, nvml: Any = None):
        self.interval, self.samples, self._stop, self._thread = interval_s, [], threading.Event(), None
        self.nvml, self.handles = nvml, []
        try:
            if self.nvml is None:
                import pynvml
                self.nvml = pynvml
            self.nvml.nvmlInit()
            self.handles = [self.nvml.nvmlDeviceGetHandleByIndex(i) for i in range(self.nvml.nvmlDeviceGetCount())]
        except Exception:  # noqa: BLE001 - no driver, no library: the benchmark runs without these columns
            self.handles = []

    def _read(self) -> list[dict[str, float]]:
        n, out = self.nvml, []
        for h in self.handles:
            try:
                out.append({"util": float(n.nvmlDeviceGetUtilizationRates(h).gpu), "temp_c": float(n.nvmlDeviceGetTemperature(h, 0)),
                            "power_w": n.nvmlDeviceGetPowerUsage(h) / 1000.0, "sm_mhz": float(n.nvmlDeviceGetClockInfo(h, 1))})
            except Exception:  # noqa: BLE001 - a query this device does not answer
                out.append({})
        return out

    def __enter__(self) -> "SystemMetricsSampler":
        self.samples = []
        if self.handles:
            self._stop.clear()

            def loop() -> None:
                while not self._stop.is_set():
                    self.samples.append(self._read())
                    self._stop.wait(self.interval)
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc: Any) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None

    def summary(self) -> dict[str, Any] | None:
        """Per GPU: mean and peak of every column over the samples; ``None`` when nothing was sampled."""
        if not self.samples:
            return None
        out = []
        for g in range(len(self.handles)):
            cols: dict[str, list[float]] = {}
            for s in self.samples:
                for k, v in (s[g] if g < len(s) else {}).items():
                    cols.setdefault(k, []).append(v)
            out.append({k: {"mean": round(statistics.fmean(v), 1), "max": max(v)} for k, v in cols.items()})
        return {"samples": len(self.samples), "interval_s": self.interval, "gpus": out}


class _NoNvml:
    """Stands in when sampling is off: initialisation fails, so the sampler holds no devices and records nothing."""

    def nvmlInit(self) -> None:
        raise RuntimeError("system metrics are off")


def plan_runs(pp: list[int], tg: list[int], all_combinations: bool) -> list[tuple[int, int]]:
    """Lists of equal length (longer than one) are pairs; otherwise, or when asked, the cartesian product."""
    if not all_combinations and len(pp) == len(tg) and len(pp) > 1:
        return list(zip(pp, tg))
    return [(p, t) for p in pp for t in tg]


def concurrent_requests(make_client: Callable[[], ExoClient], n: int, model: str, content: str, tg: int, use_prefix_cache: bool,
                        request: Callable[..., dict[str, Any]] | None = None) -> list[dict[str, Any]]:
    """N requests released at the same instant; every ``elapsed_s`` counts from the shared start."""
    barrier = threading.Barrier(n)
    start: list[float] = []
    lock = threading.Lock()
    results: list[dict[str, Any] | BaseException] = [RuntimeError("not run")] * n

    def work(i: int) -> None:
        c = make_client()
        barrier.wait()
        with lock:
            if not start:
                start.append(time.perf_counter())
        try:
            r = (request or one_request)(c, model, content, tg, use_prefix_cache)
            r["elapsed_s"] = time.perf_counter() - start[0]
            results[i] = r
        except BaseException as e:  # noqa: BLE001 - reported per request
            results[i] = e
    threads = [threading.Thread(target=work, args=(i,)) for i in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    errs = [r for r in results if isinstance(r, BaseException)]
    if errs:
        raise errs[0]
    return results  # type: ignore[return-value]


def aggregate(rows: list[dict[str, Any]], concurrency: int) -> dict[str, Any]:
    tps = [r["generation_tps"] for r in rows if r.get("generation_tps")]
    pps = [r["prompt_tps"] for r in rows if r.get("prompt_tps")]
    per_req = max(tps) if tps else None
    return {"concurrency": concurrency, "per_req_gen_tps": per_req, "agg_gen_tps": per_req * concurrency if per_req else None,
            "mean_prompt_tps": statistics.fmean(pps) if pps else None, "batch_wall_s": max(r["elapsed_s"] for r in rows),
            "pp_tokens": rows[0].get("pp_tokens"), "tg_tokens": rows[0].get("tg_tokens")}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="exo-bench")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--pp", default="512", help="prompt lengths, comma separated")
    ap.add_argument("--tg", default="128", help="generation lengths, comma separated (>= 2)")
    ap.add_argument("--concurrency", default="1")
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--use-prefix-cache", action="store_true")
    ap.add_argument("--model-dir", default=None, help="local checkpoint directory: exact prompt sizing with its tokenizer")
    ap.add_argument("--place", action="store_true", help="place an instance first (and delete it afterwards)")
    ap.add_argument("--sharding", default="Tensor", choices=["Tensor", "Pipeline", "both"])
    ap.add_argument("--instance-meta", default="any")
    ap.add_argument("--min-nodes", type=int, default=1)
    ap.add_argument("--max-nodes", type=int, default=0)
    ap.add_argument("--settle-timeout", type=float, default=60.0)
    ap.add_argument("--ready-timeout", type=float, default=1800.0)
    ap.add_argument("--danger-delete-downloads", action="store_true")
    ap.add_argument("--reuse-instance", action="store_true")
    ap.add_argument("--json-out", default=None)
    ap.add_argument("--stdout", action="store_true")
    ap.add_argument("--all-combinations", action="store_true", help="every pp x tg pair even when the two lists have equal length")
    ap.add_argument("--stream", action="store_true", help="stream the responses and record client-side first-token and inter-token times")
    ap.add_argument("--no-system-metrics", action="store_true", help="do not sample GPU utilisation / temperature / power / clocks")
    ap.add_argument("--metrics-interval", type=float, default=0.5)
    ap.add_argument("--dry-run", action="store_true", help="list the placements that match and the runs, then exit")
    a = ap.parse_args(argv)
    client = ExoClient(a.host, a.port)
    harness = None
    runs = plan_runs([int(x) for x in a.pp.split(",")], [int(x) for x in a.tg.split(",")], a.all_combinations)
    if any(tg < 2 for _, tg in runs):
        print("tg must be >= 2: the generation rate is measured between the first and the last token", file=sys.stderr)
        return 2
    if a.dry_run:
        previews = []
        try:
            previews = [p for p in client.previews(a.model) if not p.get("error")]
        except (ApiError, OSError) as e:
            print(f"no placement previews: {e}", file=sys.stderr)
        print(json.dumps({"model": a.model, "runs": [{"pp": p, "tg": t, "concurrency": int(c)} for p, t in runs for c in a.concurrency.split(",")],
                          "repeat": a.repeat, "warmup": a.warmup, "placements": [
                              {"sharding": p.get("sharding"), "instance_meta": p.get("instance_meta"),
                               "nodes": len(((p.get("instance") or {}).get(next(iter(p.get("instance") or {"": {}}), ""), {}) or {})
                                            .get("shardAssignments", {}).get("nodeToRunner", {}))} for p in previews]}))
        return 0
    if a.place:
        # resolve the name, wait for a placement of the wanted shape, make room and download, launch, wait until ready
        from .harness import Harness
        harness = Harness(client, log=lambda m: print(m, file=sys.stderr))
        a.model, _iid, dl = harness.instance_for(a)
        if dl is not None:
            print(f"downloaded in {dl:.0f}s", file=sys.stderr)
    else:
        client.wait_ready(a.model)
    counter = local_token_counter(a.model_dir) or server_token_counter(client, a.model)
    out = open(a.json_out, "a") if a.json_out else None
    rc = 0
    request = stream_request if a.stream else one_request
    sampler = None if a.no_system_metrics else SystemMetricsSampler(a.metrics_interval)
    prompts: dict[int, tuple[str, int]] = {}
    try:
        for pp, tg in runs:
            if pp not in prompts:
                prompts[pp] = build_prompt(counter, pp)
            content, actual = prompts[pp]
            for conc in [int(x) for x in a.concurrency.split(",")]:
                for rep in range(-a.warmup, a.repeat):
                    try:
                        with (sampler or SystemMetricsSampler(nvml=_NoNvml())) as sm:
                            rows = ([request(client, a.model, content, tg, a.use_prefix_cache)] if conc == 1 else
                                    concurrent_requests(lambda: ExoClient(a.host, a.port), conc, a.model, content, tg, a.use_prefix_cache, request))
                    except ApiError as e:
                        print(f"pp={pp} tg={tg} c={conc}: {e}", file=sys.stderr)
                        rc = 1
                        continue
                    if rep < 0:
                        continue
                    row = {"model": a.model, "pp_target": pp, "pp_built": actual, "tg": tg, "repeat": rep, **aggregate(rows, conc),
                           "system": sm.summary(), "requests": rows}
                    line = json.dumps(row)
                    if out:
                        out.write(line + "\n")
                        out.flush()
                    if a.stdout or not out:
                        print(line)
    finally:
        if out:
            out.close()
        if harness is not None:
            harness.teardown()
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
