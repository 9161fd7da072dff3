"""Fire N concurrent streaming chat requests and report per-request and aggregate token rates.

Counterpart of the reference's ``bench/parallel_requests.py``: a load generator for continuous
batching.  Each request streams (SSE), so time-to-first-token and inter-token rates are measured
on the client as well.

    python -m exo_b200.bench.parallel_requests --model <id> --n 8 --max-tokens 128 --prompt "Tell me a story"
"""
from __future__ import annotations

import argparse
import json
import threading
import time
import urllib.request


def stream_one(base: str, model: str, prompt: str, max_tokens: int, out: dict, barrier: threading.Barrier) -> None:
    body = json.dumps({"model": model, "stream": True, "max_tokens": max_tokens, "messages": [{"role": "user", "content": prompt}]}).encode()
    req = urllib.request.Request(base + "/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
    barrier.wait()
    t0 = time.perf_counter()
    first = last = None
    n = 0
    with urllib.request.urlopen(req, timeout=3600) as r:
        for raw in r:
            line = raw.decode().strip()
            if not line.startswith("data: ") or line == "data: [DONE]":
                continue
            d = json.loads(line[6:])
            if "error" in d:
                out["error"] = d["error"].get("message")
                return
            delta = d["choices"][0]["delta"]
            if delta.get("content") or delta.get("reasoning_content"):
                now = time.perf_counter()
                first = first or now
                last = now
                n += 1
    out.update(ttft_s=(first - t0) if first else None, tokens=n, total_s=time.perf_counter() - t0,
               gen_tps=(n - 1) / (last - first) if n > 1 and last > first else None)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--prompt", default="Write a short story about a lighthouse keeper.")
    a = ap.parse_args(argv)
    base = f"http://{a.host}:{a.port}"
    results = [dict() for _ in range(a.n)]
    barrier = threading.Barrier(a.n)
    threads = [threading.Thread(target=stream_one, args=(base, a.model, a.prompt, a.max_tokens, results[i], barrier)) for i in range(a.n)]
    t0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if r.get("tokens")]
    summary = {"n": a.n, "ok": len(ok), "wall_s": wall, "total_tokens": sum(r["tokens"] for r in ok),
               "agg_tok_s": sum(r["tokens"] for r in ok) / wall if wall > 0 else None,
               "max_ttft_s": max((r["ttft_s"] for r in ok if r.get("ttft_s")), default=None), "requests": results}
    print(json.dumps(summary))
    return 0 if len(ok) == a.n else 1


if __name__ == "__main__":
    raise SystemExit(main())
