"""Accuracy evaluation against a running cluster (multiple-choice and exact-match tasks).

Counterpart of the reference's ``bench/exo_eval.py``, reduced to what needs no dataset download:
tasks come from a local JSONL file with one of two shapes —
``{"question", "choices": [...], "answer": index}`` (scored by the letter the model answers with) or
``{"prompt", "answer": "text"}`` (exact match after normalisation).  Requests go through
``/v1/chat/completions`` with temperature 0, ``--concurrency`` at a time.
"""
from __future__ import annotations

import argparse
import json
import re
import string
import threading
from typing import Any

from .client import ExoClient

LETTERS = string.ascii_uppercase


def format_mc(q: dict[str, Any]) -> str:
    opts = "\n".join(f"{LETTERS[i]}. {c}" for i, c in enumerate(q["choices"]))
    return f"{q['question']}\n{opts}\nAnswer with the letter only."


def extract_letter(text: str, n: int) -> int | None:
    m = re.search(r"\b([A-%s])\b" % LETTERS[n - 1], text.strip().upper())
    return LETTERS.index(m.group(1)) if m else None


def normalise(s: str) -> str:
    return re.sub(r"\s+", " ", s.strip().lower().strip(string.punctuation))


def score(q: dict[str, Any], reply: str) -> bool:
    if "choices" in q:
        return extract_letter(reply, len(q["choices"])) == int(q["answer"])
    return normalise(reply) == normalise(str(q["answer"]))


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--tasks", required=True, help="JSONL file")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--no-thinking", action="store_true")
    a = ap.parse_args(argv)
    with open(a.tasks) as f:
        qs = [json.loads(ln) for ln in f if ln.strip()]
    if a.limit:
        qs = qs[:a.limit]
    results: list[bool | None] = [None] * len(qs)
    sem = threading.Semaphore(a.concurrency)

    def work(i: int) -> None:
        with sem:
            c = ExoClient(a.host, a.port)
            q = qs[i]
            body: dict[str, Any] = {"model": a.model, "temperature": 0.0, "max_tokens": a.max_tokens,
                                    "messages": [{"role": "user", "content": format_mc(q) if "choices" in q else q["prompt"]}]}
            if a.no_thinking:
                body["enable_thinking"] = False
            try:
                r = c.post("/v1/chat/completions", body)
                results[i] = score(q, r["choices"][0]["message"].get("content") or "")
            except Exception:  # noqa: BLE001 - counted as an error, not as a wrong answer
                results[i] = None
    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(qs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    done = [r for r in results if r is not None]
    print(json.dumps({"model": a.model, "n": len(qs), "answered": len(done), "correct": sum(done),
                      "accuracy": sum(done) / len(done) if done else None, "errors": len(qs) - len(done)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
