"""Tool-calling evaluation against a running cluster: does the model call the right function with
arguments that satisfy the schema, in every API dialect?

Counterpart of the reference's ``bench/eval_tool_calls.py``.  Scenarios are (prompt, tools,
expected function, required argument names); each is sent through ``/v1/chat/completions``,
``/v1/messages`` and ``/v1/responses`` and scored on: a tool call was returned (not text), the
function name matches, the arguments are valid JSON and contain the required keys with the schema's
types.  A JSONL file of extra scenarios can be supplied with ``--scenarios``.
"""
from __future__ import annotations

import argparse
import json
from typing import Any

from .client import ApiError, ExoClient

WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "Current weather for a city",
           "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "unit": {"type": "string", "enum": ["c", "f"]}},
                          "required": ["city"]}}}
CALC = {"type": "function", "function": {"name": "add", "description": "Add two integers",
        "parameters": {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "integer"}}, "required": ["a", "b"]}}}
BUILTIN = [
    {"prompt": "What is the weather in Paris right now?", "tools": [WEATHER, CALC], "expect": "get_weather", "required": ["city"]},
    {"prompt": "Use the tool to add 17 and 25.", "tools": [WEATHER, CALC], "expect": "add", "required": ["a", "b"]},
]
_JSON_TYPES = {"string": str, "integer": int, "number": (int, float), "boolean": bool, "object": dict, "array": list}


def score_call(name: str | None, arguments: Any, scenario: dict[str, Any]) -> dict[str, bool]:
    out = {"called": name is not None, "name_ok": name == scenario["expect"], "json_ok": False, "args_ok": False}
    if name is None:
        return out
    try:
        args = json.loads(arguments) if isinstance(arguments, str) else arguments
        out["json_ok"] = isinstance(args, dict)
    except (TypeError, json.JSONDecodeError):
        return out
    if not out["json_ok"]:
        return out
    props = next((t["function"]["parameters"].get("properties", {}) for t in scenario["tools"] if t["function"]["name"] == name), {})
    ok = all(k in args for k in scenario["required"])
    for k, v in args.items():
        ty = _JSON_TYPES.get((props.get(k) or {}).get("type", ""), object)
        ok = ok and isinstance(v, ty) and not (ty is int and isinstance(v, bool))
    out["args_ok"] = ok
    return out


def call_chat(c: ExoClient, model: str, sc: dict[str, Any]) -> tuple[str | None, Any]:
    r = c.post("/v1/chat/completions", {"model": model, "messages": [{"role": "user", "content": sc["prompt"]}], "tools": sc["tools"],
                                       "temperature": 0.0, "max_tokens": 512})
    tcs = r["choices"][0]["message"].get("tool_calls") or []
    return (tcs[0]["function"]["name"], tcs[0]["function"]["arguments"]) if tcs else (None, None)


def call_claude(c: ExoClient, model: str, sc: dict[str, Any]) -> tuple[str | None, Any]:
    tools = [{"name": t["function"]["name"], "description": t["function"].get("description", ""), "input_schema": t["function"]["parameters"]}
             for t in sc["tools"]]
    r = c.post("/v1/messages", {"model": model, "max_tokens": 512, "temperature": 0.0, "tools": tools,
                                "messages": [{"role": "user", "content": sc["prompt"]}]})
    for b in r["content"]:
        if b["type"] == "tool_use":
            return b["name"], b["input"]
    return None, None


def call_responses(c: ExoClient, model: str, sc: dict[str, Any]) -> tuple[str | None, Any]:
    tools = [{"type": "function", "name": t["function"]["name"], "description": t["function"].get("description", ""),
              "parameters": t["function"]["parameters"]} for t in sc["tools"]]
    r = c.post("/v1/responses", {"model": model, "input": sc["prompt"], "tools": tools, "temperature": 0.0, "max_output_tokens": 512})
    for it in r["output"]:
        if it["type"] == "function_call":
            return it["name"], it["arguments"]
    return None, None


DIALECTS = {"chat": call_chat, "claude": call_claude, "responses": call_responses}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--scenarios", default=None, help="JSONL file of {prompt, tools, expect, required}")
    ap.add_argument("--dialects", default="chat,claude,responses")
    a = ap.parse_args(argv)
    scenarios = list(BUILTIN)
    if a.scenarios:
        with open(a.scenarios) as f:
            scenarios += [json.loads(ln) for ln in f if ln.strip()]
    c = ExoClient(a.host, a.port)
    c.wait_ready(a.model, timeout=60)
    rows, passed = [], 0
    for sc in scenarios:
        for d in a.dialects.split(","):
            try:
                name, args = DIALECTS[d](c, a.model, sc)
                s = score_call(name, args, sc)
            except (ApiError, KeyError) as e:
                s = {"called": False, "name_ok": False, "json_ok": False, "args_ok": False, "error": str(e)}
            s.update(dialect=d, prompt=sc["prompt"])
            rows.append(s)
            passed += all(s.get(k) for k in ("called", "name_ok", "json_ok", "args_ok"))
    print(json.dumps({"model": a.model, "passed": passed, "total": len(rows), "rows": rows}))
    return 0 if passed == len(rows) else 1


if __name__ == "__main__":
    raise SystemExit(main())
