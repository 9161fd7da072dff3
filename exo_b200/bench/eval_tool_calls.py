"""Tool-calling evaluation against a running cluster, in every API dialect.

Counterpart of the reference's ``bench/eval_tool_calls.py`` (scenario file ``bench/scenarios.toml``).  A scenario is a
conversation (any number of earlier turns, tool calls and tool results among them), the tools on offer, and what should
happen next: a call of a named function whose arguments are valid JSON with the required keys and the schema's types
(optionally an array argument whose items each carry required keys), or — for questions no tool helps with — no call at
all.  A scenario with a ``tool_result`` continues: the result is sent back in the dialect's own form and the model has to
answer in text without calling again.  Every scenario runs through ``/v1/chat/completions``, ``/v1/messages`` and
``/v1/responses``; one dialect table holds how each builds its request, where its tool calls are, and how it takes a result
back.  Scenarios come from the built-in list, a TOML file (``[tools.<name>]`` tables + ``[[scenarios]]``) or JSONL.
"""
from __future__ import annotations

import argparse
import json
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from .client import ApiError, ExoClient

_JSON_TYPES = {"string": str, "integer": int, "number": (int, float), "boolean": bool, "object": dict, "array": list}


def function_tool(name: str, description: str, properties: dict[str, Any], required: list[str]) -> dict[str, Any]:
    return {"type": "function", "function": {"name": name, "description": description,
                                             "parameters": {"type": "object", "properties": properties, "required": required}}}


WEATHER = function_tool("get_weather", "Current weather for a city", {"city": {"type": "string"}, "unit": {"type": "string", "enum": ["c", "f"]}},
                        ["city"])
CALC = function_tool("add", "Add two integers", {"a": {"type": "integer"}, "b": {"type": "integer"}}, ["a", "b"])
TODO = function_tool("write_todos", "Replace the to-do list", {"todos": {"type": "array", "items": {
    "type": "object", "properties": {"title": {"type": "string"}, "done": {"type": "boolean"}}, "required": ["title", "done"]}}}, ["todos"])


@dataclass
class Scenario:
    name: str
    messages: list[dict[str, Any]]
    tools: list[dict[str, Any]]
    expect_call: bool = True
    expect: str | None = None                       # the function that should be called
    required: list[str] = field(default_factory=list)
    tool_result: Any = None                         # if set: sent back after a correct call; the model must then answer in text
    array_key: str | None = None                    # an array argument ...
    item_keys: list[str] = field(default_factory=list)   # ... whose items must each have these keys

    @property
    def prompt(self) -> str:
        return next((m.get("content") or "" for m in reversed(self.messages) if m["role"] == "user"), "")


def _say(text: str) -> list[dict[str, Any]]:
    return [{"role": "user", "content": text}]


BUILTIN = [
    Scenario("weather", _say("What is the weather in Paris right now?"), [WEATHER, CALC], expect="get_weather", required=["city"],
             tool_result={"temp_c": 18, "sky": "overcast"}),
    Scenario("add", _say("Use the tool to add 17 and 25."), [WEATHER, CALC], expect="add", required=["a", "b"], tool_result={"sum": 42}),
    Scenario("no-tool", _say("Say hello in French. Do not use any tool."), [WEATHER, CALC], expect_call=False),
    Scenario("after-a-result", [
        {"role": "user", "content": "Compare the weather in Paris and in Rome."},
        {"role": "assistant", "content": None, "tool_calls": [{"id": "call_1", "type": "function",
                                                                "function": {"name": "get_weather", "arguments": "{\"city\": \"Paris\"}"}}]},
        {"role": "tool", "tool_call_id": "call_1", "content": "{\"temp_c\": 18}"}], [WEATHER], expect="get_weather", required=["city"]),
    Scenario("array-of-objects", _say("Put two items on my to-do list: buy milk (not done) and call Ana (done)."), [TODO], expect="write_todos",
             required=["todos"], array_key="todos", item_keys=["title", "done"]),
]


def load_scenarios(path: Path) -> list[Scenario]:
    """TOML: ``[tools.NAME]`` (description, properties, required) and ``[[scenarios]]`` (name, messages, tools = [names],
    expect_tool_call, expected_function, required_arg_keys, tool_result, nested_array_key, required_item_keys); messages may
    carry ``tool_calls = [{id, name, arguments = {...}}]`` and ``tool_call_id``.  JSONL: one scenario object per line with
    this module's field names (``prompt`` may stand in for ``messages``)."""
    if path.suffix == ".jsonl":
        out = []
        for ln in path.read_text().splitlines():
            if ln.strip():
                d = json.loads(ln)
                if "prompt" in d:
                    d["messages"] = _say(d.pop("prompt"))
                d.setdefault("name", f"line-{len(out)}")
                out.append(Scenario(**d))
        return out
    data = tomllib.loads(path.read_text())
    tools = {n: function_tool(n, t.get("description", ""), t.get("properties", {}), t.get("required", [])) for n, t in data.get("tools", {}).items()}
    out = []
    for s in data.get("scenarios", []):
        msgs = []
        for m in s.get("messages", []):
            msg: dict[str, Any] = {"role": m["role"]}
            if "content" in m:
                msg["content"] = m["content"]
            if "tool_calls" in m:
                msg["tool_calls"] = [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": json.dumps(c["arguments"])}}
                                     for c in m["tool_calls"]]
            if "tool_call_id" in m:
                msg["tool_call_id"] = m["tool_call_id"]
            msgs.append(msg)
        out.append(Scenario(name=s["name"], messages=msgs, tools=[tools[t] for t in s["tools"]] if "tools" in s else list(tools.values()),
                            expect_call=s.get("expect_tool_call", True), expect=s.get("expected_function"),
                            required=list(s.get("required_arg_keys") or []), tool_result=s.get("tool_result"),
                            array_key=s.get("nested_array_key"), item_keys=list(s.get("required_item_keys") or [])))
    return out


# ---------------------------------------------------------------------------------------------------------------------
# scoring
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Reply:
    text: str
    calls: list[tuple[str, str, Any]]               # (call id, function name, arguments as the API returned them)
    finish: str | None = None


def score_call(name: str | None, arguments: Any, scenario: Scenario | dict[str, Any]) -> dict[str, bool]:
    """``called`` / ``name_ok`` / ``json_ok`` / ``args_ok`` for one returned call (or none)."""
    sc = scenario if isinstance(scenario, Scenario) else Scenario(
        name="", messages=_say(scenario.get("prompt", "")), tools=scenario["tools"], expect=scenario["expect"],
        required=list(scenario.get("required", [])), array_key=scenario.get("array_key"), item_keys=list(scenario.get("item_keys", [])))
    out = {"called": name is not None, "name_ok": name == sc.expect, "json_ok": False, "args_ok": False}
    if name is None:
        return out
    try:
        args = json.loads(arguments) if isinstance(arguments, str) else arguments
        out["json_ok"] = isinstance(args, dict)
    except (TypeError, json.JSONDecodeError):
        return out
    if not out["json_ok"]:
        return out
    props = next((t["function"]["parameters"].get("properties", {}) for t in sc.tools if t["function"]["name"] == name), {})
    ok = all(k in args for k in sc.required)
    for k, v in args.items():
        ty = _JSON_TYPES.get((props.get(k) or {}).get("type", ""), object)
        ok = ok and isinstance(v, ty) and not (ty is int and isinstance(v, bool))
        if "enum" in (props.get(k) or {}):
            ok = ok and v in props[k]["enum"]
    if sc.array_key:
        items = args.get(sc.array_key)
        if isinstance(items, str):                  # some models return the array as a JSON string
            try:
                items = json.loads(items)
            except json.JSONDecodeError:
                items = None
        ok = ok and isinstance(items, list) and len(items) > 0 and all(isinstance(it, dict) and all(k in it for k in sc.item_keys) for it in items)
    out["args_ok"] = ok
    return out


# ---------------------------------------------------------------------------------------------------------------------
# dialects: request, parse, and how a tool result goes back
# ---------------------------------------------------------------------------------------------------------------------
def _chat_request(model: str, messages: list[dict[str, Any]], tools: list[dict[str, Any]]) -> tuple[str, dict[str, Any]]:
    return "/v1/chat/completions", {"model": model, "messages": messages, "tools": tools, "temperature": 0.0, "max_tokens": 1024}


def _chat_parse(r: dict[str, Any]) -> Reply:
    ch = r["choices"][0]
    m = ch["message"]
    return Reply(m.get("content") or "", [(c.get("id", ""), c["function"]["name"], c["function"]["arguments"]) for c in m.get("tool_calls") or []],
                 ch.get("finish_reason"))


def _chat_followup(messages: list[dict[str, Any]], reply: Reply, result: str) -> list[dict[str, Any]]:
    cid, name, args = reply.calls[0]
    return messages + [{"role": "assistant", "content": reply.text or None, "tool_calls": [
        {"id": cid or "call_0", "type": "function", "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}}]},
        {"role": "tool", "tool_call_id": cid or "call_0", "content": result}]


def _claude_messages(messages: list[dict[str, Any]]) -> tuple[str | None, list[dict[str, Any]]]:
    """OpenAI-style history in the Messages form: system text apart, calls as ``tool_use`` blocks, results as ``tool_result``
    blocks of a user turn (consecutive results share one turn)."""
    system, out = None, []
    for m in messages:
        if m["role"] == "system":
            system = m.get("content")
        elif m["role"] == "assistant":
            blocks: list[dict[str, Any]] = [{"type": "text", "text": m["content"]}] if m.get("content") else []
            for c in m.get("tool_calls") or []:
                blocks.append({"type": "tool_use", "id": c["id"], "name": c["function"]["name"], "input": json.loads(c["function"]["arguments"] or "{}")})
            out.append({"role": "assistant", "content": blocks})
        elif m["role"] == "tool":
            block = {"type": "tool_result", "tool_use_id": m["tool_call_id"], "content": m.get("content", "")}
            if out and out[-1]["role"] == "user" and isinstance(out[-1]["content"], list) and out[-1]["content"][0]["type"] == "tool_result":
                out[-1]["content"].append(block)
            else:
                out.append({"role": "user", "content": [block]})
        else:
            out.append({"role": "user", "content": m.get("content", "")})
    return system, out


def _claude_request(model: str, messages: list[dict[str, Any]], tools: list[dict[str, Any]]) -> tuple[str, dict[str, Any]]:
    system, msgs = _claude_messages(messages)
    body = {"model": model, "max_tokens": 1024, "temperature": 0.0, "messages": msgs,
            "tools": [{"name": t["function"]["name"], "description": t["function"].get("description", ""), "input_schema": t["function"]["parameters"]}
                      for t in tools]}
    if system:
        body["system"] = system
    return "/v1/messages", body


def _claude_parse(r: dict[str, Any]) -> Reply:
    text = "".join(b.get("text", "") for b in r["content"] if b["type"] == "text")
    return Reply(text, [(b["id"], b["name"], b["input"]) for b in r["content"] if b["type"] == "tool_use"], r.get("stop_reason"))


def _responses_input(messages: list[dict[str, Any]]) -> list[dict[str, Any]]:
    out: list[dict[str, Any]] = []
    for m in messages:
        if m["role"] == "tool":
            out.append({"type": "function_call_output", "call_id": m["tool_call_id"], "output": m.get("content", "")})
            continue
        if m.get("content"):
            out.append({"role": m["role"], "content": m["content"]})
        for c in m.get("tool_calls") or []:
            out.append({"type": "function_call", "call_id": c["id"], "name": c["function"]["name"], "arguments": c["function"]["arguments"]})
    return out


def _responses_request(model: str, messages: list[dict[str, Any]], tools: list[dict[str, Any]]) -> tuple[str, dict[str, Any]]:
    return "/v1/responses", {"model": model, "input": _responses_input(messages), "temperature": 0.0, "max_output_tokens": 1024,
                             "tools": [{"type": "function", "name": t["function"]["name"], "description": t["function"].get("description", ""),
                                        "parameters": t["function"]["parameters"]} for t in tools]}


def _responses_parse(r: dict[str, Any]) -> Reply:
    text, calls = "", []
    for it in r["output"]:
        if it["type"] == "function_call":
            calls.append((it.get("call_id") or it.get("id", ""), it["name"], it["arguments"]))
        elif it["type"] == "message":
            text += "".join(p.get("text", "") for p in it.get("content", []) if p.get("type") in ("output_text", "text"))
    return Reply(text, calls, r.get("status"))


# the follow-up history is kept in the chat form for every dialect; each dialect's request builder translates it
DIALECTS = {"chat": (_chat_request, _chat_parse), "claude": (_claude_request, _claude_parse), "responses": (_responses_request, _responses_parse)}


def run_scenario(c: ExoClient, model: str, sc: Scenario, dialect: str) -> dict[str, Any]:
    """One scenario in one dialect: the first reply is scored against the expectation; with a ``tool_result`` and a correct
    call, the result goes back and the second reply must be text without another call."""
    build, parse = DIALECTS[dialect]
    row: dict[str, Any] = {"scenario": sc.name, "dialect": dialect, "prompt": sc.prompt}
    try:
        reply = parse(c.post(*build(model, sc.messages, sc.tools)))
    except (ApiError, KeyError, TypeError) as e:
        return {**row, "passed": False, "error": f"{type(e).__name__}: {e}"}
    if not sc.expect_call:
        row.update(called=bool(reply.calls), passed=not reply.calls and bool(reply.text.strip()))
        return row
    name, args = (reply.calls[0][1], reply.calls[0][2]) if reply.calls else (None, None)
    row.update(score_call(name, args, sc))
    row["passed"] = all(row[k] for k in ("called", "name_ok", "json_ok", "args_ok"))
    if row["passed"] and sc.tool_result is not None:
        result = sc.tool_result if isinstance(sc.tool_result, str) else json.dumps(sc.tool_result)
        try:
            second = parse(c.post(*build(model, _chat_followup(sc.messages, reply, result), sc.tools)))
            row["followup_ok"] = not second.calls and bool(second.text.strip())
        except (ApiError, KeyError, TypeError) as e:
            row.update(followup_ok=False, error=f"{type(e).__name__}: {e}")
        row["passed"] = row["passed"] and row["followup_ok"]
    return row


def summarize(rows: list[dict[str, Any]]) -> dict[str, Any]:
    by: dict[str, list[int]] = {}
    for r in rows:
        t = by.setdefault(r["dialect"], [0, 0])
        t[0] += bool(r["passed"])
        t[1] += 1
    return {"passed": sum(bool(r["passed"]) for r in rows), "total": len(rows), "by_dialect": {d: {"passed": p, "total": n} for d, (p, n) in by.items()}}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--scenarios", default=None, help="TOML ([tools.*] + [[scenarios]]) or JSONL file; adds to the built-in list")
    ap.add_argument("--only", default=None, help="comma-separated scenario names")
    ap.add_argument("--dialects", default="chat,claude,responses")
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--out", default=None, help="write the full result as JSON to this file")
    a = ap.parse_args(argv)
    scenarios = list(BUILTIN) + (load_scenarios(Path(a.scenarios)) if a.scenarios else [])
    if a.only:
        scenarios = [s for s in scenarios if s.name in a.only.split(",")]
    c = ExoClient(a.host, a.port)
    c.wait_ready(a.model, timeout=60)
    rows = [run_scenario(c, a.model, sc, d) for _ in range(a.repeat) for sc in scenarios for d in a.dialects.split(",")]
    result = {"model": a.model, **summarize(rows), "rows": rows}
    if a.out:
        Path(a.out).write_text(json.dumps(result, indent=1))
    print(json.dumps(result))
    return 0 if result["passed"] == result["total"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
