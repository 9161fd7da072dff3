"""Streaming output parsers: thinking sections and tool calls, for every supported dialect.

The reference chains generator stages per request (``src/exo/worker/runner/llm_inference/
model_output_parsers.py:67-492``: thinking-tag router, generic tool-call extractor, GPT-OSS
Harmony channels, DeepSeek DSML blocks with partial-marker buffering; ``tool_parsers.py:26-244``:
per-family call syntaxes and schema-driven argument coercion).  Here one character-level state
machine per request does the routing: text is scanned for the active markers, a tail that could
still grow into a marker is held back, and completed tool blocks are handed to the family's block
parser.  Markers split across tokens therefore need no special casing.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Callable

from ....api.types import ToolCallItem


@dataclass
class Piece:
    kind: str                      # "text" | "thinking" | "tool_calls" | "error"
    text: str = ""
    tool_calls: list[ToolCallItem] = field(default_factory=list)


# ------------------------------------------------------------------------------------------------
# argument coercion against the tool's JSON schema
# ------------------------------------------------------------------------------------------------
def _schema_for(tools: list[dict[str, Any]] | None, name: str) -> dict[str, Any]:
    for t in tools or []:
        fn = t.get("function", t)
        if fn.get("name") == name:
            return (fn.get("parameters") or {}).get("properties") or {}
    return {}


def coerce_value(v: Any, schema: dict[str, Any] | None) -> Any:
    """Turn a string taken from model text into the JSON type the schema asks for."""
    if not isinstance(v, str) or not schema:
        return v
    ty = schema.get("type")
    if isinstance(ty, list):
        ty = next((t for t in ty if t != "null"), None)
    s = v.strip()
    try:
        if ty == "integer":
            return int(s)
        if ty == "number":
            f = float(s)
            return int(f) if f.is_integer() and "." not in s and "e" not in s.lower() else f
        if ty == "boolean":
            if s.lower() in ("true", "1", "yes"):
                return True
            if s.lower() in ("false", "0", "no"):
                return False
        if ty in ("object", "array"):
            return json.loads(s)
        if ty == "null" and s.lower() in ("null", "none", ""):
            return None
    except (ValueError, json.JSONDecodeError):
        return v
    if ty is None:  # untyped: take JSON if it parses, else the raw string
        try:
            return json.loads(s)
        except (ValueError, json.JSONDecodeError):
            return v
    return v


def coerce_arguments(name: str, args: dict[str, Any], tools: list[dict[str, Any]] | None) -> dict[str, Any]:
    props = _schema_for(tools, name)
    return {k: coerce_value(v, props.get(k)) for k, v in args.items()}


def _item(name: str, args: Any) -> ToolCallItem:
    return ToolCallItem(name=name, arguments=args if isinstance(args, str) else json.dumps(args, ensure_ascii=False))


# ------------------------------------------------------------------------------------------------
# block parsers: text between the tool markers -> calls (None = unparseable)
# ------------------------------------------------------------------------------------------------
def parse_json_block(body: str, tools=None) -> list[ToolCallItem] | None:
    """Hermes / Qwen style: one JSON object (or several, or a list) with ``name`` and ``arguments``."""
    body = body.strip()
    objs: list[Any] = []
    dec = json.JSONDecoder()
    i = 0
    try:
        while i < len(body):
            while i < len(body) and body[i] in " \n\r\t,":
                i += 1
            if i >= len(body):
                break
            o, j = dec.raw_decode(body, i)
            objs.extend(o if isinstance(o, list) else [o])
            i = j
    except json.JSONDecodeError:
        return None
    out = []
    for o in objs:
        if not isinstance(o, dict) or "name" not in o:
            return None
        args = o.get("arguments", o.get("parameters", {}))
        if isinstance(args, str):
            try:
                args = json.loads(args)
            except json.JSONDecodeError:
                pass
        out.append(_item(str(o["name"]), args))
    return out or None


_XML_FN = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.S)
_XML_PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)


def parse_xml_function_block(body: str, tools=None) -> list[ToolCallItem] | None:
    """Qwen3-Coder style: ``<function=name><parameter=key>value</parameter>…</function>``."""
    out = []
    for name, inner in _XML_FN.findall(body):
        args = {k: v.strip("\n") for k, v in _XML_PARAM.findall(inner)}
        out.append(_item(name, coerce_arguments(name, args, tools)))
    return out or None


_GLM_KV = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)


def parse_glm_block(body: str, tools=None) -> list[ToolCallItem] | None:
    """GLM style: function name on the first line, then ``<arg_key>``/``<arg_value>`` pairs."""
    body = body.strip()
    if not body:
        return None
    name = re.split(r"[\n<]", body, 1)[0].strip()
    if not name:
        return None
    args = {k.strip(): v for k, v in _GLM_KV.findall(body)}
    return [_item(name, coerce_arguments(name, args, tools))]


_KIMI_CALL = re.compile(r"<\|tool_call_begin\|>\s*([^\s<]+?)\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", re.S)


def parse_kimi_block(body: str, tools=None) -> list[ToolCallItem] | None:
    """Kimi K2: ``<|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}<|tool_call_end|>``."""
    out = []
    for ident, args in _KIMI_CALL.findall(body):
        name = ident.split(".", 1)[-1].rsplit(":", 1)[0]
        try:
            parsed = json.loads(args)
        except json.JSONDecodeError:
            return None
        it = _item(name, parsed)
        out.append(it.model_copy(update={"id": ident}))
    return out or None


DSML = "｜DSML｜"   # ｜DSML｜
_DSML_INVOKE = re.compile(rf"<{DSML}invoke name=\"([^\"]+)\">(.*?)</{DSML}invoke>", re.S)
_DSML_PARAM = re.compile(rf"<{DSML}parameter name=\"([^\"]+)\"(?: string=\"(true|false)\")?>(.*?)</{DSML}parameter>", re.S)


def parse_dsml_block(body: str, tools=None) -> list[ToolCallItem] | None:
    """DeepSeek V3.2: ``<｜DSML｜invoke name=…>`` with ``<｜DSML｜parameter name=… string="true|false">``."""
    out = []
    for name, inner in _DSML_INVOKE.findall(body):
        args: dict[str, Any] = {}
        for k, is_str, v in _DSML_PARAM.findall(inner):
            if is_str == "true":
                args[k] = v
            else:
                try:
                    args[k] = json.loads(v)
                except json.JSONDecodeError:
                    args[k] = v
        out.append(_item(name, args))
    return out or None


@dataclass(frozen=True)
class ToolDialect:
    start: str
    end: str
    parse: Callable[[str, Any], list[ToolCallItem] | None]


TOOL_DIALECTS: dict[str, ToolDialect] = {
    "json": ToolDialect("<tool_call>", "</tool_call>", parse_json_block),
    "xml_function": ToolDialect("<tool_call>", "</tool_call>", parse_xml_function_block),
    "glm": ToolDialect("<tool_call>", "</tool_call>", parse_glm_block),
    "kimi": ToolDialect("<|tool_calls_section_begin|>", "<|tool_calls_section_end|>", parse_kimi_block),
    "dsml": ToolDialect(f"<{DSML}function_calls>", f"</{DSML}function_calls>", parse_dsml_block),
}


def tool_dialect_for(family: str, model_id: str = "") -> ToolDialect | None:
    m = model_id.lower()
    if "coder" in m and "qwen" in m:
        return TOOL_DIALECTS["xml_function"]
    if family in ("qwen", "llama", "mistral"):
        return TOOL_DIALECTS["json"]
    if family == "glm":
        return TOOL_DIALECTS["glm"]
    if family == "kimi":
        return TOOL_DIALECTS["kimi"]
    if family == "deepseek":
        return TOOL_DIALECTS["dsml"] if ("v3.2" in m or "v4" in m) else TOOL_DIALECTS["json"]
    return TOOL_DIALECTS["json"]
