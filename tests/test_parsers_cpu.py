"""Streaming thinking / tool-call parsers, with markers split across arbitrary token boundaries."""
import json

import pytest

from exo_b200.worker.engines.b200.parsers import (DSML, TOOL_DIALECTS, coerce_arguments, parse_glm_block,
                                                  parse_json_block, parse_kimi_block, tool_dialect_for)
from exo_b200.worker.engines.b200.stream_parser import HarmonyParser, StreamParser


def run(parser, text, step):
    pieces = []
    for i in range(0, len(text), step):
        pieces += parser.feed(text[i:i + step])
    pieces += parser.finish()
    merged = []
    for p in pieces:
        if merged and merged[-1][0] == p.kind and p.kind != "tool_calls":
            merged[-1] = (p.kind, merged[-1][1] + p.text)
        else:
            merged.append((p.kind, p.text if p.kind != "tool_calls" else p.tool_calls))
    return merged


@pytest.mark.parametrize("step", [1, 2, 3, 7, 1000])
def test_thinking_then_text_then_tool_call(step):
    text = '<think>let me think</think>Answer: 4<tool_call>{"name": "add", "arguments": {"a": 1, "b": 3}}</tool_call>'
    got = run(StreamParser(tool=TOOL_DIALECTS["json"]), text, step)
    assert got[0] == ("thinking", "let me think") and got[1] == ("text", "Answer: 4")
    assert got[2][0] == "tool_calls" and got[2][1][0].name == "add" and json.loads(got[2][1][0].arguments) == {"a": 1, "b": 3}


@pytest.mark.parametrize("step", [1, 4, 1000])
def test_starts_in_thinking_and_angle_brackets_in_text(step):
    got = run(StreamParser(starts_in_thinking=True), "reasoning a<b</think>x < y and <thin air>", step)
    assert got == [("thinking", "reasoning a<b"), ("text", "x < y and <thin air>")]


def test_malformed_tool_block_comes_back_as_error_text():
    got = run(StreamParser(tool=TOOL_DIALECTS["json"]), "ok<tool_call>{broken</tool_call>", 5)
    assert got[0] == ("text", "ok") and got[1][0] == "error" and "{broken" in got[1][1]


def test_block_parsers_and_coercion():
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"properties": {
        "n": {"type": "integer"}, "x": {"type": "number"}, "b": {"type": "boolean"}, "o": {"type": "object"}, "s": {"type": "string"}}}}}]
    assert coerce_arguments("f", {"n": "3", "x": "2.5", "b": "true", "o": '{"k": 1}', "s": "7"}, tools) == \
        {"n": 3, "x": 2.5, "b": True, "o": {"k": 1}, "s": "7"}
    xml = "<function=f>\n<parameter=n>\n3\n</parameter>\n<parameter=s>\nhi\n</parameter>\n</function>"
    calls = TOOL_DIALECTS["xml_function"].parse(xml, tools)
    assert calls[0].name == "f" and json.loads(calls[0].arguments) == {"n": 3, "s": "hi"}
    g = parse_glm_block("f\n<arg_key>n</arg_key>\n<arg_value>5</arg_value>", tools)
    assert json.loads(g[0].arguments) == {"n": 5}
    k = parse_kimi_block('<|tool_call_begin|>functions.f:0<|tool_call_argument_begin|>{"n": 1}<|tool_call_end|>')
    assert k[0].name == "f" and k[0].id == "functions.f:0"
    two = parse_json_block('{"name": "a", "arguments": {}}\n{"name": "b", "arguments": {"q": 1}}')
    assert [c.name for c in two] == ["a", "b"]
    body = f'<{DSML}invoke name="f"><{DSML}parameter name="s" string="true">hi</{DSML}parameter><{DSML}parameter name="n" string="false">3</{DSML}parameter></{DSML}invoke>'
    d = TOOL_DIALECTS["dsml"].parse(body, None)
    assert json.loads(d[0].arguments) == {"s": "hi", "n": 3}
    assert tool_dialect_for("kimi").start.startswith("<|tool_calls_section")
    assert tool_dialect_for("qwen", "Qwen/Qwen3-Coder-480B").parse is TOOL_DIALECTS["xml_function"].parse


@pytest.mark.parametrize("step", [1, 5, 1000])
def test_dsml_streaming_with_partial_markers(step):
    d = TOOL_DIALECTS["dsml"]
    text = f'I will call.{d.start}<{DSML}invoke name="get"><{DSML}parameter name="city" string="true">Paris</{DSML}parameter></{DSML}invoke>{d.end}'
    got = run(StreamParser(tool=d), text, step)
    assert got[0] == ("text", "I will call.") and got[1][1][0].name == "get"


@pytest.mark.parametrize("step", [1, 6, 1000])
def test_harmony_channels(step):
    text = ('<|channel|>analysis<|message|>thinking hard<|end|><|start|>assistant<|channel|>commentary to=functions.lookup '
            '<|constrain|>json<|message|>{"q": "x"}<|call|><|start|>assistant<|channel|>final<|message|>Done.<|return|>')
    got = run(HarmonyParser(), text, step)
    assert ("thinking", "thinking hard") in got and ("text", "Done.") in got
    calls = [g for g in got if g[0] == "tool_calls"][0][1]
    assert calls[0].name == "lookup" and json.loads(calls[0].arguments) == {"q": "x"}
