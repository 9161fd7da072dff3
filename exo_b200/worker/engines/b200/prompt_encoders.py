"""Prompt encoders for the DeepSeek checkpoints whose chat format is code, not a Jinja template.

DeepSeek-V3.2 and DeepSeek-V4 ship no ``chat_template``: the publisher's repository carries a Python encoder, and the
reference vendors both (``src/exo/worker/engines/mlx/vendor/dsml_encoding.py``,
``src/exo/worker/engines/mlx/vendor/deepseek_v4_encoding.py``) and selects them by model id
(``src/exo/worker/engines/mlx/utils_mlx.py:485-600``).  Here one encoder class serves both; what differs between the
two formats is data (`Dialect`):

=====================  ==============================================  ===========================================
                       V3.2                                            V4
=====================  ==============================================  ===========================================
tool-call block        ``<｜DSML｜function_calls>``                     ``<｜DSML｜tool_calls>``
tool results           ``<function_results><result>…</result>…`` in    ``<tool_result>…</tool_result>`` blocks
                       a turn of their own after the assistant turn    merged into the next user turn, ordered as
                                                                       the calls were
tools in the prompt    appended to the system text                     carried by the system / developer message
reasoning effort       —                                               ``max`` adds a fixed preamble
extra roles            —                                               ``developer``, ``latest_reminder``, tasks
=====================  ==============================================  ===========================================

Common to both: ``<｜begin▁of▁sentence｜>`` once, ``<｜User｜>`` / ``<｜Assistant｜>`` turn markers, an assistant
turn is ``reasoning</think>content[tool calls]<｜end▁of▁sentence｜>``, the generation prompt ends in ``<think>``
(thinking mode) or ``</think>`` (chat mode), and reasoning of turns before the last user message is dropped unless the
conversation uses tools.  The literal instruction text of the tools section is part of the format the models were
trained on and is kept as published.

The same class parses a completion back into ``content`` / ``reasoning_content`` / ``tool_calls``.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Any

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
USER, ASSISTANT, REMINDER = "<｜User｜>", "<｜Assistant｜>", "<｜latest_reminder｜>"
TASK_TOKENS = {t: f"<｜{t}｜>" for t in ("action", "query", "authority", "domain", "title", "read_url")}

MAX_EFFORT_PREAMBLE = (
    "Reasoning Effort: Absolute maximum with no shortcuts permitted.\n"
    "You MUST be very thorough in your thinking and comprehensively decompose the problem to resolve the root cause, "
    "rigorously stress-testing your logic against all potential paths, edge cases, and adversarial scenarios.\n"
    "Explicitly write out your entire deliberation process, documenting every intermediate step, considered "
    "alternative, and rejected hypothesis to ensure absolutely no assumption is left unchecked.\n\n")

_INVOKE_EXAMPLE = (
    '<{d}{block}>\n<{d}invoke name="$TOOL_NAME">\n'
    '<{d}parameter name="$PARAMETER_NAME" string="true|false">$PARAMETER_VALUE</{d}parameter>\n...\n</{d}invoke>\n'
    '<{d}invoke name="$TOOL_NAME2">\n...\n</{d}invoke>\n</{d}{block}>')

_TOOLS_V4 = (
    "## Tools\n\nYou have access to a set of tools to help answer the user's question. You can invoke tools by writing a "
    '"<{d}{block}>" block like the following:\n\n' + _INVOKE_EXAMPLE + "\n\n"
    'String parameters should be specified as is and set `string="true"`. For all other types (numbers, booleans, '
    'arrays, objects), pass the value in JSON format and set `string="false"`.\n\n'
    "If thinking_mode is enabled (triggered by {to}), you MUST output your complete reasoning inside {to}...{tc} BEFORE "
    "any tool calls or final response.\n\nOtherwise, output directly after {tc} with tool calls or final response.\n\n"
    "### Available Tool Schemas\n\n{schemas}\n\n"
    "You MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n")

_TOOLS_V32 = (
    "## Tools\nYou have access to a set of tools you can use to answer the user's question.\n"
    'You can invoke functions by writing a "<{d}{block}>" block like the following as part of your reply to the user:\n'
    + _INVOKE_EXAMPLE.replace("$TOOL_NAME", "$FUNCTION_NAME") + "\n\n"
    "String and scalar parameters should be specified as is without any escaping or quotes, while lists and objects "
    'should use JSON format. The "string" attribute should be set to "true" for string type parameters and "false" for '
    "other types (numbers, booleans, arrays, objects).\n\n"
    "If the thinking_mode is enabled, then after function results you should strongly consider outputting a thinking "
    "block. Here is an example:\n\n"
    "<{d}{block}>\n...\n</{d}{block}>\n\n<function_results>\n...\n</function_results>\n\n"
    "{to}...thinking about results{tc}\n\n"
    "Here are the functions available in JSONSchema format:\n<functions>\n{schemas}\n</functions>\n")

_RESPONSE_FORMAT = "## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n{schema}"


@dataclass(frozen=True)
class Dialect:
    name: str
    call_block: str                 # element name of the block that holds the invokes
    tools_text: str
    results_in_user_turn: bool      # V4: tool results ride in the next user turn; V3.2: a block after the assistant turn
    effort_preamble: bool
    extra_roles: bool
    omit_empty_think: bool          # V3.2: a turn without reasoning carries no think markers at all


V32 = Dialect("deepseek-v3.2", "function_calls", _TOOLS_V32, False, False, False, True)
V4 = Dialect("deepseek-v4", "tool_calls", _TOOLS_V4, True, True, True, False)


def _dumps(v: Any) -> str:
    return json.dumps(v, ensure_ascii=False)


def _functions(tools: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """OpenAI tool entries (``{"type": "function", "function": {...}}``) or bare function schemas → bare schemas."""
    return [t["function"] if isinstance(t, dict) and "function" in t else t for t in tools]


def _call_pairs(tool_calls: list[dict[str, Any]]) -> list[tuple[str, Any]]:
    out = []
    for tc in tool_calls:
        fn = tc.get("function", tc)
        out.append((fn.get("name", ""), fn.get("arguments", "{}")))
    return out


def _text_of(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for b in content:
        if isinstance(b, dict):
            parts.append(b.get("text", "") if b.get("type", "text") == "text" else f"[Unsupported {b.get('type')}]")
        else:
            parts.append(str(b))
    return "\n\n".join(parts)


class DeepSeekPromptEncoder:
    def __init__(self, dialect: Dialect):
        self.d = dialect
        self.block_open = f"<{DSML}{dialect.call_block}>"
        self.block_close = f"</{DSML}{dialect.call_block}>"

    # ------------------------------------------------------------------ encoding
    def tools_section(self, tools: list[dict[str, Any]]) -> str:
        return self.d.tools_text.format(d=DSML, block=self.d.call_block, to=THINK_OPEN, tc=THINK_CLOSE,
                                        schemas="\n".join(_dumps(f) for f in _functions(tools)))

    def encode_call(self, name: str, arguments: Any) -> str:
        if isinstance(arguments, str):
            try:
                arguments = json.loads(arguments)
            except ValueError:
                arguments = {"arguments": arguments}
        if not isinstance(arguments, dict):
            arguments = {"arguments": arguments}
        params = "\n".join(
            f'<{DSML}parameter name="{k}" string="{"true" if isinstance(v, str) else "false"}">'
            f'{v if isinstance(v, str) else _dumps(v)}</{DSML}parameter>' for k, v in arguments.items())
        return f'<{DSML}invoke name="{name}">\n{params}\n</{DSML}invoke>'

    def encode_calls(self, tool_calls: list[dict[str, Any]]) -> str:
        body = "\n".join(self.encode_call(n, a) for n, a in _call_pairs(tool_calls))
        return f"\n\n{self.block_open}\n{body}\n{self.block_close}"

    def _fold_tool_turns(self, messages: list[dict[str, Any]]) -> list[dict[str, Any]]:
        """``role: tool`` messages become part of a user-side turn: a list of results, in the order of the calls."""
        out: list[dict[str, Any]] = []
        order: dict[str, int] = {}
        for m in messages:
            m = dict(m)
            role = m.get("role")
            if role == "assistant" and m.get("tool_calls"):
                order = {tc.get("id", ""): i for i, tc in enumerate(m["tool_calls"]) if tc.get("id")}
            if role == "tool":
                res = {"id": m.get("tool_call_id", ""), "content": _text_of(m.get("content"))}
                if out and out[-1].get("role") == "user" and "results" in out[-1] and not out[-1].get("text_after"):
                    out[-1]["results"].append(res)
                else:
                    out.append({"role": "user", "results": [res], "content": ""})
                out[-1]["results"].sort(key=lambda r: order.get(r["id"], 0))
                continue
            if role == "user" and self.d.results_in_user_turn and out and out[-1].get("role") == "user" \
                    and "results" in out[-1] and out[-1].get("task") is None:
                out[-1]["text_after"] = (out[-1].get("text_after") or []) + [_text_of(m.get("content"))]
                continue
            out.append(m)
        return out

    def _user_turn(self, m: dict[str, Any]) -> str:
        if "results" not in m:
            return USER + _text_of(m.get("content"))
        if self.d.results_in_user_turn:
            parts = [f"<tool_result>{r['content']}</tool_result>" for r in m["results"]] + list(m.get("text_after") or [])
            return USER + "\n\n".join(parts)
        body = "\n".join(f"<result>{r['content']}</result>" for r in m["results"])
        return f"\n\n<function_results>\n{body}\n</function_results>"

    def encode(self, messages: list[dict[str, Any]], thinking: bool = True, tools: list[dict[str, Any]] | None = None,
               reasoning_effort: str | None = None, add_bos: bool = True, drop_thinking: bool = True) -> str:
        msgs = [dict(m) for m in messages]
        if tools:
            for m in msgs:
                if m.get("role") in ("system", "developer") if self.d.extra_roles else m.get("role") == "system":
                    m["tools"] = tools
                    break
            else:
                msgs.insert(0, {"role": "system", "content": "", "tools": tools})
        uses_tools = any(m.get("tools") for m in msgs)
        keep_reasoning = not drop_thinking or uses_tools      # tool chains stay coherent only with their reasoning
        msgs = self._fold_tool_turns(msgs)
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") in ("user", "developer")), default=-1)
        if thinking and not keep_reasoning:
            kept = []
            for i, m in enumerate(msgs):
                if i >= last_user or m.get("role") in ("user", "system", "latest_reminder"):
                    kept.append(m)
                elif m.get("role") == "assistant":
                    kept.append({k: v for k, v in m.items() if k != "reasoning_content"})
            msgs = kept
            last_user = max((i for i, m in enumerate(msgs) if m.get("role") in ("user", "developer")), default=-1)
        out = [BOS if add_bos else ""]
        if self.d.effort_preamble and thinking and reasoning_effort == "max":
            out.append(MAX_EFFORT_PREAMBLE)
        for i, m in enumerate(msgs):
            role = m.get("role")
            if role in ("system", "developer"):
                if role == "developer" and not self.d.extra_roles:
                    role = "system"
                text = (USER if role == "developer" else "") + _text_of(m.get("content"))
                if m.get("tools"):
                    text += "\n\n" + self.tools_section(m["tools"])
                if m.get("response_format"):
                    text += "\n\n" + _RESPONSE_FORMAT.format(schema=_dumps(m["response_format"]))
                out.append(text)
            elif role == "user":
                out.append(self._user_turn(m))
            elif role == "latest_reminder" and self.d.extra_roles:
                out.append(REMINDER + _text_of(m.get("content")))
            elif role == "assistant":
                after_task = i > 0 and msgs[i - 1].get("task") is not None
                turn = ""
                if thinking and not after_task and (keep_reasoning or i > last_user):
                    turn += (m.get("reasoning_content") or "") + THINK_CLOSE
                turn += _text_of(m.get("content"))
                if m.get("tool_calls"):
                    turn += self.encode_calls(m["tool_calls"])
                out.append(turn + ("" if m.get("wo_eos") else EOS))
            else:
                raise ValueError(f"unknown role for {self.d.name}: {role!r}")
            nxt = msgs[i + 1].get("role") if i + 1 < len(msgs) else None
            if nxt is not None and nxt not in ("assistant", "latest_reminder"):
                continue
            task = m.get("task")
            if task is not None and self.d.extra_roles:
                if task not in TASK_TOKENS:
                    raise ValueError(f"invalid task {task!r}")
                out.append(TASK_TOKENS[task] if task != "action"
                           else ASSISTANT + (THINK_OPEN if thinking else THINK_CLOSE) + TASK_TOKENS[task])
            elif role in ("user", "developer"):
                opens = thinking and (keep_reasoning or i >= last_user)
                if "results" in m and not self.d.results_in_user_turn:
                    # the assistant's own turn goes on after the results: no new turn marker
                    out.append("\n\n" + THINK_OPEN if opens else "")
                else:
                    out.append(ASSISTANT + (THINK_OPEN if opens else THINK_CLOSE))
        text = "".join(out)
        if self.d.omit_empty_think:
            text = text.replace(ASSISTANT + THINK_CLOSE, ASSISTANT)
            for empty in (THINK_OPEN + "\n\n" + THINK_CLOSE, THINK_OPEN + "\n" + THINK_CLOSE, THINK_OPEN + THINK_CLOSE):
                text = text.replace(empty, "")
        return text

    # ------------------------------------------------------------------ parsing
    _PARAM = re.compile(rf'<{re.escape(DSML)}parameter\s+name="([^"]+)"\s+string="(true|false)">(.*?)</{re.escape(DSML)}parameter>',
                        re.DOTALL)
    _INVOKE = re.compile(rf'<{re.escape(DSML)}invoke\s+name="([^"]+)">(.*?)</{re.escape(DSML)}invoke>', re.DOTALL)

    def parse_calls(self, text: str) -> list[dict[str, Any]]:
        """Every ``invoke`` of a call block → OpenAI-style tool calls (arguments as a JSON string)."""
        calls = []
        for name, body in self._INVOKE.findall(text):
            args: dict[str, Any] = {}
            for key, is_str, val in self._PARAM.findall(body):
                if key in args:
                    raise ValueError(f"duplicate parameter {key!r} in call of {name!r}")
                if is_str == "true":
                    args[key] = val
                else:
                    try:
                        args[key] = json.loads(val)
                    except ValueError:
                        args[key] = val
            calls.append({"type": "function", "function": {"name": name, "arguments": _dumps(args)}})
        return calls

    def parse_completion(self, text: str, thinking: bool = True) -> dict[str, Any]:
        """One generated assistant turn → ``{"role", "content", "reasoning_content", "tool_calls"}``."""
        if text.endswith(EOS):
            text = text[:-len(EOS)]
        reasoning = ""
        if thinking:
            head, sep, rest = text.partition(THINK_CLOSE)
            if not sep:
                raise ValueError("thinking-mode completion without </think>")
            reasoning, text = head.removeprefix(THINK_OPEN), rest
        start = text.find("\n\n" + self.block_open)
        calls: list[dict[str, Any]] = []
        if start >= 0:
            end = text.find(self.block_close, start)
            if end < 0:
                raise ValueError("unterminated tool-call block")
            if text[end + len(self.block_close):].strip():
                raise ValueError("text after the tool-call block")
            calls = self.parse_calls(text[start:end])
            text = text[:start]
        for tok in (BOS, EOS, THINK_OPEN, THINK_CLOSE, DSML):
            if tok in text or tok in reasoning:
                raise ValueError(f"special token {tok!r} inside content")
        return {"role": "assistant", "content": text, "reasoning_content": reasoning, "tool_calls": calls}


def encoder_for(model_id: str) -> DeepSeekPromptEncoder | None:
    """The code-defined chat format of a model, or ``None`` when the checkpoint's Jinja template is the format."""
    m = model_id.lower()
    if "deepseek-v4" in m:
        return DeepSeekPromptEncoder(V4)
    if "deepseek-v3.2" in m:
        return DeepSeekPromptEncoder(V32)
    return None


def strip_think_blocks(content: str) -> str:
    """Earlier assistant turns handed back by a client may still carry ``<think>…</think>``: the encoder writes the
    reasoning itself, so the markers go."""
    if not content:
        return content
    return re.sub(r"<think>.*?</think>", "", content, flags=re.DOTALL).replace(THINK_OPEN, "").replace(THINK_CLOSE, "")
