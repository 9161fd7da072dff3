"""OpenAI Responses dialect (``/v1/responses``).

Conversion rules of the reference adapter (``src/exo/api/adapters/responses.py:133-395``): string
input is one user message; list input is walked item by item: messages (text and image parts),
every flavour of tool *call* item (function, MCP, custom, shell, computer, apply-patch, built-in
searches) becomes an assistant ``tool_calls`` entry, consecutive calls merging into one assistant
message, every flavour of tool *output* item becomes a ``tool`` message, reasoning items become
assistant text, compaction summaries and MCP tool lists become system text; tools given flat are
wrapped into function tools.  Items are handled here as plain dicts keyed by ``type`` so an
unknown item type is skipped instead of failing validation.  Streaming follows the Responses
event grammar with monotonically increasing ``sequence_number``: ``response.created``,
``response.in_progress``, then per output item ``output_item.added`` … ``output_item.done``
(reasoning summary, message text, function calls), and ``response.completed``.
"""
from __future__ import annotations

import json
import time
from collections.abc import Iterable
from typing import Any, Literal

from pydantic import BaseModel, Field

from ...shared.messages import InputMessage, TextGenerationTaskParams, resolve_reasoning_params
from ...shared.wire import PrefillProgressChunk, TokenChunk, ToolCallChunk
from ..types import ReasoningEffort
from .common import Turn, image_from_url, openai_tool, sse


class Reasoning(BaseModel):
    effort: ReasoningEffort | None = None
    summary: str | None = None


class ResponsesRequest(BaseModel):
    model: str
    input: str | list[dict[str, Any]]
    instructions: str | None = None
    max_output_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    stop: str | list[str] | None = None
    seed: int | None = None
    stream: bool = False
    tools: list[dict[str, Any]] | None = None
    reasoning: Reasoning | None = None
    enable_thinking: bool | None = None
    chat_template_messages: list[dict[str, Any]] | None = None
    metadata: dict[str, Any] | None = None
    previous_response_id: str | None = None
    store: bool | None = None


CALLS_WITH_NAME = {"function_call", "mcp_call", "custom_tool_call", "mcp_approval_request"}
CALLS_WITH_ACTION = {"local_shell_call", "shell_call", "computer_call"}
BUILTIN_CALL_ARG = {"web_search_call": "query", "file_search_call": "queries", "code_interpreter_call": "code",
                    "image_generation_call": "prompt", "tool_search_call": "query"}
OUTPUTS = {"function_call_output", "local_shell_call_output", "shell_call_output", "apply_patch_call_output",
           "computer_call_output", "custom_tool_call_output", "tool_search_output"}


def _text_of(content: Any) -> str:
    if isinstance(content, str):
        return content
    return "".join(p.get("text", "") for p in content or [] if isinstance(p, dict) and "text" in p)


def _add_call(template: list[dict[str, Any]], call_id: str, name: str, arguments: str) -> None:
    call = {"id": call_id, "type": "function", "function": {"name": name, "arguments": arguments}}
    if template and template[-1].get("role") == "assistant" and "tool_calls" in template[-1]:
        template[-1]["tool_calls"].append(call)
    else:
        template.append({"role": "assistant", "content": "", "tool_calls": [call]})


async def to_params(req: ResponsesRequest) -> TextGenerationTaskParams:
    images: list[str] = []
    template: list[dict[str, Any]] | None = None
    if isinstance(req.input, str):
        inputs = [InputMessage(role="user", content=req.input)]
    else:
        inputs, template = [], []
        if req.instructions is not None:
            template.append({"role": "system", "content": req.instructions})
        for item in req.input:
            kind = item.get("type") or ("message" if "role" in item else "")
            cid = item.get("call_id") or item.get("id") or ""
            if kind == "message":
                role, content = item.get("role", "user"), item.get("content", "")
                text = _text_of(content)
                placeholders, has_img = [], False
                for p in content if isinstance(content, list) else []:
                    if p.get("type") == "input_image" and p.get("image_url"):
                        img = await image_from_url(p["image_url"])
                        if img is not None:
                            images.append(img)
                            placeholders.append({"type": "image"})
                            has_img = True
                    elif "text" in p:
                        placeholders.append({"type": "text", "text": p["text"]})
                if role in ("user", "assistant", "developer"):
                    inputs.append(InputMessage(role=role, content=text))
                template.append({"role": role, "content": placeholders if has_img and role != "system" else text})
            elif kind in CALLS_WITH_NAME:
                _add_call(template, cid, item.get("name", ""), item.get("arguments") or item.get("input") or "{}")
            elif kind in CALLS_WITH_ACTION:
                _add_call(template, cid, kind, json.dumps(item.get("action", {})))
            elif kind == "apply_patch_call":
                _add_call(template, cid, "apply_patch", json.dumps({"patch": item.get("patch") or item.get("operation")}))
            elif kind in BUILTIN_CALL_ARG:
                k = BUILTIN_CALL_ARG[kind]
                _add_call(template, cid, kind, json.dumps({k: item.get(k)}))
            elif kind in OUTPUTS:
                out = item.get("output")
                template.append({"role": "tool", "tool_call_id": cid, "content": out if isinstance(out, str) else json.dumps(out)})
            elif kind == "mcp_approval_response":
                verdict = "Approved" if item.get("approve") else "Denied"
                reason = f": {item['reason']}" if item.get("reason") else ""
                template.append({"role": "tool", "tool_call_id": item.get("approval_request_id", ""), "content": verdict + reason})
            elif kind == "reasoning":
                text = _text_of(item.get("content")) or _text_of(item.get("summary"))
                if text:
                    template.append({"role": "assistant", "content": text})
            elif kind == "compaction":
                if item.get("summary"):
                    template.append({"role": "system", "content": item["summary"]})
            elif kind == "mcp_list_tools":
                names = ", ".join(t.get("name", "") for t in item.get("tools", []))
                if names:
                    template.append({"role": "system", "content": f"Available MCP tools ({item.get('server_label', '')}): {names}"})
            # item_reference and unknown kinds: nothing to resolve them against here
        inputs = inputs or [InputMessage(role="user", content="")]
    effort, thinking = resolve_reasoning_params(req.reasoning.effort if req.reasoning else None, req.enable_thinking)
    tools = None
    if req.tools:
        tools = [t if "function" in t else openai_tool(t.get("name", ""), t.get("description", ""), t.get("parameters", {}),
                                                      **({"strict": t["strict"]} if "strict" in t else {})) for t in req.tools]
    return TextGenerationTaskParams(
        model=req.model, input=inputs, instructions=req.instructions or None, max_output_tokens=req.max_output_tokens,
        temperature=req.temperature, top_p=req.top_p, top_k=req.top_k, stop=req.stop, seed=req.seed, stream=req.stream,
        tools=tools, chat_template_messages=template or req.chat_template_messages, reasoning_effort=effort,
        enable_thinking=thinking, images=images)


def _usage(turn: Turn) -> dict[str, Any] | None:
    if turn.usage is None:
        return None
    u = turn.usage
    return {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens, "total_tokens": u.total_tokens,
            "input_tokens_details": {"cached_tokens": u.prompt_tokens_details.cached_tokens},
            "output_tokens_details": {"reasoning_tokens": u.completion_tokens_details.reasoning_tokens}}


def _message_item(turn: Turn, status: str = "completed") -> dict[str, Any]:
    return {"type": "message", "id": f"item_{turn.command_id}", "role": "assistant", "status": status,
            "content": [{"type": "output_text", "text": turn.content, "annotations": []}]}


def _reasoning_item(turn: Turn) -> dict[str, Any]:
    return {"type": "reasoning", "id": f"rs_{turn.command_id}", "summary": [{"type": "summary_text", "text": turn.thinking}]}


def _call_item(t, status: str = "completed") -> dict[str, Any]:
    return {"type": "function_call", "id": t.id, "call_id": t.id, "name": t.name, "arguments": t.arguments, "status": status}


def _response(turn: Turn, status: Literal["in_progress", "completed", "failed"], output: list[dict[str, Any]]) -> dict[str, Any]:
    r = {"id": f"resp_{turn.command_id}", "object": "response", "created_at": int(time.time()), "status": status,
         "model": turn.model, "output": output}
    if status == "completed":
        r["output_text"] = turn.content
        if (u := _usage(turn)) is not None:
            r["usage"] = u
    return r


def _output(turn: Turn) -> list[dict[str, Any]]:
    out = [_reasoning_item(turn)] if turn.reasoning else []
    out.append(_message_item(turn))
    out.extend(_call_item(t) for t in turn.tool_calls)
    return out


class ResponsesStreamEncoder:
    def __init__(self) -> None:
        self.seq = 0
        self.n_items = 0
        self.reasoning_index: int | None = None
        self.reasoning_open = False
        self.message_index: int | None = None

    def _ev(self, name: str, **body: Any) -> str:
        self.seq += 1
        return sse(json.dumps({"type": name, "sequence_number": self.seq, **body}, ensure_ascii=False), event=name)

    def _take_index(self) -> int:
        self.n_items += 1
        return self.n_items - 1

    def open(self, turn: Turn) -> Iterable[str]:
        yield self._ev("response.created", response=_response(turn, "in_progress", []))
        yield self._ev("response.in_progress", response=_response(turn, "in_progress", []))

    def progress(self, chunk: PrefillProgressChunk) -> Iterable[str]:
        return ()

    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        rid = f"rs_{turn.command_id}"
        if self.reasoning_index is None:
            self.reasoning_index, self.reasoning_open = self._take_index(), True
            yield self._ev("response.output_item.added", output_index=self.reasoning_index,
                           item={"type": "reasoning", "id": rid, "summary": []})
            yield self._ev("response.reasoning_summary_part.added", item_id=rid, output_index=self.reasoning_index,
                           summary_index=0, part={"type": "summary_text", "text": ""})
        yield self._ev("response.reasoning_summary_text.delta", item_id=rid, output_index=self.reasoning_index,
                       summary_index=0, delta=chunk.text)

    def _end_reasoning(self, turn: Turn) -> Iterable[str]:
        if not self.reasoning_open:
            return
        self.reasoning_open = False
        rid, i = f"rs_{turn.command_id}", self.reasoning_index
        yield self._ev("response.reasoning_summary_text.done", item_id=rid, output_index=i, summary_index=0, text=turn.thinking)
        yield self._ev("response.reasoning_summary_part.done", item_id=rid, output_index=i, summary_index=0,
                       part={"type": "summary_text", "text": turn.thinking})
        yield self._ev("response.output_item.done", output_index=i, item=_reasoning_item(turn))

    def _begin_message(self, turn: Turn) -> Iterable[str]:
        if self.message_index is not None:
            return
        self.message_index = self._take_index()
        iid = f"item_{turn.command_id}"
        yield self._ev("response.output_item.added", output_index=self.message_index,
                       item={"type": "message", "id": iid, "role": "assistant", "status": "in_progress", "content": []})
        yield self._ev("response.content_part.added", item_id=iid, output_index=self.message_index, content_index=0,
                       part={"type": "output_text", "text": "", "annotations": []})

    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        yield from self._end_reasoning(turn)
        yield from self._begin_message(turn)
        yield self._ev("response.output_text.delta", item_id=f"item_{turn.command_id}", output_index=self.message_index,
                       content_index=0, delta=chunk.text)

    def _end_message(self, turn: Turn) -> Iterable[str]:
        yield from self._begin_message(turn)
        iid, i = f"item_{turn.command_id}", self.message_index
        yield self._ev("response.output_text.done", item_id=iid, output_index=i, content_index=0, text=turn.content)
        yield self._ev("response.content_part.done", item_id=iid, output_index=i, content_index=0,
                       part={"type": "output_text", "text": turn.content, "annotations": []})
        yield self._ev("response.output_item.done", output_index=i, item=_message_item(turn))

    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]:
        yield from self._end_reasoning(turn)
        yield from self._end_message(turn)
        self.message_done = True
        for t in chunk.tool_calls:
            i = self._take_index()
            yield self._ev("response.output_item.added", output_index=i, item={**_call_item(t, "in_progress"), "arguments": ""})
            yield self._ev("response.function_call_arguments.delta", item_id=t.id, output_index=i, delta=t.arguments)
            yield self._ev("response.function_call_arguments.done", item_id=t.id, output_index=i, name=t.name, arguments=t.arguments)
            yield self._ev("response.output_item.done", output_index=i, item=_call_item(t))

    message_done = False

    def error(self, turn: Turn, message: str) -> Iterable[str]:
        yield self._ev("response.failed", response={**_response(turn, "failed", []), "error": {"code": "server_error", "message": message}})

    def close(self, turn: Turn) -> Iterable[str]:
        yield from self._end_reasoning(turn)
        if not self.message_done:
            yield from self._end_message(turn)
        yield self._ev("response.completed", response=_response(turn, "completed", _output(turn)))


def render(turn: Turn) -> str:
    return json.dumps(_response(turn, "completed", _output(turn)), ensure_ascii=False)
