"""Anthropic Messages dialect (``/v1/messages``).

Behaviour matched to the reference adapter (``src/exo/api/adapters/claude.py:51-490``): ``system``
(string or text blocks) becomes the instructions, with volatile ``x-anthropic-…;`` header lines
removed because they change on every request and would defeat prefix caching; ``tool_use`` blocks
of an assistant turn become OpenAI-style ``tool_calls`` for the chat template and ``tool_result``
blocks become ``tool`` messages; tools are converted to function tools; ``thinking.type`` of
``enabled``/``adaptive`` switches reasoning on.  Streaming follows Anthropic's event grammar:
``message_start``, per content block ``content_block_start`` / ``_delta`` / ``_stop`` (thinking,
then text, then one block per tool call with a single ``input_json_delta``), ``message_delta``
carrying ``stop_reason`` and output tokens, ``message_stop``.
"""
from __future__ import annotations

import json
import re
from collections.abc import Iterable
from typing import Any, Literal

from pydantic import BaseModel, Field

from ...shared.messages import InputMessage, TextGenerationTaskParams
from ...shared.wire import PrefillProgressChunk, TokenChunk, ToolCallChunk
from .common import Turn, fetch_image_base64, openai_tool, sse

StopReason = Literal["end_turn", "max_tokens", "stop_sequence", "tool_use"]
STOP_REASON: dict[str, StopReason] = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use",
                                      "content_filter": "end_turn", "function_call": "tool_use"}


class TextBlock(BaseModel):
    type: Literal["text"] = "text"
    text: str


class ImageSource(BaseModel):
    type: Literal["base64", "url"]
    media_type: str | None = None
    data: str | None = None
    url: str | None = None


class ImageBlock(BaseModel):
    type: Literal["image"] = "image"
    source: ImageSource


class ThinkingBlock(BaseModel):
    type: Literal["thinking"] = "thinking"
    thinking: str
    signature: str | None = None


class ToolUseBlock(BaseModel):
    type: Literal["tool_use"] = "tool_use"
    id: str
    name: str
    input: dict[str, Any] = Field(default_factory=dict)


class ToolResultBlock(BaseModel):
    type: Literal["tool_result"] = "tool_result"
    tool_use_id: str
    content: str | list[TextBlock | ImageBlock] | None = None
    is_error: bool | None = None


ContentBlock = TextBlock | ImageBlock | ThinkingBlock | ToolUseBlock | ToolResultBlock


class Message(BaseModel):
    role: Literal["user", "assistant"]
    content: str | list[ContentBlock]


class ToolDef(BaseModel):
    name: str
    description: str | None = None
    input_schema: dict[str, Any] = Field(default_factory=dict)


class ThinkingConfig(BaseModel):
    type: Literal["enabled", "disabled", "adaptive"]
    budget_tokens: int | None = None


class MessagesRequest(BaseModel):
    model: str
    max_tokens: int
    messages: list[Message]
    system: str | list[TextBlock] | None = None
    stop_sequences: list[str] | None = None
    stream: bool = False
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    tools: list[ToolDef] | None = None
    tool_choice: dict[str, Any] | None = None
    thinking: ThinkingConfig | None = None
    metadata: dict[str, Any] | None = None


class ClaudeUsage(BaseModel):
    input_tokens: int = 0
    output_tokens: int = 0


class MessagesResponse(BaseModel):
    id: str
    type: Literal["message"] = "message"
    role: Literal["assistant"] = "assistant"
    model: str
    content: list[TextBlock | ThinkingBlock | ToolUseBlock]
    stop_reason: StopReason | None = None
    stop_sequence: str | None = None
    usage: ClaudeUsage = Field(default_factory=ClaudeUsage)


_VOLATILE = re.compile(r"^x-anthropic-[^\n]*;\n?", re.M)


def strip_volatile_headers(text: str) -> str:
    return _VOLATILE.sub("", text)


async def _image(b: ImageBlock) -> str | None:
    if b.source.type == "base64" and b.source.data:
        return b.source.data
    if b.source.type == "url" and b.source.url:
        try:
            return await fetch_image_base64(b.source.url)
        except Exception:  # noqa: BLE001 - an unreachable image is dropped, the request goes on
            return None
    return None


def _tool_result_text(b: ToolResultBlock) -> str:
    if b.content is None:
        return ""
    return b.content if isinstance(b.content, str) else "".join(s.text for s in b.content if isinstance(s, TextBlock))


async def to_params(req: MessagesRequest) -> TextGenerationTaskParams:
    template: list[dict[str, Any]] = []
    inputs: list[InputMessage] = []
    images: list[str] = []
    instructions = None
    if req.system:
        instructions = strip_volatile_headers(req.system if isinstance(req.system, str) else "".join(b.text for b in req.system))
        template.append({"role": "system", "content": instructions})
    for msg in req.messages:
        if isinstance(msg.content, str):
            inputs.append(InputMessage(role=msg.role, content=msg.content))
            template.append({"role": msg.role, "content": msg.content})
            continue
        texts, thoughts, calls, results, placeholders = [], [], [], [], []
        for b in msg.content:
            if isinstance(b, TextBlock):
                texts.append(b.text)
                placeholders.append({"type": "text", "text": b.text})
            elif isinstance(b, ImageBlock):
                if (img := await _image(b)) is not None:
                    images.append(img)
                    placeholders.append({"type": "image"})
            elif isinstance(b, ThinkingBlock):
                thoughts.append(b.thinking)
            elif isinstance(b, ToolUseBlock):
                calls.append({"id": b.id, "type": "function", "function": {"name": b.name, "arguments": json.dumps(b.input)}})
            else:
                results.append(b)
                for sub in (b.content if isinstance(b.content, list) else []):
                    if isinstance(sub, ImageBlock) and (img := await _image(sub)) is not None:
                        images.append(img)
        content = "".join(texts)
        inputs.append(InputMessage(role=msg.role, content=content))
        extra = {"reasoning_content": "".join(thoughts)} if thoughts else {}
        if calls:
            template.append({"role": "assistant", "content": content, "tool_calls": calls, **extra})
        elif results:
            template.extend({"role": "tool", "tool_call_id": r.tool_use_id, "content": _tool_result_text(r)} for r in results)
        elif any(p["type"] == "image" for p in placeholders):
            template.append({"role": msg.role, "content": placeholders, **extra})
        else:
            template.append({"role": msg.role, "content": content, **extra})
    tools = [openai_tool(t.name, t.description or "", t.input_schema) for t in req.tools] if req.tools else None
    thinking = None if req.thinking is None else req.thinking.type in ("enabled", "adaptive")
    return TextGenerationTaskParams(
        model=req.model, input=inputs or [InputMessage(role="user", content="")], instructions=instructions or None,
        max_output_tokens=req.max_tokens, temperature=req.temperature, top_p=req.top_p, top_k=req.top_k,
        stop=req.stop_sequences, stream=req.stream, tools=tools, enable_thinking=thinking,
        chat_template_messages=template or None, images=images)


def _tool_block(t) -> ToolUseBlock:
    try:
        args = json.loads(t.arguments)
    except json.JSONDecodeError:
        args = {"_raw": t.arguments}
    return ToolUseBlock(id=f"toolu_{t.id}", name=t.name, input=args if isinstance(args, dict) else {"value": args})


class ClaudeStreamEncoder:
    def __init__(self) -> None:
        self.next_index = 0
        self.open_kind: str | None = None      # "thinking" | "text"
        self.open_index = -1
        self.any_block = False

    def _ev(self, name: str, **body: Any) -> str:
        return sse(json.dumps({"type": name, **body}, ensure_ascii=False), event=name)

    def open(self, turn: Turn) -> Iterable[str]:
        msg = MessagesResponse(id=f"msg_{turn.command_id}", model=turn.model, content=[], stop_reason=None)
        yield self._ev("message_start", message=msg.model_dump())

    def _close_open(self) -> Iterable[str]:
        if self.open_kind is not None:
            yield self._ev("content_block_stop", index=self.open_index)
            self.open_kind = None

    def _ensure(self, kind: str) -> Iterable[str]:
        if self.open_kind == kind:
            return
        yield from self._close_open()
        self.open_kind, self.open_index, self.any_block = kind, self.next_index, True
        self.next_index += 1
        block = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
        yield self._ev("content_block_start", index=self.open_index, content_block=block)

    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        yield from self._ensure("thinking")
        yield self._ev("content_block_delta", index=self.open_index, delta={"type": "thinking_delta", "thinking": chunk.text})

    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        yield from self._ensure("text")
        yield self._ev("content_block_delta", index=self.open_index, delta={"type": "text_delta", "text": chunk.text})

    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]:
        yield from self._close_open()
        for t in chunk.tool_calls:
            i, self.next_index, self.any_block = self.next_index, self.next_index + 1, True
            yield self._ev("content_block_start", index=i, content_block={"type": "tool_use", "id": f"toolu_{t.id}", "name": t.name, "input": {}})
            yield self._ev("content_block_delta", index=i, delta={"type": "input_json_delta", "partial_json": t.arguments})
            yield self._ev("content_block_stop", index=i)

    def progress(self, chunk: PrefillProgressChunk) -> Iterable[str]:
        return ()

    def error(self, turn: Turn, message: str) -> Iterable[str]:
        yield from self._close_open()
        yield self._ev("error", error={"type": "api_error", "message": message})

    def close(self, turn: Turn) -> Iterable[str]:
        yield from self._close_open()
        if not self.any_block:
            yield self._ev("content_block_start", index=0, content_block={"type": "text", "text": ""})
            yield self._ev("content_block_stop", index=0)
        yield self._ev("message_delta", delta={"stop_reason": STOP_REASON.get(turn.finish_reason or "", "end_turn"), "stop_sequence": None},
                       usage={"output_tokens": turn.completion_tokens})
        yield self._ev("message_stop")


def render(turn: Turn) -> str:
    content: list[Any] = []
    if turn.thinking:
        content.append(ThinkingBlock(thinking=turn.thinking))
    if turn.content:
        content.append(TextBlock(text=turn.content))
    content.extend(_tool_block(t) for t in turn.tool_calls)
    if not content:
        content.append(TextBlock(text=""))
    return MessagesResponse(id=f"msg_{turn.command_id}", model=turn.model, content=content,
                            stop_reason=STOP_REASON.get(turn.finish_reason or "", "end_turn"),
                            usage=ClaudeUsage(input_tokens=turn.prompt_tokens, output_tokens=turn.completion_tokens)).model_dump_json()
