"""Ollama dialect (``/ollama/api/chat``, ``/ollama/api/generate``, tags / show / ps / version).

Wire behaviour of the reference adapter (``src/exo/api/adapters/ollama.py:32-490``): options map to
sampling parameters (``num_predict`` → max tokens), ``think`` → reasoning switch, per-message
``images`` become image placeholders, ``tool`` messages get a ``tool_call_id`` from ``tool_name``
/ ``name`` / a running counter; responses are newline-delimited JSON objects, thinking deltas in
``message.thinking`` (chat) or ``thinking`` (generate), the final object carries ``done``,
``done_reason`` (``tool_call`` for tool calls) and the prompt/eval token counts; tool-call
arguments are sent as JSON objects when they parse.  ``/api/generate`` has no tool support: a
tool-call chunk simply ends the stream.
"""
from __future__ import annotations

import json
import time
from collections.abc import Iterable
from typing import Any, Literal

from pydantic import BaseModel, Field

from ...shared.messages import InputMessage, TextGenerationTaskParams
from ...shared.wire import PrefillProgressChunk, TokenChunk, ToolCallChunk
from .common import Turn

DoneReason = Literal["stop", "length", "tool_call", "error"]


def done_reason(finish: str | None) -> DoneReason | None:
    if finish is None:
        return None
    return {"stop": "stop", "length": "length", "tool_calls": "tool_call", "function_call": "tool_call", "error": "error"}.get(finish, "stop")


def _now() -> str:
    return time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())


class ToolFunction(BaseModel):
    name: str
    arguments: dict[str, Any] | str
    index: int | None = None


class OllamaToolCall(BaseModel):
    id: str | None = None
    type: Literal["function"] | None = None
    function: ToolFunction


class OllamaMessage(BaseModel):
    role: Literal["system", "user", "assistant", "tool"]
    content: str | None = None
    thinking: str | None = None
    tool_calls: list[OllamaToolCall] | None = None
    name: str | None = None
    tool_name: str | None = None
    images: list[str] | None = None


class Options(BaseModel):
    num_predict: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    stop: str | list[str] | None = None
    seed: int | None = None


class ChatRequest(BaseModel):
    model: str
    messages: list[OllamaMessage]
    stream: bool = True
    options: Options | None = None
    tools: list[dict[str, Any]] | None = None
    format: Literal["json"] | dict[str, Any] | None = None
    keep_alive: str | int | None = None
    think: bool | None = None


class GenerateRequest(BaseModel):
    model: str
    prompt: str = ""
    system: str | None = None
    stream: bool = True
    options: Options | None = None
    format: Literal["json"] | dict[str, Any] | None = None
    keep_alive: str | int | None = None
    think: bool | None = None
    raw: bool = False
    images: list[str] | None = None


class ShowRequest(BaseModel):
    name: str | None = None
    model: str | None = None
    verbose: bool | None = None


class ChatResponse(BaseModel):
    model: str
    created_at: str = Field(default_factory=_now)
    message: OllamaMessage
    done: bool
    done_reason: DoneReason | None = None
    prompt_eval_count: int | None = None
    eval_count: int | None = None


class GenerateResponse(BaseModel):
    model: str
    created_at: str = Field(default_factory=_now)
    response: str
    thinking: str | None = None
    done: bool
    done_reason: DoneReason | None = None
    prompt_eval_count: int | None = None
    eval_count: int | None = None


class ModelDetails(BaseModel):
    format: str | None = None
    family: str | None = None
    parameter_size: str | None = None
    quantization_level: str | None = None


class ModelTag(BaseModel):
    name: str
    model: str | None = None
    modified_at: str | None = None
    size: int | None = None
    digest: str | None = None
    details: ModelDetails | None = None


class TagsResponse(BaseModel):
    models: list[ModelTag]


class ShowResponse(BaseModel):
    modelfile: str | None = None
    parameters: str | None = None
    template: str | None = None
    details: ModelDetails | None = None
    model_info: dict[str, Any] | None = None
    capabilities: list[str] = []


class PsModel(BaseModel):
    name: str
    model: str
    size: int
    digest: str | None = None
    details: ModelDetails | None = None
    expires_at: str | None = None
    size_vram: int | None = None


class PsResponse(BaseModel):
    models: list[PsModel]


def _sampling(o: Options | None) -> dict[str, Any]:
    if o is None:
        return {}
    return dict(max_output_tokens=o.num_predict, temperature=o.temperature, top_p=o.top_p, top_k=o.top_k, stop=o.stop, seed=o.seed)


def chat_to_params(req: ChatRequest) -> TextGenerationTaskParams:
    system: list[str] = []
    inputs: list[InputMessage] = []
    template: list[dict[str, Any]] = []
    images: list[str] = []
    n_tool = 0
    for m in req.messages:
        content = m.content or ""
        if m.role == "system":
            system.append(content)
            template.append({"role": "system", "content": content})
            continue
        if m.role in ("user", "assistant") and (m.content is not None or m.thinking is not None or m.tool_calls or m.images):
            inputs.append(InputMessage(role=m.role, content=content))
        if m.images:
            images.extend(m.images)
            parts: list[dict[str, Any]] = [{"type": "image"} for _ in m.images]
            if content:
                parts.append({"type": "text", "text": content})
            template.append({"role": m.role, "content": parts})
            continue
        d: dict[str, Any] = {"role": m.role, "content": content}
        if m.thinking is not None:
            d["thinking"] = m.thinking
        if m.tool_calls is not None:
            d["tool_calls"] = [{
                **({"id": tc.id} if tc.id is not None else {}), **({"type": tc.type} if tc.type is not None else {}),
                "function": {"name": tc.function.name,
                             "arguments": json.dumps(tc.function.arguments) if isinstance(tc.function.arguments, dict) else tc.function.arguments,
                             **({"index": tc.function.index} if tc.function.index is not None else {})}} for tc in m.tool_calls]
        if m.name is not None:
            d["name"] = m.name
        if m.role == "tool":
            n_tool += 1
            d["tool_call_id"] = m.tool_name or m.name or f"tool_{n_tool}"
            if m.tool_name is not None:
                d["tool_name"] = m.tool_name
        template.append(d)
    return TextGenerationTaskParams(model=req.model, input=inputs or [InputMessage(role="user", content="")],
                                    instructions="\n".join(system) if system else None, stream=req.stream, tools=req.tools,
                                    enable_thinking=req.think, chat_template_messages=template or None, images=images,
                                    **_sampling(req.options))


def generate_to_params(req: GenerateRequest) -> TextGenerationTaskParams:
    template: list[dict[str, Any]] = []
    if req.system:
        template.append({"role": "system", "content": req.system})
    if req.images:
        parts: list[dict[str, Any]] = [{"type": "image"} for _ in req.images]
        if req.prompt:
            parts.append({"type": "text", "text": req.prompt})
        template.append({"role": "user", "content": parts})
    else:
        template.append({"role": "user", "content": req.prompt})
    return TextGenerationTaskParams(model=req.model, input=[InputMessage(role="user", content=req.prompt)],
                                    instructions=req.system or None, stream=req.stream, enable_thinking=req.think,
                                    chat_template_messages=template, images=list(req.images or []), **_sampling(req.options))


def _calls(items) -> list[OllamaToolCall]:
    out = []
    for i, t in enumerate(items):
        try:
            args: dict[str, Any] | str = json.loads(t.arguments)
            if not isinstance(args, dict):
                args = t.arguments
        except json.JSONDecodeError:
            args = t.arguments
        out.append(OllamaToolCall(id=t.id, type="function", function=ToolFunction(name=t.name, arguments=args, index=i)))
    return out


def _line(obj: BaseModel) -> str:
    return obj.model_dump_json(exclude_none=True) + "\n"


class OllamaChatEncoder:
    def __init__(self) -> None:
        self.done_sent = False      # a line with ``done: true`` has gone out

    def open(self, turn: Turn) -> Iterable[str]:
        return ()

    def progress(self, chunk: PrefillProgressChunk) -> Iterable[str]:
        return ()

    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        yield _line(ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content="", thinking=chunk.text), done=False))

    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        done = self.done_sent = chunk.finish_reason is not None
        yield _line(ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content=chunk.text), done=done,
                                 done_reason=done_reason(chunk.finish_reason),
                                 prompt_eval_count=turn.prompt_tokens if done else None,
                                 eval_count=turn.completion_tokens if done else None))

    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]:
        self.done_sent = True
        yield _line(ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content="", tool_calls=_calls(chunk.tool_calls),
                                                                         thinking=turn.thinking or None),
                                 done=True, done_reason="tool_call", prompt_eval_count=turn.prompt_tokens, eval_count=turn.completion_tokens))

    def error(self, turn: Turn, message: str) -> Iterable[str]:
        yield _line(ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content=message), done=True, done_reason="error"))

    def close(self, turn: Turn) -> Iterable[str]:
        if not self.done_sent:   # e.g. the turn ended inside the thinking section
            yield _line(ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content=""), done=True,
                                     done_reason=done_reason(turn.finish_reason) or "stop",
                                     prompt_eval_count=turn.prompt_tokens, eval_count=turn.completion_tokens))


class OllamaGenerateEncoder(OllamaChatEncoder):
    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        yield _line(GenerateResponse(model=turn.model, response="", thinking=chunk.text, done=False))

    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        done = self.done_sent = chunk.finish_reason is not None
        yield _line(GenerateResponse(model=turn.model, response=chunk.text, done=done, done_reason=done_reason(chunk.finish_reason),
                                     prompt_eval_count=turn.prompt_tokens if done else None,
                                     eval_count=turn.completion_tokens if done else None))

    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]:
        self.done_sent = True
        yield _line(GenerateResponse(model=turn.model, response="", done=True, done_reason="stop",
                                     prompt_eval_count=turn.prompt_tokens, eval_count=turn.completion_tokens))

    def error(self, turn: Turn, message: str) -> Iterable[str]:
        yield _line(GenerateResponse(model=turn.model, response="", done=True, done_reason="error"))

    def close(self, turn: Turn) -> Iterable[str]:
        if not self.done_sent:
            yield _line(GenerateResponse(model=turn.model, response="", done=True, done_reason=done_reason(turn.finish_reason) or "stop",
                                         prompt_eval_count=turn.prompt_tokens, eval_count=turn.completion_tokens))


def render_chat(turn: Turn) -> str:
    return ChatResponse(model=turn.model, message=OllamaMessage(role="assistant", content=turn.content, thinking=turn.thinking or None,
                                                                tool_calls=_calls(turn.tool_calls) or None),
                        done=True, done_reason=done_reason(turn.finish_reason) or "stop", prompt_eval_count=turn.prompt_tokens,
                        eval_count=turn.completion_tokens).model_dump_json(exclude_none=True)


def render_generate(turn: Turn) -> str:
    reason = "stop" if turn.tool_calls else (done_reason(turn.finish_reason) or "stop")
    return GenerateResponse(model=turn.model, response=turn.content, thinking=turn.thinking or None, done=True, done_reason=reason,
                            prompt_eval_count=turn.prompt_tokens, eval_count=turn.completion_tokens).model_dump_json(exclude_none=True)
