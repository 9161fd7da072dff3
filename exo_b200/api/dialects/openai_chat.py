"""OpenAI Chat Completions dialect (``/v1/chat/completions``).

Wire behaviour of the reference adapter (``src/exo/api/adapters/chat_completions.py:60-383``):
system messages become ``instructions`` (joined by newlines) and stay in the template messages;
image parts are pulled out into ``images`` and replaced by ``{"type": "image"}`` placeholders;
streaming sends one ``chat.completion`` object per token with ``delta`` (``reasoning_content``
for thinking), usage on the finishing chunk, prefill progress and generation stats as SSE
comments, an error object then ``[DONE]`` on failure, and always ``data: [DONE]`` last.
"""
from __future__ import annotations

import time
from collections.abc import Iterable
from typing import Any

from ...shared.messages import InputMessage, TextGenerationTaskParams, resolve_reasoning_params
from ...shared.wire import PrefillProgressChunk, TokenChunk, ToolCallChunk
from ..types import (BenchChatCompletionResponse, ChatCompletionChoice, ChatCompletionMessage,
                     ChatCompletionMessageImageUrl, ChatCompletionMessageText, ChatCompletionRequest,
                     ChatCompletionResponse, ErrorInfo, ErrorResponse, Logprobs, LogprobsContentItem, PowerUsage,
                     StreamingChoiceResponse, ToolCall)
from .common import Turn, image_from_url, sse, sse_comment


async def to_params(req: ChatCompletionRequest) -> TextGenerationTaskParams:
    system: list[str] = []
    inputs: list[InputMessage] = []
    template: list[dict[str, Any]] = []
    images: list[str] = []
    for msg in req.messages:
        parts = ([] if msg.content is None else [ChatCompletionMessageText(text=msg.content)] if isinstance(msg.content, str)
                 else [msg.content] if not isinstance(msg.content, list) else list(msg.content))
        texts, placeholders, n_img = [], [], 0
        for p in parts:
            if isinstance(p, ChatCompletionMessageImageUrl):
                img = await image_from_url(p.image_url.get("url", ""))
                if img is not None:
                    images.append(img)
                    n_img += 1
                    placeholders.append({"type": "image"})
            else:
                texts.append(p.text)
                placeholders.append({"type": "text", "text": p.text})
        content = "\n".join(texts)
        if msg.role == "system":
            system.append(content)
            template.append({"role": "system", "content": content})
            continue
        if msg.content is None and msg.reasoning_content is None and msg.tool_calls is None:
            continue
        if msg.role in ("user", "assistant", "developer"):
            inputs.append(InputMessage(role=msg.role, content=content))
        if n_img:
            m: dict[str, Any] = {"role": msg.role, "content": placeholders}
            if msg.reasoning_content is not None:
                m["reasoning_content"] = msg.reasoning_content
            template.append(m)
        else:
            template.append(msg.model_copy(update={"content": content}).model_dump(exclude_none=True))
    effort, thinking = resolve_reasoning_params(req.reasoning_effort, req.enable_thinking)
    return TextGenerationTaskParams(
        model=req.model, input=inputs or [InputMessage(role="user", content="")], instructions="\n".join(system) if system else None,
        max_output_tokens=req.max_completion_tokens if req.max_tokens is None else req.max_tokens, temperature=req.temperature,
        top_p=req.top_p, top_k=req.top_k, stop=req.stop, seed=req.seed, stream=req.stream, tools=req.tools,
        reasoning_effort=effort, enable_thinking=thinking, chat_template_messages=template or None,
        logprobs=req.logprobs or False, top_logprobs=req.top_logprobs, min_p=req.min_p,
        repetition_penalty=req.repetition_penalty, repetition_context_size=req.repetition_context_size,
        presence_penalty=req.presence_penalty, frequency_penalty=req.frequency_penalty, images=images)


def _tool_calls(items) -> list[ToolCall]:
    return [ToolCall(id=t.id, index=i, function=t) for i, t in enumerate(items)]


class ChatStreamEncoder:
    def _obj(self, turn: Turn, delta: ChatCompletionMessage, finish: str | None, logprobs: Logprobs | None = None) -> str:
        r = ChatCompletionResponse(id=turn.command_id, created=int(time.time()), model=turn.model,
                                   choices=[StreamingChoiceResponse(index=0, delta=delta, logprobs=logprobs, finish_reason=finish)],
                                   usage=turn.usage if finish else None)
        return sse(r.model_dump_json(exclude_none=True))

    def open(self, turn: Turn) -> Iterable[str]:
        return ()

    def _token(self, turn: Turn, chunk: TokenChunk, delta: ChatCompletionMessage) -> Iterable[str]:
        lp = None
        if chunk.logprob is not None:
            lp = Logprobs(content=[LogprobsContentItem(token=chunk.text, logprob=chunk.logprob, top_logprobs=chunk.top_logprobs or [])])
        yield self._obj(turn, delta, chunk.finish_reason, lp)

    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        return self._token(turn, chunk, ChatCompletionMessage(role="assistant", reasoning_content=chunk.text))

    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]:
        return self._token(turn, chunk, ChatCompletionMessage(role="assistant", content=chunk.text))

    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]:
        yield self._obj(turn, ChatCompletionMessage(role="assistant", tool_calls=_tool_calls(chunk.tool_calls)), "tool_calls")

    def progress(self, chunk: PrefillProgressChunk) -> Iterable[str]:
        yield sse_comment("prefill_progress", chunk.model_dump_json())

    def error(self, turn: Turn, message: str) -> Iterable[str]:
        err = ErrorResponse(error=ErrorInfo(message=message, type="InternalServerError", code=500))
        yield sse(err.model_dump_json(exclude_none=True))
        yield sse("[DONE]")

    def close(self, turn: Turn) -> Iterable[str]:
        if turn.stats is not None:
            yield sse_comment("generation_stats", turn.stats.model_dump_json())
        yield sse("[DONE]")


def _message(turn: Turn) -> ChatCompletionMessage:
    return ChatCompletionMessage(role="assistant", content=turn.content, reasoning_content=turn.thinking or None,
                                 tool_calls=_tool_calls(turn.tool_calls) or None)


def render(turn: Turn) -> str:
    return ChatCompletionResponse(
        id=turn.command_id, created=int(time.time()), model=turn.model, usage=turn.usage,
        choices=[ChatCompletionChoice(index=0, message=_message(turn), finish_reason=turn.finish_reason,
                                      logprobs=Logprobs(content=turn.logprobs) if turn.logprobs else None)],
    ).model_dump_json(exclude_none=True)


def render_bench(turn: Turn, power: PowerUsage | None) -> BenchChatCompletionResponse:
    return BenchChatCompletionResponse(
        id=turn.command_id, created=int(time.time()), model=turn.model, usage=turn.usage,
        choices=[ChatCompletionChoice(index=0, message=_message(turn), finish_reason=turn.finish_reason)],
        generation_stats=turn.stats, power_usage=power)
