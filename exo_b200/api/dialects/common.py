"""What every API dialect shares: the turn accumulator, the encoder protocol and SSE plumbing.

The reference writes each dialect as a pair of free-standing generators over the chunk stream
(``src/exo/api/adapters/{chat_completions,claude,responses,ollama}.py``).  Here the chunk protocol
is consumed once, by :func:`drive`: it folds chunks into a :class:`Turn` (text, reasoning, tool
calls, usage, stats, log-probs, finish reason) and tells a dialect's *encoder* what happened
(``open`` / ``reasoning`` / ``text`` / ``tool_calls`` / ``progress`` / ``error`` / ``close``).  A
dialect is then a request converter plus one small encoder class for streaming and one
``render`` function for the non-streaming body, and all four dialects agree by construction on
ordering, error handling and end-of-stream.
"""
from __future__ import annotations

import base64
import re
from collections.abc import AsyncIterator, Iterable
from contextlib import aclosing
from dataclasses import dataclass, field
from typing import Any, Protocol

import anyio

from ...shared.base import CommandId
from ...shared.wire import ErrorChunk, PrefillProgressChunk, TokenChunk, ToolCallChunk
from ..types import GenerationStats, LogprobsContentItem, ToolCallItem, Usage

TextChunk = TokenChunk | ToolCallChunk | ErrorChunk | PrefillProgressChunk
SSE_HEADERS = {"Cache-Control": "no-cache", "Connection": "close", "X-Accel-Buffering": "no"}
KEEPALIVE_S = 15.0


class GenerationError(Exception):
    """The runner reported an error for this command."""


@dataclass
class Turn:
    """Everything one assistant turn produced so far."""
    command_id: CommandId
    model: str = ""
    text: list[str] = field(default_factory=list)
    reasoning: list[str] = field(default_factory=list)
    tool_calls: list[ToolCallItem] = field(default_factory=list)
    logprobs: list[LogprobsContentItem] = field(default_factory=list)
    usage: Usage | None = None
    stats: GenerationStats | None = None
    finish_reason: str | None = None
    n_token_chunks: int = 0

    @property
    def content(self) -> str:
        return "".join(self.text)

    @property
    def thinking(self) -> str:
        return "".join(self.reasoning)

    @property
    def prompt_tokens(self) -> int:
        return self.usage.prompt_tokens if self.usage else (self.stats.prompt_tokens if self.stats else 0)

    @property
    def completion_tokens(self) -> int:
        return self.usage.completion_tokens if self.usage else (self.stats.generation_tokens if self.stats else self.n_token_chunks)


class Encoder(Protocol):
    """Streaming side of a dialect; every method returns the wire strings to send now."""
    def open(self, turn: Turn) -> Iterable[str]: ...
    def reasoning(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]: ...
    def text(self, turn: Turn, chunk: TokenChunk) -> Iterable[str]: ...
    def tool_calls(self, turn: Turn, chunk: ToolCallChunk) -> Iterable[str]: ...
    def progress(self, chunk: PrefillProgressChunk) -> Iterable[str]: ...
    def error(self, turn: Turn, message: str) -> Iterable[str]: ...
    def close(self, turn: Turn) -> Iterable[str]: ...


def fold(turn: Turn, chunk: TokenChunk | ToolCallChunk) -> None:
    turn.model = turn.model or str(chunk.model)
    turn.usage = chunk.usage or turn.usage
    turn.stats = chunk.stats or turn.stats
    if isinstance(chunk, ToolCallChunk):
        turn.tool_calls.extend(chunk.tool_calls)
        turn.finish_reason = "tool_calls"
        return
    turn.n_token_chunks += 1
    (turn.reasoning if chunk.is_thinking else turn.text).append(chunk.text)
    if chunk.logprob is not None:
        turn.logprobs.append(LogprobsContentItem(token=chunk.text, logprob=chunk.logprob, top_logprobs=chunk.top_logprobs or []))
    if chunk.finish_reason is not None:
        turn.finish_reason = chunk.finish_reason


async def drive(command_id: CommandId, chunks: AsyncIterator[TextChunk], enc: Encoder, model: str = "") -> AsyncIterator[str]:
    """Chunk stream → wire strings of one dialect.  Ends after the first finishing chunk."""
    turn = Turn(command_id, model=model)
    for s in enc.open(turn):
        yield s
    async with aclosing(chunks):      # the producer's cleanup (TaskFinished) must run now, not at garbage collection
        async for chunk in chunks:
            if isinstance(chunk, PrefillProgressChunk):
                for s in enc.progress(chunk):
                    yield s
                continue
            if isinstance(chunk, ErrorChunk):
                turn.finish_reason = "error"
                for s in enc.error(turn, chunk.error_message or "Internal server error"):
                    yield s
                return
            fold(turn, chunk)
            if isinstance(chunk, ToolCallChunk):
                out = enc.tool_calls(turn, chunk)
            elif chunk.is_thinking:
                out = enc.reasoning(turn, chunk)
            else:
                out = enc.text(turn, chunk)
            for s in out:
                yield s
            if turn.finish_reason is not None:
                break
    for s in enc.close(turn):
        yield s


async def collect(command_id: CommandId, chunks: AsyncIterator[TextChunk], model: str = "") -> Turn:
    """Chunk stream → the finished turn; raises :class:`GenerationError` on an error chunk."""
    turn = Turn(command_id, model=model)
    async with aclosing(chunks):
        async for chunk in chunks:
            if isinstance(chunk, PrefillProgressChunk):
                continue
            if isinstance(chunk, ErrorChunk):
                raise GenerationError(chunk.error_message or "Internal server error")
            fold(turn, chunk)
            if turn.finish_reason is not None:
                break
    return turn


def sse(data: str, event: str | None = None) -> str:
    return (f"event: {event}\n" if event else "") + f"data: {data}\n\n"


def sse_comment(name: str, data: str) -> str:
    """SSE comment line: clients that do not know it ignore it."""
    return f": {name} {data}\n\n"


async def with_sse_keepalive(stream: AsyncIterator[str], interval: float = KEEPALIVE_S) -> AsyncIterator[str]:
    """Interleave ``: keepalive`` comments while the producer is silent (long prefills), so proxies
    and clients keep the connection open (same purpose as ``src/exo/api/main.py`` ``with_sse_keepalive``)."""
    send, recv = anyio.create_memory_object_stream[str | None](16)

    async def pump() -> None:
        try:
            async for item in stream:
                await send.send(item)
        finally:
            with anyio.CancelScope(shield=True):
                await send.send(None)

    async with anyio.create_task_group() as tg:
        tg.start_soon(pump)
        try:
            while True:
                item: str | None = ""
                with anyio.move_on_after(interval) as scope:
                    item = await recv.receive()
                if scope.cancelled_caught:
                    yield ": keepalive\n\n"
                    continue
                if item is None:
                    return
                yield item
        finally:
            tg.cancel_scope.cancel()


# ---- images in requests -------------------------------------------------------------------------
_DATA_URL = re.compile(r"data:[^;]+;base64,(.+)", re.S)


def base64_from_data_url(url: str) -> str:
    m = _DATA_URL.match(url)
    return m.group(1) if m else url


async def fetch_image_base64(url: str) -> str:
    import aiohttp
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=30)) as s, s.get(url, headers={"User-Agent": "exo/1.0"}) as r:
        r.raise_for_status()
        return base64.b64encode(await r.read()).decode("ascii")


async def image_from_url(url: str) -> str | None:
    if not url:
        return None
    if url.startswith(("http://", "https://")):
        return await fetch_image_base64(url)
    return base64_from_data_url(url)


def openai_tool(name: str, description: str, parameters: dict[str, Any], **extra: Any) -> dict[str, Any]:
    return {"type": "function", "function": {"name": name, "description": description, "parameters": parameters, **extra}}
