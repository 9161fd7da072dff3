"""The per-request streaming state machine that routes model text into text / thinking / tool
calls (see ``parsers.py`` for the dialects).  ``HarmonyParser`` handles GPT-OSS channel markup.
"""
from __future__ import annotations

import json
import re
from typing import Any

from ....api.types import ToolCallItem
from .parsers import Piece, ToolDialect


def _held_back(buf: str, markers: list[str]) -> int:
    """Length of the longest tail of ``buf`` that is a proper prefix of some marker."""
    best = 0
    for m in markers:
        for n in range(min(len(m) - 1, len(buf)), 0, -1):
            if buf.endswith(m[:n]):
                best = max(best, n)
                break
    return best


class StreamParser:
    def __init__(self, think_start: str | None = "<think>", think_end: str | None = "</think>",
                 starts_in_thinking: bool = False, tool: ToolDialect | None = None,
                 tools: list[dict[str, Any]] | None = None):
        self.ts, self.te = think_start, think_end
        self.mode = "thinking" if (starts_in_thinking and think_end) else "normal"
        self.tool, self.tools = tool, tools
        self.buf = ""
        self.tool_body = ""
        self.calls: list[ToolCallItem] = []
        self.reasoning_chars = 0

    def _emit(self, out: list[Piece], kind: str, text: str) -> None:
        if not text:
            return
        if kind == "thinking":
            self.reasoning_chars += len(text)
        if out and out[-1].kind == kind:
            out[-1].text += text
        else:
            out.append(Piece(kind, text))

    def feed(self, text: str) -> list[Piece]:
        self.buf += text
        out: list[Piece] = []
        while True:
            if self.mode == "tool":
                assert self.tool is not None
                i = self.buf.find(self.tool.end)
                if i < 0:
                    keep = _held_back(self.buf, [self.tool.end])
                    self.tool_body += self.buf[:len(self.buf) - keep]
                    self.buf = self.buf[len(self.buf) - keep:]
                    return out
                self.tool_body += self.buf[:i]
                self.buf = self.buf[i + len(self.tool.end):]
                parsed = self.tool.parse(self.tool_body, self.tools)
                if parsed is None:
                    out.append(Piece("error", self.tool.start + self.tool_body + self.tool.end))
                else:
                    self.calls.extend(parsed)
                self.tool_body = ""
                self.mode = "normal"
                continue
            if self.mode == "thinking":
                markers = [self.te] if self.te else []
            else:
                markers = [m for m in (self.ts, self.tool.start if self.tool else None) if m]
                if self.te:
                    markers.append(self.te)   # a stray end tag is swallowed
            hits = [(self.buf.find(m), m) for m in markers if self.buf.find(m) >= 0]
            kind = "thinking" if self.mode == "thinking" else "text"
            if not hits:
                keep = _held_back(self.buf, markers)
                self._emit(out, kind, self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                return out
            i, m = min(hits)
            self._emit(out, kind, self.buf[:i])
            self.buf = self.buf[i + len(m):]
            if self.mode == "thinking":
                self.mode = "normal"
            elif m == self.ts:
                self.mode = "thinking"
            elif self.tool is not None and m == self.tool.start:
                self.mode = "tool"
            # stray think_end in normal mode: dropped

    def finish(self) -> list[Piece]:
        """Flush at end of generation: held-back text is emitted; an unterminated tool block
        comes back as plain text; collected calls are returned as one ``tool_calls`` piece."""
        out: list[Piece] = []
        if self.mode == "tool" and self.tool is not None:
            body = self.tool_body + self.buf
            parsed = self.tool.parse(body, self.tools)
            if parsed:
                self.calls.extend(parsed)
            else:
                out.append(Piece("error", self.tool.start + body))
        elif self.buf:
            self._emit(out, "thinking" if self.mode == "thinking" else "text", self.buf)
        self.buf, self.tool_body = "", ""
        if self.calls:
            out.append(Piece("tool_calls", tool_calls=list(self.calls)))
            self.calls = []
        return out


_HARMONY_HDR = re.compile(r"<\|channel\|>(\w+)([^<]*?)(?:<\|constrain\|>(\w+))?<\|message\|>", re.S)


class HarmonyParser:
    """GPT-OSS Harmony: ``<|channel|>analysis|final|commentary … <|message|>body<|end|/<|call|/<|return|>``.

    analysis → thinking, final → text, ``commentary to=functions.NAME`` → a tool call whose body is
    the JSON arguments.  Text before any channel header is treated as final text.
    """
    ENDS = ("<|end|>", "<|call|>", "<|return|>")

    def __init__(self, tools: list[dict[str, Any]] | None = None):
        self.buf = ""
        self.channel: str | None = None
        self.recipient: str | None = None
        self.body = ""
        self.calls: list[ToolCallItem] = []
        self.reasoning_chars = 0
        self.skip_role = False

    def _kind(self) -> str:
        return "thinking" if self.channel == "analysis" else "text"

    def feed(self, text: str) -> list[Piece]:
        self.buf += text
        out: list[Piece] = []
        while True:
            if self.channel is None:
                if self.skip_role:   # the role name after <|start|> is not content
                    i = self.buf.find("<|")
                    if i < 0:
                        keep = _held_back(self.buf, ["<|"])
                        self.buf = self.buf[len(self.buf) - keep:]
                        return out
                    self.buf, self.skip_role = self.buf[i:], False
                    continue
                i = self.buf.find("<|")
                if i < 0:
                    keep = _held_back(self.buf, ["<|"])
                    if self.buf[:len(self.buf) - keep]:
                        out.append(Piece("text", self.buf[:len(self.buf) - keep]))
                    self.buf = self.buf[len(self.buf) - keep:]
                    return out
                if i > 0:
                    out.append(Piece("text", self.buf[:i]))
                    self.buf = self.buf[i:]
                j = self.buf.find("|>")
                if j < 0:
                    return out                      # marker still incomplete
                marker = self.buf[:j + 2]
                if marker == "<|start|>":
                    self.buf, self.skip_role = self.buf[j + 2:], True
                    continue
                if marker != "<|channel|>":
                    self.buf = self.buf[j + 2:]     # stray control marker outside a channel
                    continue
                m = _HARMONY_HDR.match(self.buf)
                if m is None:
                    return out                      # header not complete yet (<|message|> pending)
                self.channel = m.group(1)
                rec = re.search(r"to=([\w.\-]+)", m.group(2) or "")
                self.recipient = rec.group(1) if rec else None
                self.buf = self.buf[m.end():]
                continue
            ends = [(self.buf.find(e), e) for e in self.ENDS if self.buf.find(e) >= 0]
            if not ends:
                keep = _held_back(self.buf, list(self.ENDS))
                chunk, self.buf = self.buf[:len(self.buf) - keep], self.buf[len(self.buf) - keep:]
                if self.recipient:
                    self.body += chunk
                elif chunk:
                    if self._kind() == "thinking":
                        self.reasoning_chars += len(chunk)
                    out.append(Piece(self._kind(), chunk))
                return out
            i, e = min(ends)
            chunk, self.buf = self.buf[:i], self.buf[i + len(e):]
            if self.recipient:
                self.body += chunk
                name = self.recipient.split(".", 1)[-1]
                self.calls.append(ToolCallItem(name=name, arguments=self.body.strip() or "{}"))
                self.body = ""
            elif chunk:
                if self._kind() == "thinking":
                    self.reasoning_chars += len(chunk)
                out.append(Piece(self._kind(), chunk))
            self.channel, self.recipient = None, None

    def finish(self) -> list[Piece]:
        out: list[Piece] = []
        if self.channel is not None and not self.recipient and self.buf:
            out.append(Piece(self._kind(), self.buf))
        elif self.channel is not None and self.recipient:
            name = self.recipient.split(".", 1)[-1]
            self.calls.append(ToolCallItem(name=name, arguments=(self.body + self.buf).strip() or "{}"))
        elif self.buf and not self.buf.startswith("<|"):
            out.append(Piece("text", self.buf))
        self.buf = ""
        if self.calls:
            out.append(Piece("tool_calls", tool_calls=list(self.calls)))
            self.calls = []
        return out
