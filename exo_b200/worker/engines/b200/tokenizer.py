"""Tokenizers, incremental detokenisation and chat-template rendering.

A checkpoint directory with tokenizer files is loaded through ``transformers``; one without
(random-init benchmark models, tests) gets a byte-level tokenizer.  Chat rendering follows the
reference's ``render_chat_template`` (``src/exo/worker/engines/mlx/utils_mlx.py:515-655``): the
request's ``chat_template_messages`` win over ``instructions`` + ``input``, consecutive system
messages are merged into the first, ``enable_thinking`` / ``reasoning_effort`` are passed to the
template, a trailing assistant message is continued rather than closed.
"""
from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Any

from ....shared.messages import TextGenerationTaskParams
from .prompt_encoders import encoder_for, strip_think_blocks

# Stop tokens of families whose tokenizer config does not name all of them (turn markers that end a reply); keyed by
# a substring of the lower-cased model id, first match wins (``src/exo/worker/engines/mlx/utils_mlx.py:296-332``).
KNOWN_EOS_IDS: tuple[tuple[tuple[str, ...], tuple[int, ...]], ...] = (
    (("kimi-k2",), (163586,)),
    (("glm-5",), (154820, 154827, 154829)),
    (("glm",), (151336, 151329, 151338)),
    (("gpt-oss",), (200002, 200012)),
    (("qwen3.5", "qwen-3.5", "qwen3.6", "qwen-3.6"), (248046, 248044)),
    (("gemma-4", "gemma-3"), (1, 106, 50)),
)


def known_eos_ids(model_id: str) -> tuple[int, ...]:
    m = model_id.lower()
    for keys, ids in KNOWN_EOS_IDS:
        if any(k in m for k in keys):
            return ids
    return ()


class ByteTokenizer:
    """UTF-8 bytes as tokens 0..255, ``<bos>``=256, ``<eos>``=257 (vocab must be ≥ 258)."""
    bos_token_id, eos_token_id = 256, 257
    chat_template = None
    name_or_path = "byte"

    def __init__(self, vocab_size: int = 258):
        self.vocab_size = vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", "replace")

    @property
    def eos_token_ids(self) -> list[int]:
        return [self.eos_token_id]


def load_tokenizer(model_dir: Path | None, vocab_size: int):
    if model_dir is not None and any((model_dir / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tiktoken.model")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(str(model_dir), trust_remote_code=False)
    return ByteTokenizer(vocab_size)


def eos_ids(tok: Any, model_dir: Path | None, config_eos: tuple[int, ...] = (), model_id: str = "") -> tuple[int, ...]:
    ids = set(config_eos)
    known = known_eos_ids(model_id)
    if known and getattr(tok, "vocab_size", 0) > max(known):
        ids.update(known)
    if getattr(tok, "eos_token_id", None) is not None:
        ids.add(int(tok.eos_token_id))
    if model_dir is not None and (model_dir / "generation_config.json").exists():
        try:
            e = json.loads((model_dir / "generation_config.json").read_text()).get("eos_token_id")
            ids.update([e] if isinstance(e, int) else (e or []))
        except (OSError, ValueError):
            pass
    return tuple(sorted(ids))


class Detokenizer:
    """Incremental decode that never emits half a UTF-8 character (prefix / read offsets)."""

    def __init__(self, tok: Any, prompt_tail: list[int] | None = None):
        self.tok = tok
        self.ids: list[int] = list(prompt_tail or [])[-6:]
        self.prefix, self.read = 0, len(self.ids)

    def add(self, token_id: int) -> str:
        self.ids.append(token_id)
        old = self.tok.decode(self.ids[self.prefix:self.read], skip_special_tokens=True)
        new = self.tok.decode(self.ids[self.prefix:], skip_special_tokens=True)
        if len(new) > len(old) and not new.endswith("�"):
            self.prefix, self.read = self.read, len(self.ids)
            return new[len(old):]
        return ""


def build_messages(p: TextGenerationTaskParams) -> list[dict[str, Any]]:
    if p.chat_template_messages is not None:
        msgs = [dict(m) for m in p.chat_template_messages]
    else:
        msgs = [{"role": m.role, "content": m.content} for m in p.input]
        if p.instructions:
            msgs.insert(0, {"role": "system", "content": p.instructions})
    # merge system messages into the first one (templates generally accept a single leading system turn)
    systems = [m for m in msgs if m.get("role") in ("system", "developer") and isinstance(m.get("content"), str)]
    if len(systems) > 1:
        merged = "\n\n".join(m["content"] for m in systems)
        rest = [m for m in msgs if m not in systems]
        msgs = [{"role": "system", "content": merged}] + rest
    return msgs


_LENGTH_GUARD = re.compile(r"""(inner_type\s*==\s*["']object \| object["'])\s*or\s*inner_type\|length\s*>\s*\d+""")


def without_schema_length_guard(template: str) -> str | None:
    """Some templates (GPT-OSS) render an array-of-objects parameter as ``any[]`` once its rendered type is longer than
    a fixed number of characters, which hides nested tool schemas from the model.  Returns the template with that
    length test removed (the object-union test stays), or ``None`` when the template has no such guard
    (``src/exo/worker/engines/mlx/utils_mlx.py:460-483``)."""
    patched, n = _LENGTH_GUARD.subn(lambda m: m.group(1), template)
    return patched if n else None


def normalize_tool_calls(msg: dict[str, Any]) -> None:
    """Chat templates iterate ``tool_call.function.arguments`` as a mapping: JSON-string arguments are parsed."""
    for tc in msg.get("tool_calls") or []:
        fn = tc.get("function") if isinstance(tc, dict) else None
        if isinstance(fn, dict) and isinstance(fn.get("arguments"), str):
            try:
                fn["arguments"] = json.loads(fn["arguments"])
            except ValueError:
                pass


def render_prompt(tok: Any, p: TextGenerationTaskParams) -> tuple[str, bool]:
    """Returns ``(prompt text, continues_assistant_turn)``."""
    msgs = build_messages(p)
    cont = bool(msgs) and msgs[-1].get("role") == "assistant" and bool(msgs[-1].get("content"))
    enc = encoder_for(p.model)
    if enc is not None:
        # the format is code: DeepSeek-V3.2 / V4 (thinking unless the request switches it off)
        tail = msgs.pop()["content"] if cont else ""
        for m in msgs:
            if m.get("role") == "assistant" and isinstance(m.get("content"), str):
                m["content"] = strip_think_blocks(m["content"])
        effort = {"xhigh": "max", "high": "high"}.get(p.reasoning_effort or "")
        text = enc.encode(msgs, thinking=p.enable_thinking is not False, tools=p.tools, reasoning_effort=effort)
        return text + tail, cont
    if getattr(tok, "chat_template", None):
        kw: dict[str, Any] = {}
        if p.enable_thinking is not None:
            kw["enable_thinking"] = p.enable_thinking      # Qwen3, GLM
            kw["thinking"] = p.enable_thinking             # DeepSeek templates; unknown variables are ignored
        if p.reasoning_effort is not None:
            kw["reasoning_effort"] = p.reasoning_effort
        for m in msgs:
            normalize_tool_calls(m)
            if "gpt-oss" in p.model.lower() and m.get("role") == "assistant" and "thinking" not in m \
                    and isinstance(m.get("reasoning_content"), str) and m["reasoning_content"]:
                m["thinking"] = m["reasoning_content"]
        if p.tools and isinstance(tok.chat_template, str):
            patched = without_schema_length_guard(tok.chat_template)
            if patched is not None:
                kw["chat_template"] = patched
        text = tok.apply_chat_template(msgs, tools=p.tools, tokenize=False, add_generation_prompt=not cont,
                                       continue_final_message=cont, **kw)
        return text, cont
    lines = []
    for m in msgs:
        c = m.get("content")
        if isinstance(c, list):
            c = "".join(part.get("text", "") for part in c if isinstance(part, dict))
        lines.append(f"<|{m.get('role')}|>\n{c or ''}")
    if p.tools:
        lines.insert(0, "<|tools|>\n" + json.dumps(p.tools))
    return "\n".join(lines) + ("" if cont else "\n<|assistant|>\n"), cont
