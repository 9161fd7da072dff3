"""The B200 engine behind the runner: bring-up (rank group, shard load) and serving.

``B200Builder`` is what the reference's ``MlxBuilder`` is to MLX (``src/exo/worker/engines/mlx/
builder.py:60-113``, ``utils_mlx.py:90-286``): ``connect`` joins the instance's rank group
(NCCL + a gloo side channel on 127.0.0.1:<rendezvous port>; peer-memory arenas for the fused
collectives), ``load`` reads this rank's slice of the HF checkpoint layer by layer (progress is
reported per layer), ``build`` returns the serving engine.  Rank 0 runs the scheduler and
broadcasts each step's packed plan; the other ranks execute plans and keep no request state.
"""
from __future__ import annotations

import os
import time
from collections.abc import Iterable, Iterator
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ....api.types import CompletionTokensDetails, GenerationStats, PromptTokensDetails, TopLogprobItem, Usage
from ....engine.engine import Engine as TokenEngine
from ....engine.executor import Executor
from ....engine.kv import SamplingParams
from ....engine.plan import StepPlan
from ....models.config import ModelConfig
from ....models.transformer import KVPool
from ....models.weights import (RandomSource, SafetensorsSource, ShardSpec, build_weights, fast_random_weights,
                                vocab_shard)
from ....shared import constants, tracing
from ....shared.base import Memory, ModelId, TaskId
from ....shared.messages import GenerationTask, TextGeneration
from ....shared.wire import BoundInstance, PrefillProgressChunk, TokenChunk, ToolCallChunk
from ..base import Builder, Cancelled, Engine, Finished, LoadProgress, StepItem
from .parsers import tool_dialect_for
from .stream_parser import HarmonyParser, StreamParser
from .tokenizer import Detokenizer, eos_ids, load_tokenizer, render_prompt


def find_model_dir(model_id: str) -> Path | None:
    if os.path.isdir(model_id):
        return Path(model_id)
    for base in constants.models_dirs():
        p = base / ModelId(model_id).normalize()
        if (p / "config.json").exists():
            return p
    return None


class _Request:
    def __init__(self, task: TextGeneration, prompt_ids: list[int], detok: Detokenizer, parser, stops: list[str]):
        self.task, self.prompt_ids, self.detok, self.parser, self.stops = task, prompt_ids, detok, parser, stops
        self.text = ""
        self.n_out = 0
        self.t_submit = time.perf_counter()
        self.t_first = self.t_last = 0.0
        self.prefill_reported = 0
        self.cached = 0
        self.done = False


class ServingEngine(Engine):
    """Leader-side engine: tokens in, chunks out."""

    def __init__(self, cfg: ModelConfig, token_engine: TokenEngine, tokenizer: Any, model_id: str, family: str,
                 eos: tuple[int, ...], reasoning_dialect: str = "none", rank: int = 0, control=None):
        self.cfg, self.te, self.tok = cfg, token_engine, tokenizer
        self.model_id, self.family, self.eos, self.dialect = model_id, family, eos, reasoning_dialect
        self.rank, self.control = rank, control
        self.reqs: dict[str, _Request] = {}
        self.finished_buffer: list[tuple[TaskId, StepItem]] = []
        self.peak_mem = 0

    # ---- Engine interface ----
    def warmup(self) -> None:
        self.te.warmup(4)

    @property
    def has_work(self) -> bool:
        return bool(self.reqs) or bool(self.finished_buffer) or self.te.has_work

    def _sampling(self, p) -> SamplingParams:
        bench = p.bench
        ctx_left = self.cfg.max_position
        return SamplingParams(
            temperature=0.7 if p.temperature is None else p.temperature, top_p=1.0 if p.top_p is None else p.top_p,
            top_k=p.top_k or 0, min_p=0.05 if p.min_p is None else p.min_p,
            max_tokens=min(p.max_output_tokens or constants.MAX_TOKENS, ctx_left), stop_token_ids=(),
            ignore_eos=bench, seed=p.seed, repetition_penalty=p.repetition_penalty or 1.0,
            presence_penalty=p.presence_penalty or 0.0, frequency_penalty=p.frequency_penalty or 0.0,
            logprobs=p.logprobs, top_logprobs=p.top_logprobs or (constants.DEFAULT_TOP_LOGPROBS if p.logprobs else 0))

    def submit(self, task: GenerationTask) -> None:
        assert isinstance(task, TextGeneration)
        p = task.task_params
        text, cont = render_prompt(self.tok, p)
        ids = self.tok.encode(text, add_special_tokens=not getattr(self.tok, "chat_template", None))
        if not ids:
            ids = [getattr(self.tok, "bos_token_id", 0) or 0]
        if len(ids) >= self.cfg.max_position:
            raise ValueError(f"prompt of {len(ids)} tokens exceeds the context length {self.cfg.max_position}")
        parser = None
        if not p.bench:
            if self.dialect == "channel":
                parser = HarmonyParser(p.tools)
            else:
                thinking_on = p.enable_thinking is not False and self.dialect != "none"
                starts = thinking_on and text.rstrip().endswith("<think>")
                parser = StreamParser(starts_in_thinking=starts, tool=tool_dialect_for(self.family, self.model_id) if p.tools else None,
                                      tools=p.tools)
        stops = [p.stop] if isinstance(p.stop, str) else list(p.stop or [])
        rid = str(task.task_id)
        self.reqs[rid] = _Request(task, ids, Detokenizer(self.tok, ids), parser, stops)
        self.te.submit(ids, self._sampling(p), req_id=rid, use_prefix_cache=p.use_prefix_cache or not p.bench)

    def cancel(self, task_id: TaskId) -> None:
        r = self.reqs.pop(str(task_id), None)
        if r is not None:
            self.te.cancel(str(task_id))
            self.finished_buffer.append((task_id, Cancelled()))

    # ---- output assembly ----
    def _usage(self, r: _Request, reasoning_tokens: int) -> Usage:
        return Usage(prompt_tokens=len(r.prompt_ids), completion_tokens=r.n_out, total_tokens=len(r.prompt_ids) + r.n_out,
                     prompt_tokens_details=PromptTokensDetails(cached_tokens=r.cached),
                     completion_tokens_details=CompletionTokensDetails(reasoning_tokens=reasoning_tokens))

    def _stats(self, r: _Request) -> GenerationStats:
        prefill_s = max(r.t_first - r.t_submit, 1e-9)
        gen_s = max(r.t_last - r.t_first, 1e-9)
        if torch.cuda.is_available() and self.te.exe.cuda:
            self.peak_mem = max(self.peak_mem, torch.cuda.max_memory_allocated(self.te.exe.device))
        hit = "none" if r.cached == 0 else ("exact" if r.cached >= len(r.prompt_ids) - 16 else "partial")
        return GenerationStats(prompt_tps=len(r.prompt_ids) / prefill_s,
                               generation_tps=(r.n_out - 1) / gen_s if r.n_out > 1 else 0.0,
                               prompt_tokens=len(r.prompt_ids), generation_tokens=r.n_out,
                               peak_memory_usage=Memory.from_bytes(self.peak_mem), prefix_cache_hit=hit)

    def _chunks(self, r: _Request, o, piece_text: str, finish: str | None) -> list[StepItem]:
        """Turn one sampled token (already detokenised) into chunks, running the parser pipeline."""
        out: list[StepItem] = []
        tid = o.token if o.token is not None else 0
        lp = o.logprob
        tops = None
        if o.top_logprobs:
            tops = [TopLogprobItem(token=self.tok.decode([i]), logprob=v) for i, v in o.top_logprobs]
        if r.parser is None:
            usage = self._usage(r, 0) if finish else None
            out.append(TokenChunk(model=self.model_id, text=piece_text, token_id=tid, usage=usage, finish_reason=finish,
                                  stats=self._stats(r) if finish else None, logprob=lp, top_logprobs=tops))
            return out
        pieces = r.parser.feed(piece_text)
        if finish:
            pieces += r.parser.finish()
        reasoning = getattr(r.parser, "reasoning_chars", 0) // 4
        calls = [p for p in pieces if p.kind == "tool_calls"]
        texts = [p for p in pieces if p.kind in ("text", "thinking", "error")]
        for i, p in enumerate(texts):
            last = finish and i == len(texts) - 1 and not calls
            out.append(TokenChunk(model=self.model_id, text=p.text, token_id=tid, usage=self._usage(r, reasoning) if last else None,
                                  finish_reason=finish if last else None, stats=self._stats(r) if last else None,
                                  logprob=lp, top_logprobs=tops, is_thinking=p.kind == "thinking"))
        if calls:
            out.append(ToolCallChunk(model=self.model_id, tool_calls=[c for p in calls for c in p.tool_calls],
                                     usage=self._usage(r, reasoning), stats=self._stats(r)))
        elif finish and not texts:
            out.append(TokenChunk(model=self.model_id, text="", token_id=tid, usage=self._usage(r, reasoning),
                                  finish_reason=finish, stats=self._stats(r), logprob=lp, top_logprobs=tops))
        return out

    def step(self) -> Iterable[tuple[TaskId, StepItem]]:
        out, self.finished_buffer = self.finished_buffer, []
        if not self.te.has_work:
            return out
        with tracing.trace("engine.step", self.rank, "step", cuda=self.te.exe.cuda):
            outs = self.te.step()
        now = time.perf_counter()
        for o in outs:
            r = self.reqs.get(o.req_id)
            if r is None:
                continue
            task_id = r.task.task_id
            r.cached = o.n_cached
            if o.token is None:  # still prefilling
                if o.prefill_done - r.prefill_reported >= 1024 or o.prefill_done == len(r.prompt_ids):
                    r.prefill_reported = o.prefill_done
                    out.append((task_id, PrefillProgressChunk(model=self.model_id, processed_tokens=o.prefill_done,
                                                              total_tokens=len(r.prompt_ids))))
                continue
            r.n_out += 1
            if r.n_out == 1:
                r.t_first = now
            r.t_last = now
            is_eos = o.finished and o.finish_reason == "stop" and o.token in self.eos
            piece = "" if is_eos else r.detok.add(o.token)
            finish = o.finish_reason if o.finished else None
            if r.stops and piece:
                r.text += piece
                cut = min((r.text.find(s) for s in r.stops if s and s in r.text), default=-1)
                if cut >= 0:   # stop sequence: trim the emitted text and end the request
                    piece = piece[:max(0, len(piece) - (len(r.text) - cut))]
                    finish = "stop"
                    if not o.finished:
                        self.te.cancel(o.req_id)
            for c in self._chunks(r, o, piece, finish):
                out.append((task_id, c))
            if finish:
                self.reqs.pop(o.req_id, None)
                out.append((task_id, Finished()))
        return out

    def collect_traces(self) -> list:
        spans = tracing.get_trace_buffer()
        tracing.clear_trace_buffer()
        return spans

    def close(self) -> None:
        if self.control is not None:
            self.control.close()
