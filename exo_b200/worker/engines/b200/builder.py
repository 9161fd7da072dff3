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
import queue
import threading
import time
import uuid
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
from ...disaggregated import protocol as dproto
from ...disaggregated.server import PrefillServer, remote_prefill_fetch

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}
_DTYPE_NAME = {v: k for k, v in _TORCH_DTYPE.items()}
KV_CHUNK_TOKENS = 4096


class _PrefillJob:
    """A prompt whose KV a decode instance asked for; filled in by the engine loop, sent by the server thread."""

    def __init__(self, request: dproto.PrefillRequest):
        self.request = request
        self.done = threading.Event()
        self.layers: list[tuple[torch.Tensor, torch.Tensor | None]] = []     # CPU tensors [tokens, heads, dim]
        self.n_tokens = 0
        self.error: str | None = None


class _RemoteFetch:
    """A request waiting for its prompt KV from a prefill instance (fetched on a side thread)."""

    def __init__(self, task: TextGeneration, ids: list[int], endpoint: str, model_id: str):
        self.task, self.ids = task, ids
        self.result = None
        self.error: Exception | None = None
        self.t0 = time.perf_counter()
        req = dproto.PrefillRequest(request_id=str(task.task_id), model_id=model_id, token_ids=list(ids), start_pos=0)

        def run() -> None:
            try:
                self.result = remote_prefill_fetch(endpoint, req)
            except Exception as e:  # noqa: BLE001 - any failure falls back to local prefill
                self.error = e
        self.thread = threading.Thread(target=run, name="remote-prefill", daemon=True)
        self.thread.start()


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
        # prefill/decode disaggregation: jobs served for other instances, and fetches this instance waits for
        self.prefill_server: PrefillServer | None = None
        self.prefill_server_port: int | None = None
        self.prefill_jobs: "queue.Queue[_PrefillJob]" = queue.Queue()
        self.prefill_running: dict[str, tuple[_PrefillJob, Any, int]] = {}
        self.remote: dict[str, _RemoteFetch] = {}
        self.remote_prefills = 0
        self.vision = None          # VisionProcessor, built on the first request that carries images

    # ---- images ----
    def _checkpoint_vision(self, device, dtype):
        """``(processor, tower, placeholder token, wrap)`` built from the model's own checkpoint when it carries a vision
        tower this engine knows (Qwen2-VL, Qwen3-VL / Qwen3.5, Gemma-4, Kimi-K2.5); ``None`` otherwise (the generic tower then stands in).
        ``wrap``: tokens put before and after an image's soft tokens."""
        import json
        from ....models.weights import SafetensorsSource
        from .vision_families import (Gemma4Processor, Gemma4VisionConfig, Gemma4VisionTower, KimiTower, KimiTowerConfig, KimiVLProcessor,
                                      QwenVLProcessor, QwenVLTower, QwenVLTowerConfig, family_for)
        d = find_model_dir(self.model_id)
        if d is None or not (d / "config.json").exists() or not any(d.glob("*.safetensors")):
            return None
        config = json.loads((d / "config.json").read_text())
        pre = json.loads((d / "preprocessor_config.json").read_text()) if (d / "preprocessor_config.json").exists() else {}
        proc = family_for(config, pre)
        src = SafetensorsSource(d, device="cpu", dtype=torch.float32)
        names = list(src.names())
        tok_id = lambda t: self.tok.convert_tokens_to_ids(t) if hasattr(self.tok, "convert_tokens_to_ids") else None   # noqa: E731
        if isinstance(proc, Gemma4Processor):
            prefix = next((p for p in ("model.vision_tower.", "vision_tower.") if any(n.startswith(p) for n in names)), None)
            if prefix is None:
                return None
            emb = prefix.replace("vision_tower.", "embed_vision.")
            tower = Gemma4VisionTower.from_source(src, Gemma4VisionConfig.from_config(config.get("vision_config") or {}), device, dtype,
                                                  prefix, emb)
            ph = config.get("image_token_id") or tok_id(getattr(self.tok, "image_token", "<|image|>"))
            wrap = (config.get("boi_token_id") or tok_id(getattr(self.tok, "boi_token", "<|image>")),
                    config.get("eoi_token_id") or tok_id(getattr(self.tok, "eoi_token", "<image|>")))
            return proc, tower, ph, wrap
        if isinstance(proc, KimiVLProcessor) and str(config.get("model_type")) in ("kimi_k25", "kimi_k2_5"):
            if not any(n.startswith("vision_tower.") for n in names):
                return None
            tower = KimiTower.from_source(src, KimiTowerConfig.from_config(config.get("vision_config") or {}), device, dtype)
            return proc, tower, config.get("media_placeholder_token_id") or tok_id("<|media_pad|>"), None
        if isinstance(proc, QwenVLProcessor):
            # Qwen2-VL and the Qwen3-VL line (Qwen3.5 / 3.6 included); the windowed Qwen2.5-VL tower is not built
            prefix = next((p for p in ("visual.", "model.visual.", "vision_tower.") if any(n.startswith(p) for n in names)), None)
            if prefix is None or str(config.get("model_type")) == "qwen2_5_vl":
                return None
            tower = QwenVLTower.from_source(src, QwenVLTowerConfig.from_config(config.get("vision_config") or {}), device, dtype, prefix)
            return proc, tower, config.get("image_token_id") or tok_id("<|image_pad|>"), None
        return None

    def _with_images(self, ids: list[int], images: list[str]):
        """Prompt ids with every image expanded to its feature rows: ``(ids, embeds, media)`` for the token engine.
        On a multi-rank instance this runs on rank 0; the rows follow each step's plan to the other ranks."""
        import base64
        import hashlib
        import io
        from .vision import ImageFeatures, VisionConfig, VisionProcessor, VisionTower, splice
        exe = self.te.exe
        dtype = torch.float32 if exe.device.type == "cpu" else torch.bfloat16
        if self.vision is None:
            self.vision = self._checkpoint_vision(exe.device, dtype) or VisionProcessor(
                VisionTower(VisionConfig(out_hidden=self.cfg.hidden), exe.device, dtype))
        if isinstance(self.vision, tuple):
            from PIL import Image
            proc, tower, ph, wrap = self.vision
            feats = []
            for b in images:
                raw = base64.b64decode(b.split(",", 1)[1] if b.startswith("data:") else b)
                im = Image.open(io.BytesIO(raw))
                a, g, _counts = proc([im])
                rows = tower(a[0], g[0]) if isinstance(a, list) else tower(a, g)
                feats.append(ImageFeatures(hashlib.sha256(raw).digest(), rows))
            fill = ph if ph is not None else (getattr(self.tok, "pad_token_id", None) or 0)
            out, embeds, media = splice(ids, ph, feats, fill)
            if wrap and all(isinstance(t, int) and t >= 0 for t in wrap):
                # begin / end markers around every image's soft tokens (later images shift by the markers put before them)
                shifted, k = [], 0
                for (pos, rows), (a0, a1, dg) in zip(embeds, media):
                    out[pos + k:pos + k] = [wrap[0]]
                    out[pos + k + 1 + rows.shape[0]:pos + k + 1 + rows.shape[0]] = [wrap[1]]
                    shifted.append(((pos + k + 1, rows), (a0 + k + 1, a1 + k + 1, dg)))
                    k += 2
                embeds, media = [e for e, _ in shifted], [m for _, m in shifted]
            return out, embeds, media
        feats = [self.vision.features(b) for b in images]
        ph = None
        conv = getattr(self.tok, "convert_tokens_to_ids", None)
        if conv is not None:
            cand = conv("<|image_pad|>")
            if isinstance(cand, int) and cand >= 0 and cand != getattr(self.tok, "unk_token_id", None):
                ph = cand
        fill = ph if ph is not None else (getattr(self.tok, "pad_token_id", None) or 0)
        return splice(ids, ph, feats, fill)

    # ---- Engine interface ----
    def warmup(self) -> None:
        self.te.warmup(4)

    @property
    def has_work(self) -> bool:
        return (bool(self.reqs) or bool(self.finished_buffer) or self.te.has_work or bool(self.remote)
                or bool(self.prefill_running) or not self.prefill_jobs.empty())

    # ---- disaggregation: prefill side ----
    def enable_prefill_server(self, host: str = "0.0.0.0", port: int = 0) -> int:
        """Serve prompt KV to decode instances (single-rank instances only: one rank holds every KV head)."""
        self.prefill_server = PrefillServer(self._resolve_prefill, host, port)
        self.prefill_server_port = self.prefill_server.port
        return self.prefill_server.port

    def _resolve_prefill(self, request: dproto.PrefillRequest, wfile) -> bool:
        """Server thread: queue the prompt for the engine loop, wait, stream the KV back."""
        if request.model_id and request.model_id != self.model_id:
            raise ValueError(f"this instance serves {self.model_id}, not {request.model_id}")
        job = _PrefillJob(request)
        self.prefill_jobs.put(job)
        if not job.done.wait(timeout=float(os.environ.get("EXO_PREFILL_JOB_TIMEOUT_S", "600"))):
            return False
        if job.error is not None:
            raise RuntimeError(job.error)
        kv_layers = [(li, e) for li, e in enumerate(job.layers) if not isinstance(e[0], str)]
        dt = _DTYPE_NAME[kv_layers[0][1][0].dtype] if kv_layers else "float32"
        dproto.write_header(wfile, dproto.Header(request_id=request.request_id, model_id=self.model_id,
                                                 num_layers=len(job.layers), dtype=dt, start_pos=request.start_pos))
        for li, e in enumerate(job.layers):          # recurrent layers: their whole state, once
            if isinstance(e[0], str):
                dproto.write_message(wfile, dproto.ArraysState(layer_idx=li, arrays=[
                    dproto.TensorBlob(_DTYPE_NAME[t.dtype], tuple(t.shape), t.contiguous().view(torch.uint8).numpy().tobytes()) for t in e[1]]))
        lo = min(request.start_pos, job.n_tokens)
        for t0 in range(lo, job.n_tokens, KV_CHUNK_TOKENS):
            t1 = min(job.n_tokens, t0 + KV_CHUNK_TOKENS)
            for li, (k, v) in kv_layers:
                kb = k[t0:t1].contiguous().view(torch.uint8).numpy().tobytes()
                vb = b"" if v is None else v[t0:t1].contiguous().view(torch.uint8).numpy().tobytes()
                dproto.write_message(wfile, dproto.KVChunk(layer_idx=li, num_tokens=t1 - t0, n_heads=k.shape[1] if k.dim() == 3 else 1,
                                                           head_dim=k.shape[-1], dtype=dt, keys=kb, values=vb))
        dproto.write_message(wfile, dproto.Done(total_tokens=job.n_tokens))
        return True

    def _start_prefill_jobs(self) -> None:
        while True:
            try:
                job = self.prefill_jobs.get_nowait()
            except queue.Empty:
                return
            ids = job.request.token_ids
            target = max(0, len(ids) - 2)       # the decode side computes the last two tokens itself
            if target == 0:
                job.done.set()
                continue
            rid = f"prefill-{uuid.uuid4().hex}"
            try:
                self.te.submit(ids[:target], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True), req_id=rid)
            except Exception as e:  # noqa: BLE001
                job.error = str(e)
                job.done.set()
                continue
            self.prefill_running[rid] = (job, self.te.seqs[rid], target)

    def _finish_prefill_job(self, rid: str) -> None:
        job, seq, target = self.prefill_running.pop(rid)
        try:
            # the sequence's blocks were just released but nothing has been allocated since: the data is intact
            job.layers = [(e[0], [t.cpu() for t in e[1]]) if isinstance(e[0], str) else (e[0].cpu(), None if e[1] is None else e[1].cpu())
                          for e in self.te.export_kv(seq.final_blocks, target, seq.final_seat)]
            job.n_tokens = target
        except Exception as e:  # noqa: BLE001
            job.error = str(e)
        job.done.set()

    # ---- disaggregation: decode side ----
    def _want_remote_prefill(self, p, ids: list[int]) -> bool:
        return (bool(p.prefill_endpoint) and len(ids) > constants.REMOTE_PREFILL_MIN_TOKENS
                and self.te.exe.spec.tp_size == 1 and self.te.exe.spec.pp_size == 1)

    def _admit_remote(self) -> None:
        for rid, f in list(self.remote.items()):
            if f.thread.is_alive():
                continue
            del self.remote[rid]
            r = self.reqs.get(rid)
            if r is None:      # cancelled while the KV was in flight
                continue
            p = f.task.task_params
            kv = None
            if f.error is None and f.result is not None and f.result.total_tokens > 0:
                try:
                    dt = _TORCH_DTYPE[f.result.header.dtype]
                    layers = []
                    for li in range(f.result.header.num_layers):
                        if li in f.result.states:        # a recurrent layer's state (or a layer that keeps nothing)
                            layers.append(("state", [torch.frombuffer(bytearray(b.data), dtype=_TORCH_DTYPE[b.dtype]).view(b.shape)
                                                     for b in f.result.states[li].arrays]))
                            continue
                        chunks = f.result.chunks[li]
                        shape = (-1, chunks[0].n_heads, chunks[0].head_dim)
                        k = torch.frombuffer(bytearray(b"".join(c.keys for c in chunks)), dtype=dt).view(shape)
                        vb = b"".join(c.values for c in chunks)          # empty: a latent cache has keys only (MLA)
                        v = torch.frombuffer(bytearray(vb), dtype=dt).view(shape) if vb else None
                        layers.append((k, v))
                    kv = (f.result.total_tokens, layers)
                    self.remote_prefills += 1
                except Exception:  # noqa: BLE001 - malformed stream: compute locally
                    kv = None
            self.te.submit(f.ids, self._sampling(p), req_id=rid, use_prefix_cache=p.use_prefix_cache or not p.bench,
                           kv_prefill=kv)

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
        embeds = media = None
        if p.images:
            ids, embeds, media = self._with_images(ids, list(p.images))
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
        if embeds is None and self._want_remote_prefill(p, ids):
            self.remote[rid] = _RemoteFetch(task, ids, p.prefill_endpoint, self.model_id)
            return
        self.te.submit(ids, self._sampling(p), req_id=rid, use_prefix_cache=p.use_prefix_cache or not p.bench, media=media,
                       embeds=embeds)

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
        self._start_prefill_jobs()
        self._admit_remote()
        if not self.te.has_work:
            if self.remote:
                time.sleep(0.002)      # only waiting for KV from a prefill instance
            return out
        with tracing.trace("engine.step", self.rank, "step", cuda=self.te.exe.cuda):
            outs = self.te.step()
        now = time.perf_counter()
        for o in outs:
            if o.finished and o.req_id in self.prefill_running:
                self._finish_prefill_job(o.req_id)
                continue
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
        if self.prefill_server is not None:
            self.prefill_server.stop()
        if self.control is not None:
            self.control.close()
