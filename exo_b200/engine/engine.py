"""Token-level inference engine: scheduler + executor behind ``submit`` / ``step``.

This is the object a runner process drives; it has the same call surface the reference
gives its engines (``src/exo/worker/engines/base.py:16-60``: warmup / submit / step / close),
working on token ids — tokenisation, chat templates and output parsing live above it.
"""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.weights import ModelWeights, ShardSpec
from ..ops import reference as ref
from .executor import Executor
from .kv import BlockAllocator, SamplingParams, Sequence
from .plan import FLAG_EAGER, FLAG_NO_SAMPLE, StepPlan
from .scheduler import Scheduler


@dataclass
class StepOutput:
    req_id: str
    token: int | None          # None while the request is still prefilling
    finished: bool
    finish_reason: str | None
    n_prompt: int
    n_generated: int
    n_cached: int
    logprob: float | None = None
    top_logprobs: list[tuple[int, float]] | None = None
    prefill_done: int = 0      # prompt tokens processed so far (for progress reporting)


class Engine:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, spec: ShardSpec | None = None, comm=None,
                 n_blocks: int = 512, block_size: int = 16, max_seqs: int = 64, prefill_chunk: int = 4096,
                 max_blocks_per_seq: int | None = None, device: str | torch.device = "cpu",
                 use_graphs: bool | None = None, seed: int = 0, plan_sink=None, pipe=None):
        self.cfg = cfg
        mbs = max_blocks_per_seq or min(n_blocks, -(-cfg.max_position // block_size))
        self.alloc = BlockAllocator(n_blocks, block_size)
        self.scratch_block = self.alloc.alloc()  # block 0: target of padded rows, never read
        assert self.scratch_block == 0
        self.sched = Scheduler(self.alloc, max_seqs=max_seqs, prefill_chunk=prefill_chunk, max_blocks_per_seq=mbs,
                               eos_token_ids=cfg.eos_token_ids, max_context=cfg.max_position, seed=seed)
        self.exe = Executor(cfg, weights, spec, comm, n_blocks=n_blocks, block_size=block_size,
                            max_blocks_per_seq=mbs, max_tokens_per_step=max(prefill_chunk, max_seqs),
                            max_seqs=max_seqs, device=device, use_graphs=use_graphs, pipe=pipe)
        if self.exe.kv.n_snapshots:         # hybrid model: prefixes are reusable up to blocks with a state snapshot
            self.alloc.enable_snapshots(self.exe.kv.n_snapshots)
            self.sched.state_snapshots = True
        self.seqs: dict[str, Sequence] = {}
        self.plan_sink = plan_sink  # callable(StepPlan): broadcasts the plan to follower ranks
        self.embed_sink = None      # callable([(row, rows)]): hands caller-supplied embedding rows to the follower ranks
        self.n_steps = 0

    # ---- requests ----
    def submit(self, prompt: list[int], params: SamplingParams | None = None, req_id: str | None = None,
               use_prefix_cache: bool = True, media=None, kv_prefill=None, embeds=None) -> str:
        """Queue a request.  ``embeds = [(position, rows [n, hidden])]`` replaces the token embeddings of those prompt
        positions (image features spliced over placeholder tokens; ``media`` carries their content hashes for the prefix cache).  ``kv_prefill = (n_tokens, [(k, v) per local layer])`` installs KV computed
        elsewhere (a prefill instance) for the first ``n_tokens`` prompt tokens; prefill continues after them."""
        rid = req_id or uuid.uuid4().hex
        if not prompt:
            raise ValueError("empty prompt")
        seat = 0
        if self.cfg.has_linear_layers:
            # a recurrent layer's state summarises the WHOLE prefix: cached blocks are reusable only up to one whose
            # end-of-block state was snapshotted (the scheduler's rule), and KV computed elsewhere is usable only together
            # with the recurrent layers' states after exactly those tokens, installed into a seat of this engine
            use_prefix_cache = use_prefix_cache and self.sched.state_snapshots
            if kv_prefill is not None:
                if self.sched._free_seats and any(isinstance(e[0], str) for e in kv_prefill[1]) and int(kv_prefill[0]) < len(prompt):
                    seat = self.sched._free_seats.pop()
                else:
                    kv_prefill = None
        s = Sequence(rid, list(prompt), params or SamplingParams(), media=media, use_prefix_cache=use_prefix_cache)
        s.embeds = list(embeds) if embeds else None
        if kv_prefill is not None:
            n, layers = kv_prefill
            # the last prompt token is always computed here (it yields the logits); recurrent states cannot be cut short
            n = int(n) if seat else min(int(n), len(prompt) - 1)
            if n > 0 and self.sched._ensure_blocks(s, n):
                self.import_kv(s.blocks, n, layers, seat)
                s.n_computed, s.state_slot = n, seat
            else:
                self.alloc.release_all(s.blocks)
                s.blocks = []
                if seat:
                    self.sched._free_seats.append(seat)
        self.seqs[rid] = s
        self.sched.add(s)
        return rid

    def _embed_patches(self, entries) -> list | None:
        """Rows of this step's packed token batch whose embeddings come from ``Sequence.embeds``: ``[(row, rows)]``."""
        out, row = [], 0
        for s, n in entries:
            if s.embeds and s.n_computed < len(s.prompt):
                lo, hi = s.n_computed, s.n_computed + n
                for start, t in s.embeds:
                    a, b = max(lo, start), min(hi, start + t.shape[0])
                    if a < b:
                        out.append((row + a - lo, t[a - start:b - start]))
            row += n
        return out or None

    # ---- KV hand-over (prefill/decode disaggregation) ----
    def _slots(self, blocks: list[int], n_tokens: int) -> torch.Tensor:
        bs = self.alloc.block_size
        b = torch.tensor(blocks[:-(-n_tokens // bs)], dtype=torch.long, device=self.exe.device)
        return (b[:, None] * bs + torch.arange(bs, device=self.exe.device)[None, :]).reshape(-1)[:n_tokens]

    def export_kv(self, blocks: list[int], n_tokens: int, seat: int = 0) -> list[tuple]:
        """What this engine remembers of the first ``n_tokens`` positions, per local layer: ``(k, v)`` rows ``[n_tokens, heads,
        dim]`` from ``blocks`` for attention layers; ``("state", [tensors])`` for recurrent layers (their state in ``seat``,
        which must be the state after exactly ``n_tokens`` tokens) and for layers that keep nothing (no tensors)."""
        if self.cfg.has_linear_layers and not seat:
            raise ValueError(f"{self.cfg.name}: the recurrent layers' state lives in a seat; none was given")
        slots = self._slots(blocks, n_tokens)
        out: list[tuple] = []
        for i in self.exe.spec.layers(self.cfg):
            k, v = self.exe.kv.layers[i]
            if k is None:
                out.append(("state", []))
            elif self.cfg.layer_is_linear(i):
                out.append(("state", [k[seat].clone(), v[seat].clone()]))
            else:
                out.append((k.view(-1, *k.shape[2:])[slots], None if v is None else v.view(-1, *v.shape[2:])[slots]))
        return out

    def import_kv(self, blocks: list[int], n_tokens: int, layers, seat: int = 0) -> None:
        slots = self._slots(blocks, n_tokens)
        for i, entry in zip(self.exe.spec.layers(self.cfg), layers):
            k, v = self.exe.kv.layers[i]
            if isinstance(entry[0], str):             # ("state", tensors): a recurrent layer's state, or nothing
                for dst, src in zip((k, v), entry[1]):
                    dst[seat] = src.to(device=dst.device, dtype=dst.dtype).view(dst[seat].shape)
                continue
            k_new, v_new = entry
            rows = k.view(-1, *k.shape[2:])
            rows[slots] = k_new[:n_tokens].to(device=k.device, dtype=k.dtype).reshape(-1, *rows.shape[1:])      # (a latent cache has no head axis)
            if v is not None and v_new is not None:
                v.view(-1, *v.shape[2:])[slots] = v_new[:n_tokens].to(device=v.device, dtype=v.dtype)

    def cancel(self, req_id: str) -> bool:
        ok = self.sched.cancel(req_id)
        self.seqs.pop(req_id, None)
        return ok

    @property
    def has_work(self) -> bool:
        return self.sched.has_work

    # ---- stepping ----
    def _processor(self, entries):
        """Logits processor for steps where some sequence wants penalties."""
        seqs = [s for s, _ in entries]
        if not any(s.params.has_penalties for s in seqs):
            return None
        V = self.cfg.vocab

        def proc(logits: torch.Tensor) -> torch.Tensor:
            counts = torch.zeros(len(seqs), V, device=logits.device)
            for b, s in enumerate(seqs):
                if s.params.has_penalties and s.output:
                    idx = torch.tensor(s.output, device=logits.device)
                    counts[b].index_add_(0, idx, torch.ones(len(s.output), device=logits.device))
            rep = torch.tensor([s.params.repetition_penalty for s in seqs], device=logits.device)
            pres = torch.tensor([s.params.presence_penalty for s in seqs], device=logits.device)
            freq = torch.tensor([s.params.frequency_penalty for s in seqs], device=logits.device)
            return ref.apply_penalties(logits, counts, rep, pres, freq)
        return proc

    def step(self) -> list[StepOutput]:
        plan, entries = self.sched.schedule()
        if plan is None:
            return []
        want_lp = any(s.params.logprobs for s, _ in entries)
        proc = self._processor(entries)
        if want_lp and proc is None:
            proc = lambda x: x  # noqa: E731 - forces the eager path that keeps logits
        if proc is not None:
            plan.flags |= FLAG_EAGER      # every rank must take the same path: a graph capture runs the step more than once
        patches = self._embed_patches(entries)
        # rows whose embeddings the caller supplied: the other ranks learn where they go with the plan and get the rows after it
        plan.embeds = [(int(r0), int(rows.shape[0])) for r0, rows in patches] if patches else None
        if self.plan_sink is not None:
            self.plan_sink(plan)
            if patches and self.embed_sink is not None:
                self.embed_sink(patches)
        self.exe.model.embed_patches = patches
        if plan.flags & FLAG_NO_SAMPLE:
            # prompt chunks only: nothing to read back, so the host goes straight on to the next chunk while this one
            # runs (and, with pipeline stages, while the later stages still work on it)
            self.exe.run(plan)
            sampled = np.zeros(plan.n_seqs, np.int32)
            want_lp = False
        else:
            ids = self.exe.run(plan, proc)
            sampled = self.exe.fetch(ids)
        lp = None
        if want_lp:
            k = max(1, max(s.params.top_logprobs for s, _ in entries))
            chosen = torch.as_tensor(sampled, device=self.exe.last_logits.device)
            lp = tuple(t.cpu() for t in ref.top_logprobs(self.exe.last_logits[:len(entries)], chosen, k))
        self.n_steps += 1
        outs: list[StepOutput] = []
        for b, (s, tok) in enumerate(self.sched.commit(entries, sampled)):
            o = StepOutput(s.req_id, tok, s.finished, s.finish_reason, len(s.prompt), len(s.output),
                           s.n_cached_prefix, prefill_done=min(s.n_computed, len(s.prompt)))
            if lp is not None and tok is not None and s.params.logprobs:
                row = [e[0].req_id for e in entries].index(s.req_id)
                o.logprob = float(lp[0][row])
                o.top_logprobs = [(int(i), float(v)) for v, i in zip(lp[1][row], lp[2][row])][:s.params.top_logprobs]
            outs.append(o)
            if s.finished:
                self.seqs.pop(s.req_id, None)
        return outs

    def generate(self, prompt: list[int], params: SamplingParams | None = None) -> list[int]:
        """Convenience: run one request to completion and return its generated ids."""
        rid = self.submit(prompt, params, use_prefix_cache=False)
        out: list[int] = []
        while True:
            for o in self.step():
                if o.req_id == rid:
                    if o.token is not None:
                        out.append(o.token)
                    if o.finished:
                        return out

    def warmup(self, n_tokens: int = 8) -> float:
        t0 = time.perf_counter()
        self.generate([1, 2, 3, 4], SamplingParams(temperature=0.0, max_tokens=n_tokens, ignore_eos=True))
        return time.perf_counter() - t0


class FollowerEngine:
    """Non-leader rank: executes the plans the leader broadcasts, keeps no request state."""

    def __init__(self, executor: Executor):
        self.exe = executor

    def run_plan(self, plan: StepPlan) -> None:
        self.exe.run(plan)
