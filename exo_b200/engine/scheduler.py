"""Continuous-batching scheduler with chunked prefill, on paged KV.

Behaviour relative to the reference's batch generator
(``src/exo/worker/runner/llm_inference/batch_generator.py:320-572`` and
``src/exo/worker/engines/mlx/generator/batch_generate.py:104-330``): requests are admitted up
to a concurrency cap (reference: ``EXO_MAX_CONCURRENT_REQUESTS=8``), prompts are prefilled in
chunks of at most ``prefill_chunk`` tokens (reference ``prefill_step_size=4096``), each step
decodes one token for every running sequence.  The difference is that a newcomer's prefill
chunk rides in the *same* step as the running batch's decode tokens (ragged attention), so
admitting a long prompt does not stall the sequences that are already streaming.
"""
from __future__ import annotations

import time
from collections import deque

import numpy as np

from .kv import BlockAllocator, OutOfBlocks, Sequence
from .plan import MAX_STATE_OPS, STATE_RESTORE, STATE_SAVE, StepPlan, FLAG_ALL_GREEDY, FLAG_NO_SAMPLE


class Scheduler:
    def __init__(self, alloc: BlockAllocator, max_seqs: int = 64, prefill_chunk: int = 4096,
                 max_blocks_per_seq: int = 2048, eos_token_ids: tuple[int, ...] = (), max_context: int = 1 << 20,
                 seed: int = 0):
        self.alloc = alloc
        self.max_seqs, self.prefill_chunk = max_seqs, prefill_chunk
        self.max_blocks_per_seq = max_blocks_per_seq
        self.eos = set(eos_token_ids)
        self.max_context = max_context
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.rng = np.random.default_rng(seed)
        self._rngs: dict[str, np.random.Generator] = {}
        self.n_preempted = 0
        # seats 1..max_seqs for per-sequence recurrent state (linear-attention layers); seat 0 is the scratch seat of
        # padding rows.  A sequence holds a seat exactly while it is in `running`.
        self._free_seats = list(range(max_seqs, 0, -1))
        # models with recurrent layers: a cached prefix is only usable up to a block whose end-of-block state was
        # snapshotted (`BlockAllocator.snap_of`); set by the engine when the model has such layers and a snapshot pool
        self.state_snapshots = False

    # ---- request lifecycle ----
    def add(self, seq: Sequence) -> None:
        seq.t_submit = time.perf_counter()
        if seq.params.seed is not None:
            self._rngs[seq.req_id] = np.random.default_rng(seq.params.seed)
        self.waiting.append(seq)

    def cancel(self, req_id: str) -> bool:
        for s in list(self.waiting):
            if s.req_id == req_id:
                self.waiting.remove(s)
                s.finished, s.cancelled, s.finish_reason = True, True, "cancelled"
                return True
        for s in self.running:
            if s.req_id == req_id:
                self._finish(s, "cancelled")
                s.cancelled = True
                return True
        return False

    def _finish(self, s: Sequence, reason: str) -> None:
        s.finished, s.finish_reason = True, reason
        self._publish_full_blocks(s)
        s.final_blocks = list(s.blocks)       # still holds the sequence's KV until the allocator hands them out again
        s.final_seat = s.state_slot            # ... and this seat its recurrent state until another sequence sits there
        self.alloc.release_all(s.blocks)
        s.blocks = []
        if s in self.running:
            self.running.remove(s)
        self._release_seat(s)
        self._rngs.pop(s.req_id, None)

    def _release_seat(self, s: Sequence) -> None:
        if s.state_slot:
            self._free_seats.append(s.state_slot)
            s.state_slot = 0

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- block management ----
    def _ensure_blocks(self, s: Sequence, n_tokens: int) -> bool:
        need = -(-n_tokens // self.alloc.block_size)
        if need > self.max_blocks_per_seq:
            return False
        try:
            while len(s.blocks) < need:
                s.blocks.append(self.alloc.alloc())
        except OutOfBlocks:
            return False
        return True

    def _publish_full_blocks(self, s: Sequence) -> None:
        if not s.use_prefix_cache:
            return
        n_full = s.n_computed // self.alloc.block_size
        if n_full <= s.n_published:
            return
        hashes = self.alloc.block_hashes(s.tokens[:n_full * self.alloc.block_size], s.media)
        for i in range(s.n_published, n_full):
            self.alloc.publish(s.blocks[i], hashes[i])
        s.n_published = n_full

    def _admit(self, s: Sequence) -> bool:
        """Attach cached prefix blocks and allocate the first chunk's blocks."""
        bs = self.alloc.block_size
        if s.n_computed == 0 and s.use_prefix_cache and not s.blocks:
            # never reuse the whole prompt: the last token must be recomputed to get logits
            hashes = self.alloc.block_hashes(s.tokens[:s.n_tokens - 1], s.media)
            got = self.alloc.match_prefix(hashes)
            if self.state_snapshots:
                # keep the longest run of cached blocks that ends in a block with a state snapshot
                keep, snap = 0, None
                for j in range(len(got), 0, -1):
                    snap = self.alloc.snapshot_at(hashes[j - 1])
                    if snap is not None:
                        keep = j
                        break
                self.alloc.release_all(got[keep:])
                got = got[:keep]
                s.restore_snap = snap if keep else None
            s.blocks = got
            s.n_computed = s.n_cached_prefix = len(got) * bs
            s.n_published = len(got)
        return True

    def _snapshot_boundary(self, s: Sequence) -> int:
        """Token count at which a prompt's recurrent state is snapshotted: the last block boundary before the prompt's
        final token (that token is always computed by the request itself).  0: none."""
        if not self.state_snapshots or not s.use_prefix_cache:
            return 0
        bs = self.alloc.block_size
        return ((len(s.prompt) - 1) // bs) * bs

    def _chunk(self, s: Sequence, budget: int) -> int:
        """Tokens of ``s`` to compute this step: up to the budget, and never across its snapshot boundary (the state must
        be taken exactly there)."""
        n = min(s.n_tokens - s.n_computed, budget)
        b = self._snapshot_boundary(s)
        if s.n_computed < b < s.n_computed + n:
            n = b - s.n_computed
        return n

    def _preempt_one(self, keep: Sequence) -> bool:
        """Evict the most recently admitted running sequence (recompute later)."""
        for victim in reversed(self.running):
            if victim is keep:
                continue
            self.alloc.release_all(victim.blocks)
            victim.blocks, victim.n_computed, victim.n_published = [], 0, 0
            victim.restore_snap = None
            # generated tokens become part of the prompt to recompute
            self.running.remove(victim)
            self._release_seat(victim)          # its recurrent state is recomputed with its KV
            self.waiting.appendleft(victim)
            self.n_preempted += 1
            return True
        return False

    # ---- planning ----
    def schedule(self) -> tuple[StepPlan | None, list[tuple[Sequence, int]]]:
        """Pick the work of the next step.  Returns the plan and ``[(seq, n_new_tokens)]``."""
        entries: list[tuple[Sequence, int]] = []
        budget = self.prefill_chunk
        # 1. decode tokens of running sequences (and continuation chunks of running prefills).  Blocks are secured
        #    for every decoding sequence first: making room may preempt a sequence that was looked at earlier in
        #    this very call, so the entries are only built once no further eviction can happen.
        decoding: list[Sequence] = []
        for s in list(self.running):
            if s.in_prefill or s not in self.running:
                continue
            while not self._ensure_blocks(s, s.n_tokens):
                if not self._preempt_one(s):
                    self._finish(s, "length")
                    break
            if s.finished or s not in self.running:
                continue
            decoding.append(s)
        for s in decoding:
            if s in self.running and not s.finished:      # still seated after the later sequences' preemptions
                entries.append((s, 1))
                budget -= 1
        for s in list(self.running):
            if not s.in_prefill or budget <= 0:
                continue
            n = self._chunk(s, budget)
            if not self._ensure_blocks(s, s.n_computed + n):
                continue
            entries.append((s, n))
            budget -= n
        # 2. admit newcomers while there is token budget and a free seat
        while self.waiting and len(self.running) < self.max_seqs and budget > 0:
            s = self.waiting[0]
            if s.n_tokens >= self.max_context:      # after preemption the generated tokens are recomputed as prompt
                self.waiting.popleft()
                s.finished, s.finish_reason = True, "length"
                continue
            self._admit(s)
            n = self._chunk(s, budget)
            if not self._ensure_blocks(s, s.n_computed + n):
                if not self.running and not entries:
                    # cannot ever fit
                    self.waiting.popleft()
                    self.alloc.release_all(s.blocks)
                    s.blocks = []
                    s.finished, s.finish_reason = True, "length"
                    continue
                break
            self.waiting.popleft()
            s.t_prefill_start = time.perf_counter()
            if not s.state_slot:                   # (a sequence whose prompt state was installed from elsewhere already sits)
                s.state_slot = self._free_seats.pop() if self._free_seats else 0
            self.running.append(s)
            entries.append((s, n))
            budget -= n
        if not entries:
            return None, []
        return self._build_plan(entries), entries

    def _uniform(self, s: Sequence) -> float:
        g = self._rngs.get(s.req_id, self.rng)
        return float(g.random())

    def _build_plan(self, entries: list[tuple[Sequence, int]]) -> StepPlan:
        bs = self.alloc.block_size
        B = len(entries)
        T = sum(n for _, n in entries)
        max_blocks = max(len(s.blocks) for s, _ in entries)
        tokens = np.empty(T, np.int32)
        positions = np.empty(T, np.int32)
        slots = np.empty(T, np.int32)
        cu_q = np.zeros(B + 1, np.int32)
        seq_lens = np.empty(B, np.int32)
        logit_rows = np.full(B, -1, np.int32)
        top_k = np.zeros(B, np.int32)
        temp = np.zeros(B, np.float32)
        top_p = np.ones(B, np.float32)
        min_p = np.zeros(B, np.float32)
        uni = np.zeros(B, np.float32)
        bt = np.zeros((B, max_blocks), np.int32)
        t = 0
        all_greedy = True
        samples = False
        for b, (s, n) in enumerate(entries):
            lo = s.n_computed
            blk = s.blocks_array()
            if n == 1:                   # decode row: no temporaries
                tokens[t] = s.token_at(lo)
                positions[t] = lo
                slots[t] = int(blk[lo // bs]) * bs + lo % bs
            else:
                tokens[t:t + n] = s.token_span(lo, lo + n)
                pos = np.arange(lo, lo + n, dtype=np.int32)
                positions[t:t + n] = pos
                slots[t:t + n] = blk[pos // bs] * bs + pos % bs
            cu_q[b + 1] = t + n
            seq_lens[b] = lo + n
            if lo + n == s.n_tokens:  # the step reaches the sequence's last token → sample
                samples = True
                logit_rows[b] = t + n - 1
                p = s.params
                temp[b], top_p[b], min_p[b], top_k[b] = p.temperature, p.top_p, p.min_p, p.top_k
                if not p.greedy:
                    all_greedy = False
                    uni[b] = self._uniform(s)
            bt[b, :len(blk)] = blk
            t += n
        ops: list[tuple[int, int, int]] = []
        if self.state_snapshots:
            for s, n in entries:
                if s.restore_snap is not None and len(ops) < MAX_STATE_OPS:
                    ops.append((STATE_RESTORE, s.state_slot, s.restore_snap))
                s.restore_snap = None
            for s, n in entries:
                b = self._snapshot_boundary(s)
                if b >= bs and s.n_computed < b == s.n_computed + n and s.state_slot and len(ops) < MAX_STATE_OPS:
                    sid = self.alloc.reserve_snapshot(self.alloc.block_hashes(s.tokens[:b], s.media)[-1])
                    if sid is not None:
                        ops.append((STATE_SAVE, s.state_slot, sid))
        return StepPlan(n_tokens=T, n_seqs=B, max_q_len=max(n for _, n in entries), state_ops=tuple(ops),
                        flags=(FLAG_ALL_GREEDY if all_greedy else 0) | (0 if samples else FLAG_NO_SAMPLE), tokens=tokens, positions=positions, slots=slots,
                        cu_q=cu_q, seq_lens=seq_lens, logit_rows=logit_rows, top_k=top_k, temperature=temp,
                        top_p=top_p, min_p=min_p, uniform=uni, prev_rows=np.full(B, -1, np.int32), block_tables=bt,
                        req_ids=tuple(s.req_id for s, _ in entries),
                        state_slots=np.fromiter((s.state_slot for s, _ in entries), np.int32, B))

    # ---- results ----
    def commit(self, entries: list[tuple[Sequence, int]], sampled: np.ndarray) -> list[tuple[Sequence, int | None]]:
        """Account for an executed step.  ``sampled[b]`` is the token drawn for entry ``b``
        (ignored where the entry was a non-final prefill chunk).  Returns ``(seq, new token)``."""
        now = time.perf_counter()
        out: list[tuple[Sequence, int | None]] = []
        for b, (s, n) in enumerate(entries):
            if s.finished:
                continue
            s.n_computed += n
            self._publish_full_blocks(s)
            if s.n_computed < s.n_tokens:
                out.append((s, None))  # still prefilling
                continue
            tok = int(sampled[b])
            s.output.append(tok)
            if len(s.output) == 1:
                s.t_first_token = now
            s.t_last_token = now
            out.append((s, tok))
            p = s.params
            if not p.ignore_eos and (tok in self.eos or tok in p.stop_token_ids):
                self._finish(s, "stop")
            elif len(s.output) >= p.max_tokens or s.n_tokens >= self.max_context:
                self._finish(s, "length")
        return out
