"""StepPlan: the complete, self-contained description of one engine step.

A plan is produced once per step by the scheduler (on the controller / rank 0) and is all a
GPU rank needs to execute that step — ranks keep no per-request state.  This replaces the
reference's per-step cross-rank agreement collectives (task-id all-gather, cancel all-sum,
barriers: ``src/exo/worker/engines/mlx/utils_mlx.py:833-938``,
``src/exo/worker/runner/llm_inference/batch_generator.py:375-398``) with one host-side
broadcast of a packed int32 buffer.

Packed layout (int32 words): ``[T, B, R, max_q_len, flags, bucket_T, bucket_B, max_blocks]``
then ``tokens[T'] positions[T'] slots[T'] cu_q[B'+1] seq_lens[B'] logit_rows[B']
top_k[B'] temperature[B'] top_p[B'] min_p[B'] uniform[B'] prev_rows[B'] state_slots[B'] block_tables[B'*max_blocks]
state_ops[1 + 3*MAX_STATE_OPS]`` (count, then ``kind, seat, snapshot`` triples: host-side instructions to copy recurrent state
between sequence seats and prefix-cache snapshots around the step) where
``T'``/``B'`` are the padded (bucket) sizes, floats are bit-cast.  Padding rows point at the
reserved scratch block 0 so that a graph captured for the bucket runs unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

HEADER = 8
FLAG_TOKENS_FROM_PREV = 1  # decode: take input tokens from the previous step's samples on device
FLAG_ALL_GREEDY = 2
FLAG_EAGER = 4             # the leader runs this step outside its CUDA graphs (logits processors): followers do the same
FLAG_NO_SAMPLE = 8         # every row is a prompt chunk that stops short of its sequence's end: no logits, no ids, no read-back
MAX_STATE_OPS = 32
STATE_RESTORE, STATE_SAVE = 1, 2   # snapshot -> seat before the step's kernels; seat -> snapshot after them


@dataclass
class PlanLayout:
    """Word offsets of each array inside the packed buffer for given bucket sizes."""
    T: int
    B: int
    max_blocks: int

    def __post_init__(self) -> None:
        o = HEADER
        self.tokens = o; o += self.T
        self.positions = o; o += self.T
        self.slots = o; o += self.T
        self.cu_q = o; o += self.B + 1
        self.seq_lens = o; o += self.B
        self.logit_rows = o; o += self.B
        self.top_k = o; o += self.B
        self.temperature = o; o += self.B
        self.top_p = o; o += self.B
        self.min_p = o; o += self.B
        self.uniform = o; o += self.B
        self.prev_rows = o; o += self.B
        self.state_slots = o; o += self.B
        o = (o + 3) // 4 * 4  # keep the table 16-byte aligned
        self.block_tables = o; o += self.B * self.max_blocks
        self.state_ops = o; o += 1 + 3 * MAX_STATE_OPS
        self.words = o


@dataclass
class StepPlan:
    """Host-side (numpy) step description; ``n_tokens``/``n_seqs`` are the unpadded sizes."""
    n_tokens: int
    n_seqs: int
    max_q_len: int
    flags: int
    tokens: np.ndarray        # [T] int32
    positions: np.ndarray     # [T] int32
    slots: np.ndarray         # [T] int32
    cu_q: np.ndarray          # [B+1] int32
    seq_lens: np.ndarray      # [B] int32
    logit_rows: np.ndarray    # [B] int32 (-1 → this sequence wants no logits this step)
    top_k: np.ndarray         # [B] int32
    temperature: np.ndarray   # [B] float32
    top_p: np.ndarray         # [B] float32
    min_p: np.ndarray         # [B] float32
    uniform: np.ndarray       # [B] float32
    prev_rows: np.ndarray     # [B] int32 row of the previous step's samples feeding this row (-1: use tokens)
    block_tables: np.ndarray  # [B, max_blocks] int32
    req_ids: tuple[str, ...] = ()
    state_slots: np.ndarray | None = None   # [B] int32 seat of each sequence's recurrent state (0: none / padding rows)
    state_ops: tuple[tuple[int, int, int], ...] = ()   # (STATE_RESTORE | STATE_SAVE, seat, snapshot)

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1

    def pack(self, out: np.ndarray, bucket_T: int, bucket_B: int, max_blocks: int) -> PlanLayout:
        """Serialise into ``out`` (int32, >= layout.words) padded to the bucket sizes."""
        L = PlanLayout(bucket_T, bucket_B, max_blocks)
        T, B = self.n_tokens, self.n_seqs
        assert T <= bucket_T and B <= bucket_B and self.block_tables.shape[1] <= max_blocks
        out[:L.words] = 0
        out[0:HEADER] = (T, B, B, self.max_q_len, self.flags, bucket_T, bucket_B, max_blocks)
        out[L.tokens:L.tokens + T] = self.tokens
        out[L.positions:L.positions + T] = self.positions
        out[L.slots:L.slots + T] = self.slots
        # padded tokens write their KV into scratch block 0 (slots 0..block_size-1 are never read)
        out[L.cu_q:L.cu_q + B + 1] = self.cu_q
        if bucket_B > B:
            # padded sequences: one query token each when decoding (graph shape), else empty
            if self.max_q_len == 1 and bucket_T == bucket_B:
                out[L.cu_q + B + 1:L.cu_q + bucket_B + 1] = np.arange(T + 1, T + 1 + bucket_B - B, dtype=np.int32)
                out[L.seq_lens + B:L.seq_lens + bucket_B] = 1
            else:
                out[L.cu_q + B + 1:L.cu_q + bucket_B + 1] = T
        out[L.seq_lens:L.seq_lens + B] = self.seq_lens
        out[L.logit_rows:L.logit_rows + B] = np.maximum(self.logit_rows, 0)
        out[L.top_k:L.top_k + B] = self.top_k
        fv = out.view(np.float32)
        fv[L.temperature:L.temperature + B] = self.temperature
        fv[L.top_p:L.top_p + B] = self.top_p
        fv[L.top_p + B:L.top_p + bucket_B] = 1.0
        fv[L.min_p:L.min_p + B] = self.min_p
        fv[L.uniform:L.uniform + B] = self.uniform
        out[L.prev_rows:L.prev_rows + bucket_B] = -1
        out[L.prev_rows:L.prev_rows + B] = self.prev_rows
        if self.state_slots is not None:
            out[L.state_slots:L.state_slots + B] = self.state_slots
        bt = out[L.block_tables:L.block_tables + bucket_B * max_blocks].reshape(bucket_B, max_blocks)
        bt[:B, :self.block_tables.shape[1]] = self.block_tables
        assert len(self.state_ops) <= MAX_STATE_OPS
        out[L.state_ops] = len(self.state_ops)
        for j, op in enumerate(self.state_ops):
            out[L.state_ops + 1 + 3 * j:L.state_ops + 4 + 3 * j] = op
        return L

    @staticmethod
    def unpack(buf: np.ndarray) -> "StepPlan":
        T, B, _, mq, flags, bT, bB, mb = (int(x) for x in buf[:HEADER])
        L = PlanLayout(bT, bB, mb)
        fv = buf.view(np.float32)
        return StepPlan(
            n_tokens=T, n_seqs=B, max_q_len=mq, flags=flags,
            tokens=buf[L.tokens:L.tokens + T].copy(), positions=buf[L.positions:L.positions + T].copy(),
            slots=buf[L.slots:L.slots + T].copy(), cu_q=buf[L.cu_q:L.cu_q + B + 1].copy(),
            seq_lens=buf[L.seq_lens:L.seq_lens + B].copy(), logit_rows=buf[L.logit_rows:L.logit_rows + B].copy(),
            top_k=buf[L.top_k:L.top_k + B].copy(), temperature=fv[L.temperature:L.temperature + B].copy(),
            top_p=fv[L.top_p:L.top_p + B].copy(), min_p=fv[L.min_p:L.min_p + B].copy(),
            uniform=fv[L.uniform:L.uniform + B].copy(), prev_rows=buf[L.prev_rows:L.prev_rows + B].copy(),
            block_tables=buf[L.block_tables:L.block_tables + bB * mb].reshape(bB, mb)[:B].copy(),
            state_slots=buf[L.state_slots:L.state_slots + B].copy(),
            state_ops=tuple(tuple(int(x) for x in buf[L.state_ops + 1 + 3 * j:L.state_ops + 4 + 3 * j])
                            for j in range(int(buf[L.state_ops]))))


def bucket(n: int, buckets: tuple[int, ...]) -> int:
    for b in buckets:
        if n <= b:
            return b
    return n
