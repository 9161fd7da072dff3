"""Paged-KV bookkeeping on the host: block allocator and block-hash prefix cache.

The reference keeps one contiguous, growing KV cache per sequence and a prefix cache of
deep-copied caches matched by longest common token prefix
(``src/exo/worker/engines/mlx/cache.py:232-470``: LRU eviction under memory pressure,
exact-hit keeps the last token, media-region hashes invalidate matches).  Here KV lives in
fixed 16-token blocks; a full block is identified by the hash chain of the tokens up to and
including it (plus any media hashes covering it), so prefix reuse is a block-table lookup
and costs no copy.  Blocks are reference counted; cached blocks with no user sit in an LRU
and are reclaimed when the allocator runs dry.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field


class OutOfBlocks(RuntimeError):
    pass


class BlockAllocator:
    def __init__(self, n_blocks: int, block_size: int = 16):
        self.n_blocks, self.block_size = n_blocks, block_size
        self.free: list[int] = list(range(n_blocks - 1, -1, -1))
        self.ref = [0] * n_blocks
        # prefix cache: chain hash -> block, and reverse map
        self.by_hash: dict[bytes, int] = {}
        self.hash_of: dict[int, bytes] = {}
        self.lru: OrderedDict[int, None] = OrderedDict()  # cached, unreferenced blocks (oldest first)
        self.hits = 0
        self.queries = 0
        # recurrent-state snapshots of hybrid models: the state of a sequence at the END of a cached block, keyed by that
        # block's chain hash (a prefix can only be reused up to a block that has one); least recently used first
        self.snap_of: OrderedDict[bytes, int] = OrderedDict()
        self.free_snaps: list[int] = []

    # ---- allocation ----
    @property
    def n_free(self) -> int:
        return len(self.free) + len(self.lru)

    def alloc(self) -> int:
        if self.free:
            b = self.free.pop()
        elif self.lru:
            b, _ = self.lru.popitem(last=False)
            h = self.hash_of.pop(b)
            del self.by_hash[h]
            self._drop_snapshot(h)
        else:
            raise OutOfBlocks("KV pool exhausted")
        self.ref[b] = 1
        return b

    def incref(self, b: int) -> None:
        if self.ref[b] == 0:
            self.lru.pop(b, None)
        self.ref[b] += 1

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        assert self.ref[b] >= 0
        if self.ref[b] == 0:
            if b in self.hash_of:
                self.lru[b] = None
            else:
                self.free.append(b)

    def release_all(self, blocks: list[int]) -> None:
        for b in blocks:
            self.release(b)

    # ---- prefix cache ----
    @staticmethod
    def chain_hash(prev: bytes, tokens: list[int], extra: bytes = b"") -> bytes:
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(b"".join(int(t).to_bytes(4, "little", signed=False) for t in tokens))
        h.update(extra)
        return h.digest()

    def block_hashes(self, tokens: list[int], media: list[tuple[int, int, bytes]] | None = None) -> list[bytes]:
        """Hash chain over the full blocks of ``tokens``; ``media`` = (start, end, content hash)
        spans whose hash is mixed into every block they overlap."""
        bs, out, prev = self.block_size, [], b""
        for i in range(len(tokens) // bs):
            extra = b""
            if media:
                for s, e, mh in media:
                    if s < (i + 1) * bs and e > i * bs:
                        extra += mh
            prev = self.chain_hash(prev, tokens[i * bs:(i + 1) * bs], extra)
            out.append(prev)
        return out

    def match_prefix(self, hashes: list[bytes]) -> list[int]:
        """Longest run of cached blocks for the hash chain; increfs what it returns."""
        self.queries += 1
        got: list[int] = []
        for h in hashes:
            b = self.by_hash.get(h)
            if b is None:
                break
            self.incref(b)
            got.append(b)
        if got:
            self.hits += 1
        return got

    def publish(self, block: int, h: bytes) -> int:
        """Register a now-full block.  If an identical block is cached already the caller's
        block stays private (no dedupe of live blocks) and the cached one is kept."""
        if h in self.by_hash or block in self.hash_of:
            return self.by_hash.get(h, block)
        self.by_hash[h] = block
        self.hash_of[block] = h
        return block

    def clear_cache(self) -> None:
        for b in list(self.lru):
            self.lru.pop(b)
            h = self.hash_of.pop(b)
            del self.by_hash[h]
            self.free.append(b)
        for b, h in list(self.hash_of.items()):
            del self.by_hash[h]
            del self.hash_of[b]
        for h in list(self.snap_of):
            self._drop_snapshot(h)

    # ---- recurrent-state snapshots ----
    def enable_snapshots(self, n: int) -> None:
        self.free_snaps = list(range(n - 1, -1, -1))

    def _drop_snapshot(self, h: bytes) -> None:
        sid = self.snap_of.pop(h, None)
        if sid is not None:
            self.free_snaps.append(sid)

    def snapshot_at(self, h: bytes) -> int | None:
        """Snapshot holding the state at the end of the block with chain hash ``h`` (refreshes its age)."""
        sid = self.snap_of.get(h)
        if sid is not None:
            self.snap_of.move_to_end(h)
        return sid

    def reserve_snapshot(self, h: bytes) -> int | None:
        """A snapshot id for the state at the end of block ``h``: ``None`` if one exists already or none can be had;
        the least recently used snapshot gives way when the pool is full."""
        if h in self.snap_of:
            return None
        if self.free_snaps:
            sid = self.free_snaps.pop()
        elif self.snap_of:
            _, sid = self.snap_of.popitem(last=False)
        else:
            return None
        self.snap_of[h] = sid
        return sid

    def usage(self) -> float:
        return 1.0 - len(self.free) / max(1, self.n_blocks)


@dataclass
class SamplingParams:
    """Per-request decoding controls; defaults follow the reference's sampler
    (``src/exo/worker/engines/mlx/generator/generate.py:614-619``: temp 0.7, top_p 1.0,
    min_p 0.05, top_k 0)."""
    temperature: float = 0.7
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.05
    max_tokens: int = 256
    stop_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False  # bench mode: EOS banned so exactly max_tokens are produced
    seed: int | None = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logprobs: bool = False
    top_logprobs: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


@dataclass(eq=False)          # identity semantics: sequences live in lists that are searched every step
class Sequence:
    req_id: str
    prompt: list[int]
    params: SamplingParams
    media: list[tuple[int, int, bytes]] | None = None
    use_prefix_cache: bool = True
    output: list[int] = field(default_factory=list)
    blocks: list[int] = field(default_factory=list)
    n_computed: int = 0          # tokens whose KV is in the cache
    n_cached_prefix: int = 0     # of which came from the prefix cache
    n_published: int = 0         # full blocks already registered in the prefix cache
    finished: bool = False
    finish_reason: str | None = None
    embeds: list | None = None   # [(first prompt position, rows [n, hidden])]: input embeddings that replace the token embeddings (vision)
    cancelled: bool = False
    t_submit: float = 0.0
    t_first_token: float = 0.0
    t_last_token: float = 0.0
    t_prefill_start: float = 0.0
    rng_state: int = 0
    final_blocks: list[int] = field(default_factory=list)   # block ids at the moment the sequence finished
    state_slot: int = 0          # seat of the sequence's recurrent state while it is running (0: none)
    final_seat: int = 0          # the seat at the moment the sequence finished
    restore_snap: int | None = None   # snapshot to copy into the seat before the sequence's first step (prefix reuse)

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    def token_at(self, i: int) -> int:
        n = len(self.prompt)
        return self.prompt[i] if i < n else self.output[i - n]

    def token_span(self, lo: int, hi: int) -> list[int]:
        """Tokens ``[lo, hi)`` of prompt + output without building the concatenated list."""
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.output[lo - n:hi - n]
        return self.prompt[lo:] + self.output[:hi - n]

    def blocks_array(self):
        """``blocks`` as an int32 array.  Rebuilt when the list object was replaced (admission, preemption) or has
        grown (one block every block_size tokens); the list is never edited in the middle."""
        import numpy as np
        c = self.__dict__.get("_blk_np")
        if c is None or c[0] is not self.blocks or c[1].shape[0] != len(self.blocks):
            c = (self.blocks, np.asarray(self.blocks, np.int32))
            self.__dict__["_blk_np"] = c
        return c[1]

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def in_prefill(self) -> bool:
        return self.n_tokens - self.n_computed > 1
