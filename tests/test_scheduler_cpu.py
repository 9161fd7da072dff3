"""Scheduler behaviour under KV pressure (host only)."""
import numpy as np

from exo_b200.engine.kv import BlockAllocator, SamplingParams, Sequence
from exo_b200.engine.scheduler import Scheduler


def _run_step(sched):
    plan, entries = sched.schedule()
    if plan is None:
        return None, []
    # every entry's slots must lie inside blocks the sequence owns at plan time
    t = 0
    for b, (s, n) in enumerate(entries):
        assert s.blocks, "a scheduled sequence must hold blocks"
        owned = set(s.blocks)
        for slot in plan.slots[t:t + n]:
            assert int(slot) // sched.alloc.block_size in owned
        t += n
    sched.commit(entries, np.full(len(entries), 7, np.int64))
    return plan, entries


def test_preempting_a_sequence_already_looked_at_this_step_drops_its_entry():
    """Three blocks of 16 tokens.  A (5-token prompt) decodes next to B (31-token prompt); when B needs its third
    block, A — examined earlier in the same scheduling pass — is the only possible victim.  The step must go on
    without A instead of carrying a stale entry for a sequence that no longer owns blocks."""
    alloc = BlockAllocator(3, 16)
    sched = Scheduler(alloc, max_seqs=4, prefill_chunk=64, max_blocks_per_seq=8)
    greedy = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
    a = Sequence("a", list(range(5)), greedy, use_prefix_cache=False)
    b = Sequence("b", list(range(31)), greedy, use_prefix_cache=False)
    sched.add(a)
    sched.add(b)
    for _ in range(12):
        plan, entries = _run_step(sched)
        if plan is None:
            break
        ids = [s.req_id for s, _ in entries]
        assert len(ids) == len(set(ids))
    assert sched.n_preempted >= 1
    # the preempted sequence is either waiting to be recomputed or running again with blocks of its own
    for s in (a, b):
        if not s.finished and s in sched.running:
            assert s.blocks


def test_block_pool_is_conserved_across_preemption_and_finish():
    alloc = BlockAllocator(4, 16)
    sched = Scheduler(alloc, max_seqs=4, prefill_chunk=32, max_blocks_per_seq=8)
    p = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    for i, n in enumerate((5, 17, 30)):
        sched.add(Sequence(f"s{i}", list(range(n)), p, use_prefix_cache=False))
    for _ in range(400):
        if not sched.has_work:
            break
        _run_step(sched)
    assert not sched.has_work
    assert alloc.n_free == 4 and all(r == 0 for r in alloc.ref)


def test_state_seats_are_distinct_while_running_and_return_on_finish_and_preemption():
    """Every running sequence holds its own seat (1..max_seqs; 0 is the scratch seat of padding rows) for its recurrent
    state; the plan carries the seats row by row; a finished or preempted sequence gives its seat back."""
    alloc = BlockAllocator(4, 16)
    sched = Scheduler(alloc, max_seqs=3, prefill_chunk=32, max_blocks_per_seq=8)
    p = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    for i, n in enumerate((5, 17, 30)):
        sched.add(Sequence(f"s{i}", list(range(n)), p, use_prefix_cache=False))
    seen = set()
    for _ in range(400):
        if not sched.has_work:
            break
        plan, entries = _run_step(sched)
        if plan is None:
            continue
        seats = [s.state_slot for s in sched.running]
        assert all(1 <= x <= 3 for x in seats) and len(set(seats)) == len(seats)
        assert list(plan.state_slots[:len(entries)]) == [s.state_slot or plan.state_slots[i] for i, (s, _) in enumerate(entries)]
        assert all(1 <= int(x) <= 3 for x in plan.state_slots[:len(entries)])
        seen.update(int(x) for x in plan.state_slots[:len(entries)])
        for s in sched.waiting:
            assert s.state_slot == 0
    assert not sched.has_work and sched.n_preempted >= 1
    assert sorted(sched._free_seats) == [1, 2, 3] and len(seen) >= 2


def test_prompt_chunks_short_of_the_end_carry_the_no_sample_flag_and_skip_the_read_back():
    """A 100-token prompt in chunks of 32: the first three steps neither project logits nor read ids back; the fourth
    (which reaches the last prompt token) samples.  A decode row riding along makes the step sample again."""
    import torch

    from exo_b200.engine.engine import Engine
    from exo_b200.engine.plan import FLAG_NO_SAMPLE
    from exo_b200.models.config import preset
    from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
    alloc = BlockAllocator(32, 16)
    sched = Scheduler(alloc, max_seqs=4, prefill_chunk=32, max_blocks_per_seq=16)
    greedy = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    sched.add(Sequence("long", list(range(100)), greedy, use_prefix_cache=False))
    flags = []
    for _ in range(5):
        plan, _ = _run_step(sched)
        flags.append(bool(plan.flags & FLAG_NO_SAMPLE))
    assert flags == [True, True, True, False, False]
    # through the engine: the fetches counted are those of sampling steps only, and the tokens equal a one-chunk run
    cfg = preset("tiny-llama")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cpu")
    prompt = [int(t) for t in torch.randint(0, cfg.vocab, (100,), generator=torch.Generator().manual_seed(3))]
    chunked = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=32)
    whole = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=256)
    a = chunked.generate(prompt, greedy)
    assert a == whole.generate(prompt, greedy)
    assert chunked.n_steps == 3 + 4 and chunked.exe.d2h_bytes == 4 * 4 and whole.exe.d2h_bytes == 4 * 4


def test_state_snapshots_follow_their_blocks_and_age_out():
    """A snapshot belongs to the cached block whose end it describes: it disappears with that block, the least recently
    used one gives way when the pool is full, and a prefix is only matched up to a block that has one."""
    alloc = BlockAllocator(4, 16)
    alloc.enable_snapshots(2)
    toks = list(range(64))
    h = alloc.block_hashes(toks)
    blocks = [alloc.alloc() for _ in range(3)]
    for b, hh in zip(blocks, h):
        alloc.publish(b, hh)
    assert alloc.reserve_snapshot(h[0]) == 0 and alloc.reserve_snapshot(h[1]) == 1
    assert alloc.reserve_snapshot(h[0]) is None                      # exists already
    assert alloc.snapshot_at(h[0]) == 0                              # ... and is now the most recently used
    assert alloc.reserve_snapshot(h[2]) == 1 and alloc.snapshot_at(h[1]) is None      # the pool was full: h[1]'s gave way
    # scheduler side: three cached blocks, snapshots at the ends of blocks 0 and 2 only
    sched = Scheduler(alloc, max_seqs=2, prefill_chunk=64, max_blocks_per_seq=8)
    sched.state_snapshots = True
    alloc.release_all(blocks)
    s = Sequence("a", toks[:40] + [999] * 9, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    sched.add(s)
    plan, entries = sched.schedule()
    assert s.n_cached_prefix == 16 and plan.state_ops[0] == (1, s.state_slot, 0)       # block 1 has no snapshot: stop at block 0
    assert plan.n_tokens == 48 - 16                                  # and the chunk ends at this prompt's own boundary (48)
    # evicting a cached block takes its snapshot along
    alloc2 = BlockAllocator(1, 16)
    alloc2.enable_snapshots(1)
    b = alloc2.alloc()
    alloc2.publish(b, h[0])
    assert alloc2.reserve_snapshot(h[0]) == 0
    alloc2.release(b)
    assert alloc2.alloc() == b and alloc2.snapshot_at(h[0]) is None and alloc2.free_snaps == [0]
