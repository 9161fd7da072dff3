"""Host-side guards between the leader's block allocator and every rank's KV pool."""
import os
import socket

import numpy as np
import pytest
import torch

from exo_b200.engine.executor import Executor
from exo_b200.engine.plan import FLAG_ALL_GREEDY, StepPlan
from exo_b200.models.config import preset
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights


def _plan(slot: int, block: int) -> StepPlan:
    one = np.ones(1, np.float32)
    return StepPlan(n_tokens=1, n_seqs=1, max_q_len=1, flags=FLAG_ALL_GREEDY, tokens=np.array([3], np.int32),
                    positions=np.array([0], np.int32), slots=np.array([slot], np.int32), cu_q=np.array([0, 1], np.int32),
                    seq_lens=np.array([1], np.int32), logit_rows=np.array([0], np.int32), top_k=np.zeros(1, np.int32),
                    temperature=0 * one, top_p=one, min_p=0 * one, uniform=0 * one, prev_rows=np.array([-1], np.int32),
                    block_tables=np.array([[block]], np.int32))


def test_executor_rejects_plans_that_address_storage_outside_its_pool():
    cfg = preset("tiny-llama")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0))
    exe = Executor(cfg, w, n_blocks=8, block_size=16, max_blocks_per_seq=4, max_tokens_per_step=32, max_seqs=4)
    exe.run(_plan(slot=16, block=1))                      # inside the pool
    with pytest.raises(ValueError, match="slot"):
        exe.run(_plan(slot=8 * 16, block=1))               # first slot past the pool
    with pytest.raises(ValueError, match="block"):
        exe.run(_plan(slot=16, block=8))


def _agree(rank, world, port, q):
    import torch.distributed as dist
    from exo_b200.worker.engines.b200.bringup import B200Builder, PlanChannel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b = object.__new__(B200Builder)
    b.world, b.control = world, PlanChannel(dist.group.WORLD, rank)
    q.put((rank, b._agree_min(500 - 120 * rank)))          # rank 1 has room for fewer blocks
    dist.destroy_process_group()


def test_ranks_with_different_memory_budgets_agree_on_the_smallest_block_count():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_agree, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got == {0: 380, 1: 380}
