"""Tensor/expert-parallel sharding on CPU ranks (gloo, world size 2 and 4) against the oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from exo_b200.models.config import preset
from exo_b200.models.oracle import OracleModel, oracle_prompt
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, prompt, n_new, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from exo_b200.engine.engine import Engine
        from exo_b200.engine.kv import SamplingParams
        from exo_b200.parallel.comm import GlooComm
        cfg = preset(name)
        spec = ShardSpec(tp_rank=rank, tp_size=world)
        w = build_weights(cfg, spec, RandomSource(seed=0))
        eng = Engine(cfg, w, spec, GlooComm(), n_blocks=64)
        out = eng.generate(prompt, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
        if rank == 0:
            q.put(out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,world", [("tiny-llama", 2), ("tiny-llama", 4), ("tiny-moe", 2), ("tiny-mla", 2)])
def test_tp_ranks_reproduce_oracle_tokens(name, world):
    cfg = preset(name)
    prompt = oracle_prompt(48, cfg.vocab, seed=11).tolist()
    want = OracleModel(cfg, RandomSource(seed=0)).greedy(torch.tensor(prompt), 10)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, name, prompt, 10, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
