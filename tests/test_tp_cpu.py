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


# One row per checkpoint family / block feature the engine shards (the reference's counterpart is its table of tiny
# random-init configs, ``src/exo/worker/tests/unittests/test_mlx/test_tp_bit_exact.py:15-307``): Llama, Qwen2 (biases,
# tied embeddings), Qwen3 (q/k norm), Qwen3-MoE, DeepSeek-V3 / Kimi / GLM-MoE-Lite (MLA + sigmoid experts), GLM-4.x-MoE
# (half-rotary, biases, shared expert), Mixtral (block_sparse_moe), MiniMax (q/k norm over all heads: a cross-rank
# statistic; KV heads replicated at 4 ranks), GPT-OSS attention (sinks + sliding window), YaRN.
FAMILIES = [("tiny-llama", 2), ("tiny-llama", 4), ("tiny-moe", 2), ("tiny-mla", 2), ("tiny-mla", 4), ("tiny-qwen3", 2),
            ("tiny-qwen2", 2), ("tiny-glm4-moe", 2), ("tiny-glm4-moe", 4), ("tiny-mixtral", 2), ("tiny-mixtral", 4),
            ("tiny-minimax", 2), ("tiny-minimax", 4), ("tiny-gpt-oss", 2), ("tiny-yarn", 2),
            ("tiny-qwen3-next", 2),     # gated-delta-rule heads split by key-head group, state per rank
            ("tiny-gemma4", 2),         # per-layer head sizes, one global KV head on two ranks, replicated per-layer inputs
            ("tiny-nemotron-h", 2),     # Mamba-2 heads and groups split, relu^2 experts whole, shared expert sliced
            ("tiny-step3p5", 2)]        # per-layer query-head counts and RoPE, head gates split with the heads, clamped SwiGLU


@pytest.mark.parametrize("name,world", FAMILIES)
def test_tp_ranks_reproduce_oracle_tokens(name, world):
    cfg = preset(name)
    prompt = oracle_prompt(48, cfg.vocab, seed=11).tolist()
    if cfg.family in ("gemma4", "nemotron_h"):      # the oracle model has no such block (the library is its oracle): compare with one rank
        from exo_b200.engine.engine import Engine
        from exo_b200.engine.kv import SamplingParams
        from exo_b200.models.weights import ShardSpec, build_weights
        want = Engine(cfg, build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cpu"), n_blocks=32, device="cpu").generate(
            prompt, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    else:
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


def _pp_worker(rank, world, port, name, pp, prompt, n_new, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from exo_b200.engine.engine import Engine
        from exo_b200.engine.kv import SamplingParams
        from exo_b200.parallel.comm import GlooComm, PipeComm
        cfg = preset(name)
        tp = world // pp
        pp_rank, tp_rank = divmod(rank, tp)
        # every rank creates every group, in the same order
        tp_groups = [dist.new_group([s * tp + t for t in range(tp)]) for s in range(pp)]
        lane_groups = [dist.new_group([s * tp + t for s in range(pp)]) for t in range(tp)]
        per = cfg.n_layers // pp
        spec = ShardSpec(tp_rank=tp_rank, tp_size=tp, pp_rank=pp_rank, pp_size=pp, layer_start=pp_rank * per,
                         layer_end=cfg.n_layers if pp_rank == pp - 1 else (pp_rank + 1) * per)
        w = build_weights(cfg, spec, RandomSource(seed=0))
        comm = GlooComm(tp_groups[pp_rank]) if tp > 1 else None
        pipe = PipeComm(pp_rank, pp, tp_rank, tp, lane_groups[tp_rank])
        eng = Engine(cfg, w, spec, comm, n_blocks=64, pipe=pipe, prefill_chunk=32)
        out = eng.generate(prompt, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
        if rank == 0:
            q.put((out, pipe.n_hops))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,world,pp", [("tiny-llama", 2, 2), ("tiny-llama", 4, 2), ("tiny-moe", 2, 2)])
def test_pipeline_stages_reproduce_oracle_tokens(name, world, pp):
    """PP2 and PP2 x TP2: stages own contiguous layer ranges, the residual stream hops stage to
    stage (chunked prefill of 48 tokens in 32-token chunks, then decode), ids come back to rank 0."""
    cfg = preset(name)
    prompt = oracle_prompt(48, cfg.vocab, seed=11).tolist()
    if cfg.family in ("gemma4", "nemotron_h"):      # the oracle model has no such block (the library is its oracle): compare with one rank
        from exo_b200.engine.engine import Engine
        from exo_b200.engine.kv import SamplingParams
        from exo_b200.models.weights import ShardSpec, build_weights
        want = Engine(cfg, build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cpu"), n_blocks=32, device="cpu").generate(
            prompt, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    else:
        want = OracleModel(cfg, RandomSource(seed=0)).greedy(torch.tensor(prompt), 10)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, world, port, name, pp, prompt, 10, q)) for r in range(world)]
    for p in procs:
        p.start()
    got, hops = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
    assert hops == 2 + 9      # first stage: one send per step (2 prefill chunks + 9 decode steps after the first token)
