"""End-to-end engine on a GPU: oracle equality in fp32, bf16 self-consistency, CUDA-graph decode."""
import pytest
import torch

from exo_b200.models.config import ModelConfig, RopeConfig, preset
from exo_b200.models.oracle import run_oracle, OracleModel, oracle_prompt
from exo_b200.models.weights import RandomSource, ShardSpec, build_weights, fast_random_weights
from exo_b200.engine.engine import Engine
from exo_b200.engine.kv import SamplingParams

pytestmark = pytest.mark.gpu
GREEDY = dict(temperature=0.0, ignore_eos=True)


def test_tiny_llama_fp32_gpu_matches_cpu_oracle():
    golden = run_oracle(128, 64)
    cfg = preset("tiny-llama")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cuda")
    eng = Engine(cfg, w, n_blocks=64, device="cuda")
    out = eng.generate(golden["prompt"], SamplingParams(max_tokens=64, **GREEDY))
    assert out == golden["tokens"]


def test_graph_decode_equals_eager_decode_bf16():
    cfg = ModelConfig(name="t", n_layers=3, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1536, vocab=4096,
                      rope=RopeConfig(theta=500000.0), dtype="bf16")
    w = fast_random_weights(cfg, ShardSpec(), "cuda")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (50, 31, 77)]
    outs = []
    for graphs in (False, True):
        eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=graphs, max_seqs=4)
        ids = [eng.submit(p, SamplingParams(max_tokens=20, **GREEDY), use_prefix_cache=False) for p in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1]
    assert all(len(x) == 20 for x in outs[0])


def test_large_batch_uses_tensor_core_gemm_and_matches_small_batch_path():
    """Same prompts decoded alone (M<=8 kernels) and in a batch of 12 (tcgen05 GEMM): the
    per-sequence greedy tokens may differ only through bf16 rounding, so compare logits."""
    cfg = ModelConfig(name="t", n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1536, vocab=4096,
                      rope=RopeConfig(theta=500000.0), dtype="bf16")
    w = fast_random_weights(cfg, ShardSpec(), "cuda")
    eng = Engine(cfg, w, n_blocks=256, device="cuda", use_graphs=False, max_seqs=16)
    prompts = [oracle_prompt(20 + i, cfg.vocab, seed=i).tolist() for i in range(12)]
    for p in prompts:
        eng.submit(p, SamplingParams(max_tokens=2, **GREEDY), use_prefix_cache=False)
    eng.step()
    batch_logits = eng.exe.last_logits.float().clone()
    solo = []
    for p in prompts:
        e2 = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False)
        e2.submit(p, SamplingParams(max_tokens=1, **GREEDY), use_prefix_cache=False)
        e2.step()
        solo.append(e2.exe.last_logits.float()[0].clone())
    solo = torch.stack(solo)
    err = (batch_logits - solo).abs().max().item()
    assert err < 0.05 * solo.abs().max().item() + 0.05, err


def test_moe_and_mla_on_gpu_match_oracle_fp32():
    for name in ("tiny-moe", "tiny-mla"):
        cfg = preset(name)
        w = build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cuda")
        eng = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False)
        p = oracle_prompt(40, cfg.vocab, seed=3).tolist()
        want = OracleModel(cfg, RandomSource(seed=0)).greedy(torch.tensor(p), 8)
        assert eng.generate(p, SamplingParams(max_tokens=8, **GREEDY)) == want


def test_hybrid_linear_attention_model_on_gpu_matches_oracle_and_graphs():
    """Qwen3-Next-shaped model: gated-delta-rule layers (recurrent state per sequence seat) beside gated softmax attention.
    fp32 against the oracle with a chunked prompt; bf16 with CUDA graphs against eager, several sequences at once."""
    cfg = preset("tiny-qwen3-next")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0), device="cuda")
    p = oracle_prompt(40, cfg.vocab, seed=3).tolist()
    want = OracleModel(cfg, RandomSource(seed=0)).greedy(torch.tensor(p), 8)
    eng = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False, prefill_chunk=16)
    assert eng.generate(p, SamplingParams(max_tokens=8, **GREEDY)) == want
    cfg = preset("tiny-qwen3-next")
    cfg.dtype = "bf16"
    w = fast_random_weights(cfg, ShardSpec(), "cuda")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (50, 31, 77)]
    outs = []
    for graphs in (False, True):
        eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=graphs, max_seqs=4)
        ids = [eng.submit(q, SamplingParams(max_tokens=12, **GREEDY)) for q in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1] and all(len(x) == 12 for x in outs[0])
    # prefix reuse: a prompt that contains an earlier one (a chat's next turn) continues from the recurrent state that was
    # snapshotted at the earlier prompt's last block boundary (80 of its 90 tokens)
    a = oracle_prompt(90, cfg.vocab, seed=1).tolist()
    b = a[:85] + oracle_prompt(30, cfg.vocab, seed=2).tolist()
    fresh = Engine(cfg, w, n_blocks=128, device="cuda", max_seqs=4).generate(b, SamplingParams(max_tokens=10, **GREEDY))
    eng = Engine(cfg, w, n_blocks=128, device="cuda", max_seqs=4)
    got = {}
    for q in (a, b):
        rid = eng.submit(q, SamplingParams(max_tokens=10, **GREEDY))
        seq = eng.seqs[rid]
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got.setdefault(o.req_id, []).append(o.token)
    assert seq.n_cached_prefix == 80 and got[rid] == fresh


def test_nemotron_h_bf16_graphs_equal_eager():
    """bf16 Nemotron-H-shaped model: the decode step (Mamba-2 kernels, relu^2 experts on the grouped expert kernels) under
    CUDA graphs gives the tokens of the eager run."""
    cfg = preset("tiny-nemotron-h")
    cfg.dtype = "bf16"
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05, dtype=torch.bfloat16), device="cuda")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (50, 31, 77)]
    outs = []
    for graphs in (False, True):
        eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=graphs, max_seqs=4)
        ids = [eng.submit(q, SamplingParams(max_tokens=12, **GREEDY)) for q in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1] and all(len(x) == 12 for x in outs[0])


def test_nemotron_h_on_gpu_matches_the_cpu_engine():
    """Nemotron-H-shaped model (Mamba-2 layers on the state-space kernels, attention without positions, relu^2 MLP and
    experts): fp32 on the GPU reproduces the CPU engine's tokens with a chunked prompt and two sequences in flight."""
    cfg = preset("tiny-nemotron-h")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (70, 23)]
    outs = []
    for dev in ("cpu", "cuda"):
        w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05), device=dev)
        eng = Engine(cfg, w, n_blocks=64, device=dev, prefill_chunk=32, max_seqs=4, use_graphs=False)     # fp32 experts: PyTorch ops
        ids = [eng.submit(q, SamplingParams(max_tokens=8, **GREEDY)) for q in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1] and all(len(x) == 8 for x in outs[0])


def test_step35_on_gpu_matches_the_cpu_engine_and_graphs():
    """Step-3.5-shaped model (layers with their own query-head count, RoPE and window, a gate per head, sigmoid-routed
    experts with clamped SwiGLU beside a shared expert): fp32 on the GPU reproduces the CPU engine's tokens with a chunked
    prompt; bf16 under CUDA graphs equals eager."""
    cfg = preset("tiny-step3p5")
    p = oracle_prompt(70, cfg.vocab, seed=3).tolist()
    want = Engine(cfg, build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05), device="cpu"), n_blocks=64, device="cpu",
                  prefill_chunk=32).generate(p, SamplingParams(max_tokens=8, **GREEDY))
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05), device="cuda")
    eng = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False, prefill_chunk=32)
    assert eng.generate(p, SamplingParams(max_tokens=8, **GREEDY)) == want
    cfg = preset("tiny-step3p5")
    cfg.dtype = "bf16"
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05, dtype=torch.bfloat16), device="cuda")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (50, 31, 77)]
    outs = []
    for graphs in (False, True):
        eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=graphs, max_seqs=4)
        ids = [eng.submit(q, SamplingParams(max_tokens=12, **GREEDY), use_prefix_cache=False) for q in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1] and all(len(x) == 12 for x in outs[0])


def test_gemma4_on_gpu_matches_the_cpu_engine_and_graphs():
    """Gemma-4-shaped model (sliding and full layers with their own head sizes, v = k, shared-KV layers, per-layer inputs,
    soft-capped logits): fp32 on the GPU reproduces the CPU engine's tokens with a chunked prompt; bf16 with CUDA graphs
    equals eager."""
    cfg = preset("tiny-gemma4")
    p = oracle_prompt(70, cfg.vocab, seed=3).tolist()
    want = Engine(cfg, build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05), device="cpu"), n_blocks=64, device="cpu",
                  prefill_chunk=32).generate(p, SamplingParams(max_tokens=8, **GREEDY))
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05), device="cuda")
    eng = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False, prefill_chunk=32)
    assert eng.generate(p, SamplingParams(max_tokens=8, **GREEDY)) == want
    cfg = preset("tiny-gemma4")
    cfg.dtype = "bf16"
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, std=0.05, dtype=torch.bfloat16), device="cuda")
    prompts = [oracle_prompt(n, cfg.vocab, seed=n).tolist() for n in (50, 31, 77)]
    outs = []
    for graphs in (False, True):
        eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=graphs, max_seqs=4)
        ids = [eng.submit(q, SamplingParams(max_tokens=12, **GREEDY), use_prefix_cache=False) for q in prompts]
        got = {i: [] for i in ids}
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    got[o.req_id].append(o.token)
        outs.append([got[i] for i in ids])
    assert outs[0] == outs[1] and all(len(x) == 12 for x in outs[0])


@pytest.mark.parametrize("name,quant", [("tiny-moe", "none"), ("tiny-moe", "mxfp8"), ("tiny-llama", "mxfp8"), ("tiny-mla", "dsfp8")])
def test_bf16_moe_and_fp8_models_on_gpu_track_the_cpu_definition(name, quant):
    """bf16 activations through the MoE kernels (router, grouped GEMMs / GEMVs) and the fp8-weight GEMMs, with and
    without CUDA graphs: the logits of the last prompt position stay close to the CPU fp32 run of the same
    (dequantised) weights, and the decode runs under graph capture (nothing on the path syncs with the host)."""
    from dataclasses import replace
    cfg = replace(preset(name), dtype="bf16", quant=quant)
    src = RandomSource(seed=0, std=0.05, dtype=torch.bfloat16)
    w_gpu = build_weights(cfg, ShardSpec(), src, device="cuda")
    w_cpu = build_weights(cfg, ShardSpec(), src, device="cpu")
    p = oracle_prompt(40, cfg.vocab, seed=3).tolist()
    cpu = Engine(cfg, w_cpu, n_blocks=64, device="cpu")
    cpu.generate(p, SamplingParams(max_tokens=1, **GREEDY))
    want = cpu.exe.last_logits.float()[0]
    for graphs in ((False,) if cfg.mla else (False, True)):      # the MLA attention is not a captured kernel yet
        eng = Engine(cfg, w_gpu, n_blocks=64, device="cuda", use_graphs=graphs, max_seqs=4)
        toks = eng.generate(p, SamplingParams(max_tokens=6, **GREEDY))
        assert len(toks) == 6 and all(0 <= t < cfg.vocab for t in toks)
        from exo_b200.ops import cuda as K
        K.gemm_check()
    e2 = Engine(cfg, w_gpu, n_blocks=64, device="cuda", use_graphs=False)
    e2.generate(p, SamplingParams(max_tokens=1, **GREEDY))
    got = e2.exe.last_logits.float()[0].cpu()
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 0.06, err


def test_embedding_splice_on_gpu_equals_the_tokens_it_stands_for():
    """Feature rows passed as ``embeds`` replace the placeholder tokens' embeddings in the GPU prefill step too."""
    from dataclasses import replace
    cfg = replace(preset("tiny-llama"), dtype="bf16")
    w = build_weights(cfg, ShardSpec(), RandomSource(seed=0, dtype=torch.bfloat16), device="cuda")
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(5, cfg.vocab, (300,), generator=g).tolist()
    stand_in = torch.randint(5, cfg.vocab, (40,), generator=g).tolist()
    real = prompt[:100] + stand_in + prompt[140:]
    holes = prompt[:100] + [0] * 40 + prompt[140:]
    rows = w.embed[torch.tensor(stand_in, device="cuda")]
    want = Engine(cfg, w, n_blocks=64, device="cuda").generate(real, SamplingParams(max_tokens=6, **GREEDY))
    for chunk in (4096, 128):
        eng = Engine(cfg, w, n_blocks=64, device="cuda", prefill_chunk=chunk)
        rid = eng.submit(holes, SamplingParams(max_tokens=6, **GREEDY), embeds=[(100, rows)], media=[(100, 140, b"x" * 32)])
        got = []
        while eng.has_work:
            got += [o.token for o in eng.step() if o.req_id == rid and o.token is not None]
        assert got == want, (chunk, got, want)


@pytest.mark.parametrize("shape", ["small", "qk-norm-bias", "llama-8b-layer"])
def test_whole_step_decode_kernel_matches_the_per_op_path(shape):
    """Batch-1 decode as one persistent kernel against the same step as separate kernels: the logits of every decode
    step agree to bf16 rounding, the greedy tokens are the same, and the KV cache the kernel appended to serves a later
    prefill-with-history correctly (a second request decoded through the per-op path on the same engine)."""
    from exo_b200.ops import cuda as K
    if shape == "small":
        cfg = ModelConfig(name="m", n_layers=3, hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=2048, vocab=4096,
                          rope=RopeConfig(theta=500000.0), dtype="bf16")
    elif shape == "qk-norm-bias":
        cfg = ModelConfig(name="m", family="qwen3", n_layers=2, hidden=1024, n_heads=8, n_kv_heads=8, head_dim=128, ffn=3072,
                          vocab=4096, qk_norm=True, attn_bias=True, rope=RopeConfig(theta=10000.0, partial_rotary_factor=0.5),
                          dtype="bf16")
    else:
        cfg = ModelConfig(name="m", n_layers=2, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=8192,
                          rope=RopeConfig(theta=500000.0), dtype="bf16")
    w = fast_random_weights(cfg, ShardSpec(), "cuda")
    prompt = oracle_prompt(333, cfg.vocab, seed=4).tolist()         # 333 keys: splits with uneven and (at 148 CTAs) short ranges
    runs = {}
    default = K.use_decode_mega
    for mega in (False, True):
        K.use_decode_mega = mega
        try:
            eng = Engine(cfg, w, n_blocks=128, device="cuda", use_graphs=False)
            assert bool(getattr(eng.exe.model, "_mega", None)) is False
            rid = eng.submit(prompt, SamplingParams(max_tokens=24, **GREEDY), use_prefix_cache=False)
            toks, logits = [], []
            while eng.has_work:
                for o in eng.step():
                    if o.req_id == rid and o.token is not None:
                        toks.append(o.token)
                        logits.append(eng.exe.last_logits.float()[0, :cfg.vocab].clone())
            assert bool(eng.exe.model._mega) is mega
            K.check_status("cuda")
            runs[mega] = (toks, torch.stack(logits))
        finally:
            K.use_decode_mega = default
    (t0, l0), (t1, l1) = runs[False], runs[True]
    # the two runs see the same inputs up to and including the first step whose greedy tokens differ (random weights
    # give near-ties, and bf16 noise may flip one): the logits of those steps must agree to rounding
    agree = next((i for i, (a, b) in enumerate(zip(t0, t1)) if a != b), len(t0) - 1)
    a, b = l0[:agree + 1], l1[:agree + 1]
    err = (a - b).abs().max().item()
    assert err < 0.03 * a.abs().max().item() + 0.02, (err, agree)
    assert agree >= 3, (t0, t1)


def test_whole_step_decode_kernel_under_cuda_graphs_and_bs1_generate():
    from exo_b200.ops import cuda as K
    cfg = ModelConfig(name="m", n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, head_dim=128, ffn=2048, vocab=4096,
                      rope=RopeConfig(theta=500000.0), dtype="bf16")
    w = fast_random_weights(cfg, ShardSpec(), "cuda")
    prompt = oracle_prompt(40, cfg.vocab, seed=9).tolist()
    default, K.use_decode_mega = K.use_decode_mega, True
    try:
        eager = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=False).generate(prompt, SamplingParams(max_tokens=40, **GREEDY))
        graph_eng = Engine(cfg, w, n_blocks=64, device="cuda", use_graphs=True)
        graphed = graph_eng.generate(prompt, SamplingParams(max_tokens=40, **GREEDY))
    finally:
        K.use_decode_mega = default
    assert bool(graph_eng.exe.model._mega) and graphed == eager and len(eager) == 40
    K.check_status("cuda")
