"""Multi-head latent attention kernels (DeepSeek dimensions: kv_lora 512, rope 64, nope 128, v 128) against the
fp32 PyTorch definitions, and an MLA model end to end on the GPU."""
import pytest
import torch

from exo_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
L, R, NOPE, V = 512, 64, 128, 128


def _inv_freq():
    return (1.0 / (10000.0 ** (torch.arange(0, R, 2, device="cuda").float() / R))).contiguous()


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)).item()


def test_kv_append_normalises_the_latent_part_and_rotates_the_rope_part():
    from exo_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    T = 37
    kva = torch.randn(T, L + R, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(L, device="cuda", generator=g)).bfloat16()
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g, dtype=torch.int32)
    slots = torch.randperm(64 * 16, device="cuda", generator=g)[:T].to(torch.int32)
    got = torch.zeros(64, 16, L + R, device="cuda", dtype=torch.bfloat16)
    want = torch.zeros_like(got)
    ops.mla_kv_append(kva, w, 1e-6, pos, _inv_freq(), 1.0, got, slots, L)
    ref.mla_kv_append(kva, w, 1e-6, pos, _inv_freq(), 1.0, want, slots, L)
    assert _rel(got, want) < 2e-2
    untouched = torch.ones(64 * 16, dtype=torch.bool, device="cuda")
    untouched[slots.long()] = False
    assert float(got.view(-1, L + R)[untouched].float().abs().max()) == 0.0      # only the given slots are written


@pytest.mark.parametrize("T", [1, 16, 200])
@pytest.mark.parametrize("H", [16, 32])
def test_query_and_output_absorption(T, H):
    from exo_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(T + H)
    q = torch.randn(T, H, NOPE + R, device="cuda", generator=g).bfloat16()
    w_uk = (torch.randn(H, NOPE, L, device="cuda", generator=g) / 11).bfloat16()
    w_uv = (torch.randn(H, V, L, device="cuda", generator=g) / 22).bfloat16()
    pos = torch.randint(0, 9000, (T,), device="cuda", generator=g, dtype=torch.int32)
    got = ops.mla_q_absorb(q, w_uk, pos, _inv_freq(), 1.0, NOPE, L)
    want = ref.mla_q_absorb(q, w_uk, pos, _inv_freq(), 1.0, NOPE)
    assert got.shape == (T, H, L + R) and _rel(got, want) < 2e-2
    o_lat = torch.randn(T, H, L, device="cuda", generator=g).bfloat16()
    got_o = ops.mla_o_absorb(o_lat, w_uv)
    want_o = ref.mla_o_absorb(o_lat, w_uv)
    assert got_o.shape == (T, H * V) and _rel(got_o, want_o) < 2e-2


def _cache(n_blocks, g):
    c = torch.randn(n_blocks, 16, L + R, device="cuda", generator=g) * 0.5
    return c.bfloat16()


@pytest.mark.parametrize("H", [4, 16, 32, 128])
@pytest.mark.parametrize("lens", [(1,), (17, 300, 129), (2048, 5, 1000, 640)])
def test_latent_decode_attention_against_fp32_definition(H, lens):
    from exo_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(H + len(lens))
    B = len(lens)
    per = max(-(-n // 16) for n in lens) + 1
    cache = _cache(B * per + 1, g)
    bt = (torch.arange(B * per, device="cuda", dtype=torch.int32).view(B, per) + 1)
    bt = bt[:, torch.randperm(per, device="cuda", generator=g)]          # pages in no particular order
    seq = torch.tensor(lens, device="cuda", dtype=torch.int32)
    cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    q = (torch.randn(B, H, L + R, device="cuda", generator=g) * 0.3).bfloat16()
    scale = (NOPE + R) ** -0.5
    for _ in range(2):                                                   # twice: the tickets must come back clean
        got = ops.mla_paged_attention(q, cache, bt, seq, cu, scale, L, 1)
    want = ref.mla_paged_attention(q[..., :L], q[..., L:], cache, bt, seq, cu, scale, L)
    assert _rel(got, want) < 3e-2
    from exo_b200.ops import cuda as K
    K.check_status()


def test_latent_prefill_attention_is_causal_per_sequence():
    from exo_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    H = 16
    q_lens, ctx = (40, 1, 130), (0, 77, 256)          # new tokens and tokens already in the cache, per sequence
    B = len(q_lens)
    lens = [a + b for a, b in zip(q_lens, ctx)]
    per = max(-(-n // 16) for n in lens) + 1
    cache = _cache(B * per + 1, g)
    bt = torch.arange(B * per, device="cuda", dtype=torch.int32).view(B, per) + 1
    seq = torch.tensor(lens, device="cuda", dtype=torch.int32)
    cu = torch.tensor([0, 40, 41, 171], device="cuda", dtype=torch.int32)
    T = sum(q_lens)
    q = (torch.randn(T, H, L + R, device="cuda", generator=g) * 0.3).bfloat16()
    scale = (NOPE + R) ** -0.5
    got = ops.mla_paged_attention(q, cache, bt, seq, cu, scale, L, max(q_lens))
    want = ref.mla_paged_attention(q[..., :L], q[..., L:], cache, bt, seq, cu, scale, L)
    assert _rel(got, want) < 3e-2


def test_mla_model_with_real_head_dimensions_decodes_under_cuda_graphs_and_tracks_the_cpu_definition():
    """A small DeepSeek-style model whose attention dimensions are the real ones, so every MLA kernel is on the
    path: prefill (GEMM absorption) and decode (CUDA-core absorption, split-KV attention) with CUDA graphs."""
    from exo_b200.engine.engine import Engine
    from exo_b200.engine.kv import SamplingParams
    from exo_b200.models.config import ModelConfig
    from exo_b200.models.oracle import oracle_prompt
    from exo_b200.models.weights import RandomSource, ShardSpec, build_weights
    from exo_b200.ops import cuda as K
    cfg = ModelConfig(name="small-mla", family="deepseek_v3", n_layers=2, hidden=512, n_heads=16, n_kv_heads=16, head_dim=192,
                      ffn=1024, vocab=2048, mla=True, q_lora_rank=256, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64,
                      v_head_dim=128, n_experts=8, n_experts_per_tok=2, moe_ffn=256, n_shared_experts=1, first_dense_layers=1,
                      router="sigmoid", routed_scaling=1.5, n_group=2, topk_group=1, router_bias=True, dtype="bf16")
    src = RandomSource(seed=0, std=0.05, dtype=torch.bfloat16)
    w_gpu = build_weights(cfg, ShardSpec(), src, device="cuda")
    w_cpu = build_weights(cfg, ShardSpec(), src, device="cpu")
    p = oracle_prompt(150, cfg.vocab, seed=3).tolist()
    greedy = dict(temperature=0.0, ignore_eos=True)
    cpu = Engine(cfg, w_cpu, n_blocks=64, device="cpu")
    cpu.generate(p, SamplingParams(max_tokens=1, **greedy))
    want = cpu.exe.last_logits.float()[0]
    eng = Engine(cfg, w_gpu, n_blocks=64, device="cuda", max_seqs=4)
    assert eng.exe.use_graphs
    toks = eng.generate(p, SamplingParams(max_tokens=6, **greedy))
    assert len(toks) == 6 and eng.exe.graphs
    K.check_status()
    e2 = Engine(cfg, w_gpu, n_blocks=64, device="cuda", use_graphs=False)
    e2.generate(p, SamplingParams(max_tokens=1, **greedy))
    got = e2.exe.last_logits.float()[0].cpu()
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 0.06, err
