"""Qwen3-Next (gated delta rule + gated attention + shared-expert gate) against the ``transformers`` implementation.

A tiny randomly initialised ``Qwen3NextForCausalLM`` is exported under the hub's tensor names; the engine loads that
checkpoint and must reproduce the library's logits over a prompt (chunked prefill included: the recurrent state and the
convolution history cross chunk and step borders) and its greedy continuation.
"""
import json

import pytest
import torch

from exo_b200.engine.engine import Engine
from exo_b200.engine.kv import SamplingParams
from exo_b200.models.config import ModelConfig
from exo_b200.models.transformer import Decoder, KVPool, StepInputs
from exo_b200.models.weights import SafetensorsSource, ShardSpec, build_weights, write_safetensors

tf = pytest.importorskip("transformers")
if not hasattr(tf, "Qwen3NextForCausalLM"):
    pytest.skip("this transformers build has no Qwen3-Next", allow_module_level=True)


@pytest.fixture(scope="module")
def exported(tmp_path_factory):
    torch.manual_seed(0)
    hc = tf.Qwen3NextConfig(
        vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
        linear_value_head_dim=32, linear_conv_kernel_dim=4, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
        shared_expert_intermediate_size=64, decoder_sparse_step=1, mlp_only_layers=[1], norm_topk_prob=True,
        rms_norm_eps=1e-6, max_position_embeddings=512, tie_word_embeddings=False)
    model = tf.Qwen3NextForCausalLM(hc).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.normal_(0, 0.2 if "norm" in n else 0.5 if ("A_log" in n or "dt_bias" in n) else 0.08)
    tensors = {}
    for k, v in model.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):          # the library keeps experts stacked; the hub keeps one tensor each
            stem, F = k[:-len("gate_up_proj")], v.shape[1] // 2
            for e in range(v.shape[0]):
                tensors[f"{stem}{e}.gate_proj.weight"] = v[e, :F].clone()
                tensors[f"{stem}{e}.up_proj.weight"] = v[e, F:].clone()
        elif k.endswith("mlp.experts.down_proj"):
            stem = k[:-len("down_proj")]
            for e in range(v.shape[0]):
                tensors[f"{stem}{e}.down_proj.weight"] = v[e].clone()
        else:
            tensors[k] = v.clone()
    d = tmp_path_factory.mktemp("qwen3next")
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    write_safetensors(d / "model.safetensors", tensors)
    cfg = ModelConfig.from_pretrained(d)
    cfg.dtype = "fp32"
    return model, cfg, d


def test_config_fields(exported):
    _, cfg, _ = exported
    assert cfg.family == "qwen3_next" and cfg.layer_types == ("linear", "linear", "linear", "full")
    assert cfg.rope.partial_rotary_factor == 0.25 and cfg.attn_gate and cfg.norm_one_plus and cfg.shared_expert_gate
    assert [cfg.layer_is_moe(i) for i in range(4)] == [True, False, True, True]


def _step(dec, kv, toks, start, seat=1):
    T = len(toks)
    n = start + T
    bt = torch.arange(1, 1 + (n + 15) // 16, dtype=torch.int32)[None]
    pos = torch.arange(start, n, dtype=torch.int32)
    inp = StepInputs(tokens=torch.tensor(toks, dtype=torch.int32), positions=pos, slots=(16 + pos).int(),
                     cu_q=torch.tensor([0, T], dtype=torch.int32), seq_lens=torch.tensor([n], dtype=torch.int32),
                     block_tables=bt, logit_rows=torch.arange(T), max_q_len=T,
                     state_slots=torch.tensor([seat], dtype=torch.int32))
    return dec.logits(inp, kv)


def test_logits_match_library_across_chunks_and_steps(exported):
    model, cfg, d = exported
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    dec = Decoder(cfg, w)
    kv = KVPool(cfg, ShardSpec(), n_blocks=16, device="cpu", max_seqs=2)
    toks = torch.randint(0, cfg.vocab, (1, 100), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = model(toks).logits[0]
    got = torch.cat((_step(dec, kv, toks[0, :70].tolist(), 0),          # longer than one chunk of the chunked form
                     _step(dec, kv, toks[0, 70:97].tolist(), 70),       # continues from the stored state (sequential form)
                     _step(dec, kv, toks[0, 97:98].tolist(), 97),       # single-token steps
                     _step(dec, kv, toks[0, 98:99].tolist(), 98),
                     _step(dec, kv, toks[0, 99:100].tolist(), 99)), 0)
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
    # a new sequence on the same seat starts from zero state (its first position is 0)
    again = _step(dec, kv, toks[0, :10].tolist(), 0)
    assert torch.allclose(again, want[:10], atol=2e-3, rtol=2e-3)


def test_engine_greedy_matches_library(exported):
    model, cfg, d = exported
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    prompt = torch.randint(0, cfg.vocab, (1, 23), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want = model.generate(prompt, max_new_tokens=8, do_sample=False)[0, 23:].tolist()
    eng = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=16)      # the prompt takes two prefill chunks
    got = eng.generate(prompt[0].tolist(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert got == want


def test_prefix_reuse_restores_the_recurrent_state(exported):
    """A second request that shares a prompt prefix re-uses the cached blocks up to the snapshotted block boundary: its
    recurrent layers continue from the state saved there, and the tokens equal those of an engine that computes the
    whole prompt."""
    from exo_b200.engine.plan import STATE_RESTORE, STATE_SAVE, StepPlan
    _, cfg, d = exported
    w = build_weights(cfg, ShardSpec(), SafetensorsSource(d, dtype=torch.float32), device="cpu")
    g = torch.Generator().manual_seed(3)
    first = torch.randint(0, cfg.vocab, (45,), generator=g).tolist()
    second = first[:40] + torch.randint(0, cfg.vocab, (21,), generator=g).tolist()        # 40 shared tokens, then its own
    greedy = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    fresh = Engine(cfg, w, n_blocks=32, device="cpu").generate(second, greedy)             # generate(): prefix cache off
    eng = Engine(cfg, w, n_blocks=32, device="cpu", prefill_chunk=64)
    assert eng.sched.state_snapshots and eng.exe.kv.n_snapshots >= 2
    plans = []
    eng.exe.run, run = (lambda plan, *a, **k: (plans.append(plan), run(plan, *a, **k))[1]), eng.exe.run
    outs = {}
    for prompt in (first, second):
        rid = eng.submit(prompt, greedy)
        while eng.has_work:
            for o in eng.step():
                if o.token is not None:
                    outs.setdefault(o.req_id, []).append(o.token)
        outs[rid] = outs.pop(rid)
    ops = [op for p in plans for op in p.state_ops]
    # the first prompt (45 tokens) is cut at 32 = the last block boundary before its final token, and saved there
    assert [p.n_tokens for p in plans[:2]] == [32, 13] and ops[0][0] == STATE_SAVE
    # the second re-uses those two blocks: restore, then 61 - 32 tokens of its own, cut again at its boundary (48)
    seq2 = [p for p in plans if p.state_ops and p.state_ops[0][0] == STATE_RESTORE][0]
    assert seq2.positions[0] == 32 and seq2.n_tokens == 16 and seq2.state_ops[0][2] == ops[0][2]
    assert list(outs.values())[1] == fresh
    # the instructions travel inside the packed plan (tensor-parallel followers unpack them)
    import numpy as np
    buf = np.zeros(4096, np.int32)
    seq2.pack(buf, seq2.n_tokens, seq2.n_seqs, seq2.block_tables.shape[1])
    assert StepPlan.unpack(buf).state_ops == seq2.state_ops
