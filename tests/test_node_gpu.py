"""The product on a GPU: node processes → master → worker → runner child process → B200 engine, driven over HTTP.

One node per GPU (real NVML telemetry, loopback bus), a small random-weight Llama checkpoint on disk whose
attention has the 128-wide heads the tensor-core kernels take.  The instance is placed over HTTP, a chat completion
is streamed, and the text is compared with the same checkpoint run through ``Engine.generate`` in this process.
"""
import json
import socket

import anyio
import httpx
import pytest
import torch

from exo_b200.models.config import ModelConfig
from exo_b200.models.weights import RandomSource, SafetensorsSource, ShardSpec, build_weights, write_safetensors

pytestmark = pytest.mark.gpu


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_checkpoint(models_dir):
    d = models_dir / "org--small"
    d.mkdir(parents=True)
    hidden, layers, heads, kv, ffn, vocab = 512, 2, 4, 2, 1024, 512
    (d / "config.json").write_text(json.dumps({
        "model_type": "llama", "architectures": ["LlamaForCausalLM"], "hidden_size": hidden, "num_hidden_layers": layers,
        "num_attention_heads": heads, "num_key_value_heads": kv, "intermediate_size": ffn, "vocab_size": vocab,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048, "eos_token_id": 257}))
    src = RandomSource(seed=0, std=0.05)
    D = hidden // heads
    names = {"model.embed_tokens.weight": (vocab, hidden), "model.norm.weight": (hidden,), "lm_head.weight": (vocab, hidden)}
    for i in range(layers):
        p = f"model.layers.{i}."
        names.update({p + "input_layernorm.weight": (hidden,), p + "post_attention_layernorm.weight": (hidden,),
                      p + "self_attn.q_proj.weight": (heads * D, hidden), p + "self_attn.k_proj.weight": (kv * D, hidden),
                      p + "self_attn.v_proj.weight": (kv * D, hidden), p + "self_attn.o_proj.weight": (hidden, heads * D),
                      p + "mlp.gate_proj.weight": (ffn, hidden), p + "mlp.up_proj.weight": (ffn, hidden),
                      p + "mlp.down_proj.weight": (hidden, ffn)})
    write_safetensors(d / "model.safetensors", {k: src.get(k, v) for k, v in names.items()})
    return d


async def wait_for(fn, timeout=60.0):
    with anyio.fail_after(timeout):
        while True:
            v = await fn()
            if v:
                return v
            await anyio.sleep(0.1)


@pytest.mark.parametrize("n_gpus", [1, 2])
def test_chat_completion_over_http_runs_on_the_gpu_engine(n_gpus, tmp_path, monkeypatch):
    if torch.cuda.device_count() < n_gpus:
        pytest.skip(f"needs {n_gpus} GPUs")
    from exo_b200.main import Args, Node
    from exo_b200.routing.router import LoopbackHub, make_router
    from exo_b200.shared import constants
    from exo_b200.shared.base import NodeId
    import exo_b200.api.main as api_main
    monkeypatch.setenv("EXO_ENGINE", "b200")
    monkeypatch.setenv("EXO_MAX_KV_BLOCKS", "256")
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    models = tmp_path / "models"
    ckpt = make_checkpoint(models)
    monkeypatch.setattr(constants, "EXO_DEFAULT_MODELS_DIR", models)
    monkeypatch.setattr(constants, "EXO_MODELS_DIRS", (models,))
    monkeypatch.setattr(constants, "EXO_MODELS_READ_ONLY_DIRS", ())
    monkeypatch.setattr(constants, "EXO_EVENT_LOG_DIR", tmp_path / "event_log")
    monkeypatch.setattr(constants, "EXO_TRACING_CACHE_DIR", tmp_path / "traces")
    monkeypatch.setattr(constants, "EXO_CUSTOM_MODEL_CARDS_DIR", tmp_path / "cards")
    monkeypatch.setattr(api_main, "API_EVENT_LOG_DIR", tmp_path / "event_log" / "api")
    monkeypatch.setenv("EXO_MODELS_DIRS", str(models))          # the runner child resolves the checkpoint from the environment
    monkeypatch.setenv("EXO_DEFAULT_MODELS_DIR", str(models))
    port = free_port()
    n_new = 12
    body = {"model": "org/small", "messages": [{"role": "user", "content": "The quick brown fox"}], "max_tokens": n_new,
            "temperature": 0.0}
    got: dict[str, object] = {}

    async def main():
        hub = LoopbackHub()
        ids = [NodeId(c * 32) for c in "ab"[:n_gpus]]
        nodes = [Node(Args(spawn_api=(i == 0), api_port=port, force_master=(i == 0), gpu=i, offline=True), ids[i],
                      make_router(ids[i], hub.attach(ids[i]))) for i in range(n_gpus)]
        async with anyio.create_task_group() as tg:
            for n in nodes:
                tg.start_soon(n.run)
            async with httpx.AsyncClient(base_url=f"http://127.0.0.1:{port}", timeout=120) as http:
                async def ready():
                    try:
                        st = (await http.get("/state")).json()
                    except httpx.TransportError:
                        return None
                    return st if len(st["nodeBackends"]) == n_gpus and len(st["nodeMemory"]) == n_gpus else None
                await wait_for(ready)
                r = await http.post("/place_instance", json={"model_id": "org/small", "sharding": "Tensor", "min_nodes": n_gpus})
                assert r.status_code == 200, r.text

                async def instance_ready():
                    st = (await http.get("/state")).json()
                    runners = st["runners"]
                    failed = [v for v in runners.values() if "RunnerFailed" in v]
                    assert not failed, failed
                    return len(runners) == n_gpus and all("RunnerReady" in v for v in runners.values())
                await wait_for(instance_ready, 240)
                r = await http.post("/v1/chat/completions", json=body)
                assert r.status_code == 200, r.text
                got["plain"] = r.json()
                async with http.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as s:
                    lines = [ln async for ln in s.aiter_lines() if ln.startswith("data: ")]
                assert lines[-1] == "data: [DONE]"
                got["stream"] = "".join(json.loads(ln[6:])["choices"][0]["delta"].get("content") or "" for ln in lines[:-1])
                r = await http.post("/bench/chat/completions", json=body)
                assert r.status_code == 200, r.text
                got["bench"] = r.json()
                iid = next(iter((await http.get("/state")).json()["instances"]))
                assert (await http.delete(f"/instance/{iid}")).status_code == 200

                async def gone():
                    st = (await http.get("/state")).json()
                    return not st["instances"] and not st["runners"]
                await wait_for(gone, 60)
            for n in nodes:
                n._tg.cancel_tasks()
            tg.cancel_scope.cancel()
    anyio.run(main)

    plain = got["plain"]
    text = plain["choices"][0]["message"]["content"]
    assert plain["usage"]["completion_tokens"] == n_new or plain["choices"][0]["finish_reason"] == "stop"
    assert got["stream"] == text                      # streaming and non-streaming agree (same engine, greedy)
    bench = got["bench"]
    assert bench["usage"]["completion_tokens"] == n_new and "generation_stats" in json.dumps(bench)
    if n_gpus == 1:
        # the same checkpoint through the token engine in this process: identical kernels, identical tokens
        from exo_b200.engine.engine import Engine
        from exo_b200.engine.kv import SamplingParams
        from exo_b200.shared.messages import InputMessage, TextGenerationTaskParams
        from exo_b200.worker.engines.b200.tokenizer import ByteTokenizer, Detokenizer, render_prompt
        cfg = ModelConfig.from_pretrained(ckpt)
        cfg.dtype = "bf16"
        w = build_weights(cfg, ShardSpec(), SafetensorsSource(ckpt, dtype=torch.bfloat16), device="cuda")
        tok = ByteTokenizer(cfg.vocab)
        params = TextGenerationTaskParams(model="org/small", input=[InputMessage(role="user", content="The quick brown fox")],
                                          temperature=0.0, max_output_tokens=n_new)
        ids = tok.encode(render_prompt(tok, params)[0], add_special_tokens=True)
        eng = Engine(cfg, w, n_blocks=64, device="cuda")
        want = eng.generate(ids, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
        detok = Detokenizer(tok, ids)
        want_text = "".join(detok.add(t) for t in want)
        assert bench["choices"][0]["message"]["content"] == want_text, (bench["choices"][0]["message"]["content"], want_text, want)
