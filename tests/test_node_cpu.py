"""Two whole nodes in one process (loopback bus, fake GPUs, fake engine) driven through the HTTP API."""
import json
import socket

import anyio
import httpx
import pytest

from exo_b200.main import Args, Node
from exo_b200.routing.router import LoopbackHub, make_router
from exo_b200.shared import constants
from exo_b200.shared.base import NodeId
from exo_b200.utils import info_gatherer
from exo_b200.utils.info_gatherer import GpuSample


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def fake_gpus():
    return [GpuSample(index=i, name="NVIDIA B200", uuid=f"GPU-{i}", mem_total=180 << 30, mem_free=170 << 30, power_mw=400_000,
                      temp_c=40, util_pct=10, p2p_ok=[1, 1], nvlink_peers_links=[0, 0], active_links=18) for i in range(2)]


@pytest.fixture
def cluster_env(tmp_path, monkeypatch):
    monkeypatch.setenv("EXO_ENGINE", "fake")
    monkeypatch.setattr(info_gatherer, "nvml_probe", fake_gpus)
    monkeypatch.setattr(info_gatherer, "kernels_available", lambda: True)
    models = tmp_path / "models"
    models.mkdir()
    for name in ("EXO_DEFAULT_MODELS_DIR",):
        monkeypatch.setattr(constants, name, models)
    monkeypatch.setattr(constants, "EXO_MODELS_DIRS", (models,))
    monkeypatch.setattr(constants, "EXO_MODELS_READ_ONLY_DIRS", ())
    monkeypatch.setattr(constants, "EXO_EVENT_LOG_DIR", tmp_path / "event_log")
    monkeypatch.setattr(constants, "EXO_TRACING_CACHE_DIR", tmp_path / "traces")
    monkeypatch.setattr(constants, "EXO_CUSTOM_MODEL_CARDS_DIR", tmp_path / "cards")
    import exo_b200.api.main as api_main
    monkeypatch.setattr(api_main, "API_EVENT_LOG_DIR", tmp_path / "event_log" / "api")
    d = models / "org--tiny"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architectures": ["LlamaForCausalLM"], "hidden_size": 256, "num_hidden_layers": 4,
                                               "num_key_value_heads": 2, "max_position_embeddings": 2048}))
    (d / "model.safetensors").write_bytes(b"\0" * 1024)
    return tmp_path


async def wait_for(fn, timeout=30.0, what=""):
    with anyio.fail_after(timeout):
        while True:
            v = await fn()
            if v:
                return v
            await anyio.sleep(0.05)


def test_two_nodes_place_generate_in_every_dialect_and_delete(cluster_env):
    port = free_port()

    async def main():
        hub = LoopbackHub()
        ids = [NodeId("a" * 32), NodeId("b" * 32)]
        nodes = [Node(Args(spawn_api=(i == 0), api_port=port, force_master=(i == 0), gpu=i, no_downloads=False, offline=True),
                      ids[i], make_router(ids[i], hub.attach(ids[i]))) for i in range(2)]
        async with anyio.create_task_group() as tg:
            for n in nodes:
                tg.start_soon(n.run)
            async with httpx.AsyncClient(base_url=f"http://127.0.0.1:{port}", timeout=30) as http:
                async def ready():
                    try:
                        st = (await http.get("/state")).json()
                    except httpx.TransportError:
                        return None
                    ok = len(st["nodeBackends"]) == 2 and len(st["nodeMemory"]) == 2 and len(st["nodeNvlink"]) == 2
                    return st if ok and len(st["topology"]["connections"]) > 0 else None
                st = await wait_for(ready)
                assert (await http.get("/node_id")).json() == ids[0]
                # the dashboard (one static page that polls /state) is served from the root
                page = await http.get("/")
                assert page.status_code == 200 and "exo-b200" in page.text and "/instance/previews" in page.text
                # previews offer 1- and 2-GPU placements; the tensor one spans both nodes
                pv = (await http.get("/instance/previews", params={"model_id": "org/tiny"})).json()["previews"]
                sizes = sorted({len(p["instance"]["NvlinkInstance"]["shardAssignments"]["nodeToRunner"]) for p in pv if p["instance"]})
                assert sizes == [1, 2], pv
                r = await http.post("/place_instance", json={"model_id": "org/tiny", "sharding": "Tensor", "min_nodes": 2})
                assert r.status_code == 200, r.text

                async def instance_ready():
                    st = (await http.get("/state")).json()
                    runners = st["runners"]
                    return len(runners) == 2 and all("RunnerReady" in v for v in runners.values())
                await wait_for(instance_ready, 60)
                # OpenAI chat, non-streaming and streaming
                body = {"model": "org/tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}
                r = await http.post("/v1/chat/completions", json=body)
                assert r.status_code == 200, r.text
                msg = r.json()["choices"][0]
                assert msg["message"]["content"] == "tok0 tok1 tok2 tok3 " and msg["finish_reason"] == "stop"
                async with http.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as s:
                    lines = [ln async for ln in s.aiter_lines() if ln.startswith("data: ")]
                assert lines[-1] == "data: [DONE]"
                deltas = [json.loads(ln[6:])["choices"][0]["delta"].get("content", "") for ln in lines[:-1]]
                assert "".join(deltas) == "tok0 tok1 tok2 tok3 "
                # Claude
                r = await http.post("/v1/messages", json={"model": "org/tiny", "max_tokens": 4, "messages": [{"role": "user", "content": "hi"}]})
                assert r.status_code == 200 and r.json()["content"][0]["text"].startswith("tok0") and r.json()["stop_reason"] == "end_turn"
                # Responses
                r = await http.post("/v1/responses", json={"model": "org/tiny", "input": "hi", "max_output_tokens": 4})
                assert r.status_code == 200 and r.json()["output_text"].startswith("tok0") and r.json()["status"] == "completed"
                # Ollama (ndjson stream by default)
                r = await http.post("/ollama/api/chat", content=json.dumps({"model": "org/tiny", "messages": [{"role": "user", "content": "hi"}]}))
                objs = [json.loads(x) for x in r.text.strip().splitlines()]
                assert objs[-1]["done"] and objs[-1]["done_reason"] == "stop" and "".join(o["message"]["content"] for o in objs).startswith("tok0")
                assert (await http.get("/ollama/api/ps")).json()["models"][0]["name"] == "org/tiny"
                assert any(m["id"] == "org/tiny" for m in (await http.get("/v1/models", params={"status": "downloaded"})).json()["data"])
                # unknown model -> 404 in the error envelope
                r = await http.post("/v1/chat/completions", json={**body, "model": "org/none"})
                assert r.status_code == 404 and "No instance found" in r.json()["error"]["message"]
                # bench endpoint reports stats-bearing response shape
                r = await http.post("/bench/chat/completions", json=body)
                assert r.status_code == 200 and "power_usage" in r.json()
                # the benchmark tool drives the same endpoint (blocking client, so off the event loop)
                from exo_b200.bench import exo_bench
                out_file = cluster_env / "bench.jsonl"
                rc = await anyio.to_thread.run_sync(lambda: exo_bench.main(
                    ["--port", str(port), "--model", "org/tiny", "--pp", "1", "--tg", "4", "--concurrency", "1,2", "--warmup", "0",
                     "--json-out", str(out_file)]))
                rows = [json.loads(ln) for ln in out_file.read_text().splitlines()]
                assert rc == 0 and [r["concurrency"] for r in rows] == [1, 2] and len(rows[1]["requests"]) == 2
                # delete: runners shut down, instance disappears
                iid = next(iter((await http.get("/state")).json()["instances"]))
                assert (await http.delete(f"/instance/{iid}")).status_code == 200

                async def gone():
                    st = (await http.get("/state")).json()
                    return not st["instances"] and not st["runners"]
                await wait_for(gone, 30)
                evs = (await http.get("/events")).json()
                assert any("InstanceCreated" in e for e in evs) and any("InstanceDeleted" in e for e in evs)
            for n in nodes:
                n._tg.cancel_tasks()
            tg.cancel_scope.cancel()
    anyio.run(main)
