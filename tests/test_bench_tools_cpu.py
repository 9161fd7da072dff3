"""Benchmark / evaluation tool logic that needs no cluster."""
from exo_b200.bench.eval_tool_calls import BUILTIN, score_call
from exo_b200.bench.exo_bench import aggregate, build_prompt
from exo_b200.bench.exo_eval import extract_letter, score


def test_prompt_sizing_hits_exact_token_counts():
    overhead = 11                                   # chat-template tokens around the content
    count = lambda s: overhead + len(s) // 2        # "a " is one token
    for target in (64, 512, 4096):
        content, n = build_prompt(count, target)
        assert n == target and count(content) == target
    # a tokenizer that merges atoms cannot hit every count: the closest one is returned
    lumpy = lambda s: overhead + (len(s) // 2) // 3 * 3
    _, n = build_prompt(lumpy, 100)
    assert abs(n - 100) <= 2


def test_aggregate_uses_fastest_stream_times_concurrency():
    rows = [{"generation_tps": 40.0, "prompt_tps": 1000.0, "elapsed_s": 3.0, "pp_tokens": 512, "tg_tokens": 128},
            {"generation_tps": 50.0, "prompt_tps": 3000.0, "elapsed_s": 3.5, "pp_tokens": 512, "tg_tokens": 128}]
    a = aggregate(rows, 2)
    assert a["per_req_gen_tps"] == 50.0 and a["agg_gen_tps"] == 100.0 and a["batch_wall_s"] == 3.5 and a["mean_prompt_tps"] == 2000.0


def test_tool_call_and_answer_scoring():
    sc = BUILTIN[1]
    assert all(score_call("add", '{"a": 17, "b": 25}', sc).values())
    assert not score_call("add", '{"a": "17", "b": 25}', sc)["args_ok"]       # wrong JSON type
    assert not score_call("add", '{"a": 17}', sc)["args_ok"]                 # missing required key
    assert not score_call("get_weather", '{"city": "x"}', sc)["name_ok"]
    assert score_call(None, None, sc) == {"called": False, "name_ok": False, "json_ok": False, "args_ok": False}
    assert not score_call("add", "{not json", sc)["json_ok"]
    assert extract_letter("I think the answer is (c).", 4) == 2 and extract_letter("no idea", 4) is None
    assert score({"question": "q", "choices": ["x", "y"], "answer": 0}, "A") and not score({"prompt": "p", "answer": "4"}, "five")


def test_prefill_decode_bench_planning_and_tables(tmp_path):
    from exo_b200.bench import prefill_decode_bench as pdb

    def preview(nodes, sharding="Tensor", error=None):
        inst = {"NvlinkInstance": {"shardAssignments": {"nodeToRunner": {n: f"r{n}" for n in nodes}}}}
        return {"sharding": sharding, "instance": None if error else inst, "error": error}
    prev = [preview(["a", "b"]), preview(["a"]), preview(["b"], error="no memory"), preview(["b"], "Pipeline"), preview(["c"])]
    a, b = pdb.pick_disjoint(prev, "Tensor", 1)
    assert pdb.nodes_of(a["instance"]) == {"a"} and pdb.nodes_of(b["instance"]) == {"c"}
    assert pdb.pick_disjoint(prev[:4], "Tensor", 1) is None
    rows = [{"phase": "baseline", "pp": 2048, "tg": 128, "ttft_s": t, "prompt_tps": 2048 / t, "generation_tps": 50.0, "elapsed_s": t + 2.56}
            for t in (0.5, 0.7, 0.6)]
    base = pdb.summarise(rows)
    assert base[(2048, 128)]["ttft_s"] == 0.6
    dis = {(2048, 128): {"ttft_s": 0.3, "prompt_tps": 6826.0, "generation_tps": 55.0, "elapsed_s": 2.6}}
    text = pdb.diff_table(base, dis)
    assert "2.00" in text and "1.10" in text and text.splitlines()[0].split()[0] == "pp"
    cfg = tmp_path / "pd.toml"
    cfg.write_text('[defaults]\nmodel = "org/m"\npp = "1024,4096"\nrepeat = 3\n')
    a = pdb.parse_args(["--config", str(cfg), "--tg", "64"])
    assert (a.model, pdb.ints(a.pp), a.repeat, pdb.ints(a.tg)) == ("org/m", [1024, 4096], 3, [64])


class FakeCluster:
    """The slice of the HTTP API the harness uses, in memory."""

    def __init__(self):
        gib = 1 << 30
        self.models = [{"hugging_face_id": "meta-llama/Llama-3.1-8B-Instruct", "storage_size_megabytes": 16 * 1024},
                       {"hugging_face_id": "meta-llama/Llama-3.1-70B-Instruct", "storage_size_megabytes": 140 * 1024},
                       {"hugging_face_id": "Qwen/Qwen3-8B", "storage_size_megabytes": 16 * 1024}]
        shard = lambda m: {"TensorShardMetadata": {"modelCard": {"modelId": m}}}
        self.state_ = {"instances": {}, "runners": {}, "nodeDisk": {"n1": {"available": {"inBytes": 20 * gib}}, "n2": {"available": {"inBytes": 4 * gib}}},
                       "downloads": {"n1": [], "n2": [{"DownloadCompleted": {"shardMetadata": shard("Qwen/Qwen3-8B"), "total": {"inBytes": 16 * gib}}},
                                                      {"DownloadCompleted": {"shardMetadata": shard("org/small"), "total": {"inBytes": 1 * gib}}}]},
                       "nodeMemory": {"n1": {}, "n2": {}}}
        self.preview_calls, self.deleted, self.started = 0, [], []
        self.shard = shard

    def get(self, path, **params):
        if path == "/models":
            return {"data": self.models}
        raise KeyError(path)

    def previews(self, model_id):
        self.preview_calls += 1
        if self.preview_calls < 3:
            return []                                  # the second node has not joined yet
        inst = lambda nodes: {"NvlinkInstance": {"shardAssignments": {"modelId": model_id, "nodeToRunner": {n: "r" + n for n in nodes},
                                                                      "runnerToShard": {"r" + n: self.shard(model_id) for n in nodes}}}}
        return [{"sharding": "Tensor", "instance": inst(["n1", "n2"])}, {"sharding": "Pipeline", "instance": inst(["n1", "n2"])},
                {"sharding": "Tensor", "instance": inst(["n1"])}, {"sharding": "Tensor", "instance": None, "error": "no memory"}]

    def state(self):
        return self.state_

    def delete(self, path):
        node, model = path.split("/", 3)[2:]
        self.deleted.append((node, model))
        self.state_["downloads"][node] = [e for e in self.state_["downloads"][node]
                                          if next(iter(e["DownloadCompleted"]["shardMetadata"].values()))["modelCard"]["modelId"] != model]

    def post(self, path, body, timeout=None):
        if path == "/download/start":
            self.started.append(body["targetNodeId"])
            model = next(iter(body["shardMetadata"].values()))["modelCard"]["modelId"]
            self.state_["downloads"][body["targetNodeId"]].append({"DownloadCompleted": {"shardMetadata": self.shard(model), "total": {"inBytes": 1}}})
        elif path == "/instance":
            inst = body["instance"]
            self.state_["instances"]["i1"] = inst
            for r in next(iter(inst.values()))["shardAssignments"]["runnerToShard"]:
                self.state_["runners"][r] = {"RunnerReady": {}}

    def instances_of(self, model_id):
        return [(i, t) for i, t in self.state_["instances"].items() if next(iter(t.values()))["shardAssignments"]["modelId"] == model_id]

    def delete_instance(self, iid):
        self.state_["instances"].pop(iid)


def test_harness_resolves_places_frees_disk_downloads_and_launches():
    import argparse

    import pytest

    from exo_b200.bench.harness import Harness, add_instance_args
    fc = FakeCluster()
    logs: list[str] = []
    h = Harness(fc, log=logs.append, sleep=lambda s: None)
    assert h.resolve_model("Llama-3.1-8B-Instruct") == "meta-llama/Llama-3.1-8B-Instruct"
    assert h.resolve_model("qwen3-8b") == "Qwen/Qwen3-8B" and h.resolve_model("org/unknown") == "org/unknown"
    with pytest.raises(ValueError):
        h.resolve_model("llama-3.1")
    ap = argparse.ArgumentParser()
    add_instance_args(ap)
    a = ap.parse_args(["--model", "Llama-3.1-8B-Instruct", "--min-nodes", "2"])
    with pytest.raises(RuntimeError, match="GiB free"):             # n2 has 4 GiB free, the model needs 16
        h.instance_for(a)
    a = ap.parse_args(["--model", "Llama-3.1-8B-Instruct", "--min-nodes", "2", "--danger-delete-downloads"])
    model, iid, dl = h.instance_for(a)
    assert model == "meta-llama/Llama-3.1-8B-Instruct" and iid == "i1" and dl is not None
    assert fc.preview_calls >= 3 and any("no placement" in ln for ln in logs)       # waited for the cluster to settle
    assert fc.deleted == [("n2", "org/small"), ("n2", "Qwen/Qwen3-8B")] and sorted(fc.started) == ["n1", "n2"]   # smallest first
    snap = h.snapshot()
    assert snap["instances"]["i1"]["nodes"] == ["n1", "n2"] and snap["instances"]["i1"]["kind"] == "NvlinkInstance"
    a2 = ap.parse_args(["--model", "Llama-3.1-8B-Instruct", "--reuse-instance"])
    assert h.instance_for(a2)[1] == "i1"
    h.teardown()
    assert not fc.state_["instances"]
    assert len(h.placements(model, "Pipeline", "nvlink", 1, 0, 1.0)) == 1 and h.placements(model, "Tensor", "ring", 1, 0, 0.0) == []


def test_tool_call_eval_runs_every_dialect_with_followups_and_scenario_files(tmp_path):
    """The evaluator against a scripted HTTP server: chat / Messages / Responses request forms, history translation,
    a no-call scenario, the follow-up turn after a tool result, nested array arguments, scenario files."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer
    from exo_b200.bench import eval_tool_calls as etc
    from exo_b200.bench.client import ExoClient
    seen = []

    def answer(path, body):
        """Call `get_weather` / `add` / `write_todos` when the last turn asks for it; answer in text after a tool result."""
        seen.append((path, body))
        if path == "/v1/chat/completions":
            msgs, last = body["messages"], body["messages"][-1]
            after_result = last["role"] == "tool" and len([m for m in msgs if m["role"] == "tool"]) == (2 if "Rome" in msgs[0]["content"] else 1)
            text = msgs[0]["content"]
        elif path == "/v1/messages":
            last = body["messages"][-1]
            results = sum(b["type"] == "tool_result" for m in body["messages"] if isinstance(m["content"], list) for b in m["content"])
            text = body["messages"][0]["content"]
            after_result = isinstance(last["content"], list) and last["content"][0]["type"] == "tool_result" and results == (2 if "Rome" in text else 1)
        else:
            items = body["input"]
            text = items[0]["content"]
            after_result = items[-1].get("type") == "function_call_output" and \
                sum(i.get("type") == "function_call_output" for i in items) == (2 if "Rome" in text else 1)
        call = None
        if not after_result and "Do not use any tool" not in text:
            call = ("get_weather", {"city": "Rome" if "Rome" in text else "Paris"}) if "weather" in text else \
                ("write_todos", {"todos": [{"title": "buy milk", "done": False}, {"title": "call Ana", "done": True}]}) if "to-do" in text else \
                ("add", {"a": 17, "b": 25})
        if path == "/v1/chat/completions":
            m = {"role": "assistant", "content": None if call else "Bonjour / done."}
            if call:
                m["tool_calls"] = [{"id": "c9", "type": "function", "function": {"name": call[0], "arguments": json.dumps(call[1])}}]
            return {"choices": [{"message": m, "finish_reason": "tool_calls" if call else "stop"}]}
        if path == "/v1/messages":
            return {"content": [{"type": "tool_use", "id": "tu1", "name": call[0], "input": call[1]}] if call else [{"type": "text", "text": "Bonjour."}],
                    "stop_reason": "tool_use" if call else "end_turn"}
        return {"status": "completed", "output": [{"type": "function_call", "call_id": "fc1", "name": call[0], "arguments": json.dumps(call[1])}] if call
                else [{"type": "message", "content": [{"type": "output_text", "text": "Bonjour."}]}]}

    class H(BaseHTTPRequestHandler):
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            out = json.dumps(answer(self.path, body)).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def log_message(self, *a):
            pass
    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        c = ExoClient("127.0.0.1", srv.server_address[1])
        rows = [etc.run_scenario(c, "m", sc, d) for sc in etc.BUILTIN for d in ("chat", "claude", "responses")]
        assert all(r["passed"] for r in rows), [r for r in rows if not r["passed"]]
        s = etc.summarize(rows)
        assert s["passed"] == s["total"] == 15 and s["by_dialect"]["claude"] == {"passed": 5, "total": 5}
        assert sum(r.get("followup_ok", False) for r in rows) == 6                # weather and add, three dialects each
        # the history with an earlier call and its result reaches each dialect in its own form
        hist = [b for p, b in seen if p == "/v1/messages" and "Rome" in str(b["messages"][0]["content"])][0]["messages"]
        assert hist[1]["content"][0] == {"type": "tool_use", "id": "call_1", "name": "get_weather", "input": {"city": "Paris"}}
        assert hist[2]["content"][0]["type"] == "tool_result" and hist[2]["content"][0]["tool_use_id"] == "call_1"
        resp = [b for p, b in seen if p == "/v1/responses" and "Rome" in str(b["input"][0].get("content"))][0]["input"]
        assert [i.get("type", "message") for i in resp] == ["message", "function_call", "function_call_output"]
        # a model that calls a tool where none is wanted, or answers in text where one is, fails
        bad = etc.Scenario("x", [{"role": "user", "content": "What is the weather in Paris?"}], [etc.WEATHER], expect_call=False)
        assert not etc.run_scenario(c, "m", bad, "chat")["passed"]
        bad2 = etc.Scenario("y", [{"role": "user", "content": "Say hi. Do not use any tool."}], [etc.WEATHER], expect="get_weather", required=["city"])
        assert not etc.run_scenario(c, "m", bad2, "responses")["passed"]
    finally:
        srv.shutdown()
    # scenario files
    (tmp_path / "s.toml").write_text("""
[tools.lookup]
description = "Look a word up"
required = ["word"]
[tools.lookup.properties.word]
type = "string"

[[scenarios]]
name = "lookup"
description = "one call"
expect_tool_call = true
expected_function = "lookup"
required_arg_keys = ["word"]
tools = ["lookup"]
tool_result = { meaning = "a greeting" }
[[scenarios.messages]]
role = "user"
content = "Look up 'hello'."
[[scenarios.messages]]
role = "assistant"
tool_calls = [{ id = "a1", name = "lookup", arguments = { word = "hi" } }]
[[scenarios.messages]]
role = "tool"
tool_call_id = "a1"
content = "short for hello"
""")
    (sc,) = etc.load_scenarios(tmp_path / "s.toml")
    assert sc.expect == "lookup" and sc.tools[0]["function"]["parameters"]["required"] == ["word"] and sc.tool_result == {"meaning": "a greeting"}
    assert json.loads(sc.messages[1]["tool_calls"][0]["function"]["arguments"]) == {"word": "hi"} and sc.prompt == "Look up 'hello'."
    (tmp_path / "s.jsonl").write_text(json.dumps({"prompt": "add 1 and 2", "tools": [etc.CALC], "expect": "add", "required": ["a", "b"]}) + "\n")
    (sj,) = etc.load_scenarios(tmp_path / "s.jsonl")
    assert sj.messages == [{"role": "user", "content": "add 1 and 2"}] and all(etc.score_call("add", {"a": 1, "b": 2}, sj).values())
    todo = etc.BUILTIN[4]
    assert not etc.score_call("write_todos", {"todos": [{"title": "x"}]}, todo)["args_ok"]          # an item without `done`
    assert etc.score_call("write_todos", {"todos": json.dumps([{"title": "x", "done": True}])}, todo)["json_ok"]
    assert not etc.score_call("get_weather", {"city": "Paris", "unit": "kelvin"}, etc.BUILTIN[0])["args_ok"]   # outside the enum


def test_exo_bench_streaming_metrics_sampler_pairs_and_dry_run(capsys):
    """`exo_bench` against a scripted server: paired pp / tg lists, a streamed run with client-side timings, the GPU sampler
    on a fake NVML, and the dry run."""
    import json
    import threading
    import time
    from http.server import BaseHTTPRequestHandler, HTTPServer
    from exo_b200.bench import exo_bench as eb
    assert eb.plan_runs([512, 2048], [64, 128], False) == [(512, 64), (2048, 128)]
    assert len(eb.plan_runs([512, 2048], [64, 128], True)) == 4 and eb.plan_runs([512], [64, 128], False) == [(512, 64), (512, 128)]

    class Nvml:
        calls = 0

        def nvmlInit(self): pass
        def nvmlDeviceGetCount(self): return 2
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetUtilizationRates(self, h): Nvml.calls += 1; return type("U", (), {"gpu": 50 + 10 * h})()
        def nvmlDeviceGetTemperature(self, h, kind): return 60 + h
        def nvmlDeviceGetPowerUsage(self, h): return 700_000
        def nvmlDeviceGetClockInfo(self, h, kind): return 1900
    with eb.SystemMetricsSampler(0.01, nvml=Nvml()) as sm:
        time.sleep(0.4)
    s = sm.summary()
    assert s["samples"] >= 3 and s["gpus"][1]["util"] == {"mean": 60.0, "max": 60.0} and s["gpus"][0]["power_w"]["max"] == 700.0
    assert eb.SystemMetricsSampler(nvml=eb._NoNvml()).summary() is None
    bodies = []

    class H(BaseHTTPRequestHandler):
        def do_GET(self):
            out = json.dumps({"previews": [{"sharding": "Tensor", "instance_meta": "Nvlink", "error": None, "instance": {
                "NvlinkInstance": {"shardAssignments": {"nodeToRunner": {"a": "r0", "b": "r1"}}}}}, {"error": "no memory"}]}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            bodies.append(body)
            n_prompt = len(body["messages"][0]["content"]) // 2 + 5
            stats = {"prompt_tps": 1000.0, "generation_tps": 50.0, "prompt_tokens": n_prompt, "generation_tokens": body["max_tokens"]}
            self.send_response(200)
            if body.get("stream"):
                self.send_header("Content-Type", "text/event-stream")
                self.end_headers()
                for i in range(3):
                    self.wfile.write(("data: " + json.dumps({"choices": [{"delta": {"content": "x"}}]}) + "\n\n").encode())
                    self.wfile.flush()
                    time.sleep(0.01)
                self.wfile.write(("data: " + json.dumps({"choices": [{"delta": {}, "finish_reason": "length"}]}) + "\n\n").encode())
                self.wfile.write((": generation_stats " + json.dumps(stats) + "\n\n").encode())
                self.wfile.write(b"data: [DONE]\n\n")
                return
            out = json.dumps({"usage": {"prompt_tokens": n_prompt, "completion_tokens": body["max_tokens"]}, "generation_stats": stats}).encode()
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def log_message(self, *a):
            pass
    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    port = str(srv.server_address[1])
    try:
        assert eb.main(["--port", port, "--model", "m", "--pp", "64,128", "--tg", "4,8", "--dry-run"]) == 0
        dry = json.loads(capsys.readouterr().out)
        assert [(r["pp"], r["tg"]) for r in dry["runs"]] == [(64, 4), (128, 8)] and dry["placements"] == [
            {"sharding": "Tensor", "instance_meta": "Nvlink", "nodes": 2}]
        assert not bodies
        client = eb.ExoClient("127.0.0.1", int(port))
        r = eb.stream_request(client, "m", "a " * 20, 4, False)
        assert r["client_chunks"] == 3 and r["client_ttft_s"] > 0 and r["client_gap_ms_p50"] >= 5 and r["generation_tps"] == 50.0 and r["tg_tokens"] == 4
        rows = eb.concurrent_requests(lambda: eb.ExoClient("127.0.0.1", int(port)), 3, "m", "a " * 20, 4, False, eb.stream_request)
        assert len(rows) == 3 and all(x["client_chunks"] == 3 for x in rows) and eb.aggregate(rows, 3)["agg_gen_tps"] == 150.0
    finally:
        srv.shutdown()
