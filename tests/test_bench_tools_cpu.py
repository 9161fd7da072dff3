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
