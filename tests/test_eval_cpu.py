"""The evaluation tool without a cluster: answer extraction, the code sandbox, retries, checkpoint resume."""
import json

import pytest

from exo_b200.bench import exo_eval as ev
from exo_b200.bench.client import ApiError


def test_answer_extractors():
    assert ev.extract_choice("Let me think.\nAnswer: B\nActually...\nAnswer: (C)") == "C"
    assert ev.extract_choice("**Answer:** d") == "D" and ev.extract_choice("b") == "B"
    assert ev.extract_choice("I think it is B or C") is None
    assert ev.extract_choice("Answer: J", "ABCDEFGHIJ") == "J" and ev.extract_choice("Answer: J", "ABCD") is None
    assert ev.extract_boxed(r"so \boxed{1} then \boxed{\frac{3}{4}}") == r"\frac{3}{4}"
    assert ev.extract_boxed("no box") is None and ev.extract_boxed(r"\boxed{unbalanced") is None
    assert ev.integer_answer_matches("042", 42) and ev.integer_answer_matches(r"1,\!024", 1024)
    assert ev.integer_answer_matches("1,024", 1024) and ev.integer_answer_matches("$73$", 73)
    assert not ev.integer_answer_matches("7.5", 7) and not ev.integer_answer_matches(None, 1)
    assert ev.extract_code("x\n```python\na = 1\n```\ny\n```\nb = 2\n```") == "b = 2"
    assert ev.extract_code("    return 1\n", keep_indent=True) is None
    assert ev.extract_code("def f():\n    return 1") == "def f():\n    return 1"


def test_suites_build_prompts_and_score():
    gp = ev.gpqa_items([{"Question": "2+2?", "Correct Answer": "4", "Incorrect Answer 1": "3", "Incorrect Answer 2": "5",
                         "Incorrect Answer 3": "22"}])[0]
    assert "Answer: A/B/C/D" in gp.messages[0]["content"] and gp.messages[0]["content"].count(") ") >= 4
    line = next(ln for ln in gp.messages[0]["content"].splitlines() if ln.endswith(") 4"))
    assert line[0] == gp.gold and gp.check(f"Answer: {gp.gold}")[1] and not gp.check("Answer: " + "ABCD".replace(gp.gold, "")[0])[1]
    assert ev.gpqa_items([{"Question": "2+2?", "Correct Answer": "4", "Incorrect Answer 1": "3", "Incorrect Answer 2": "5",
                           "Incorrect Answer 3": "22"}])[0].gold == gp.gold           # the shuffle is the same on every run
    mm = ev.mmlu_pro_items([{"question_id": 7, "question": "q", "options": ["a", "b", "c", "N/A"], "answer_index": 2}])[0]
    assert mm.gold == "C" and "A/B/C'" in mm.messages[0]["content"] and mm.qid == "7"
    am = ev.aime_items([{"id": 3, "problem": "p", "answer": "204"}])[0]
    assert am.check(r"thus \boxed{204}") == ("204", True, "") and not am.check("204")[1]
    assert ev.score({"question": "q", "choices": ["x", "y"], "answer": 1}, "B") and ev.score({"prompt": "p", "answer": "Paris"}, " paris. ")


HUMANEVAL = {"task_id": "HumanEval/0", "entry_point": "add", "prompt": "def add(a, b):\n    \"\"\"sum\"\"\"\n",
             "test": "def check(f):\n    assert f(2, 3) == 5\n    assert f(-1, 1) == 0\n"}


def test_code_suites_run_programs_under_limits():
    it = ev.humaneval_items([HUMANEVAL])[0]
    assert it.check("```python\n    return a + b\n```")[1]
    assert it.check("```python\nreturn a + b\n```")[1]                              # unindented body
    assert it.check("```python\ndef add(a, b):\n    return a + b\n```")[1]          # whole function again
    assert not it.check("```python\n    return a - b\n```")[1]
    assert it.check("I cannot")[2] == "no code block"
    ok, _out, err = ev.run_python("while True:\n    pass\n", timeout=1.0)
    assert not ok and err == "timeout"
    ok, _out, _err = ev.run_python("x = bytearray(3 << 30)\n", timeout=5.0, mem_bytes=1 << 30)
    assert not ok
    lcb = ev.livecodebench_items([
        {"question_id": "b", "question_content": "sum two ints", "starter_code": "",
         "public_test_cases": json.dumps([{"input": "1 2\n", "output": "3\n", "testtype": "stdin"}]), "metadata": "{}"},
        {"question_id": "a", "question_content": "double", "starter_code": "class Solution:\n    def twice(self, x):\n",
         "public_test_cases": json.dumps([{"input": "[1, 2]\n", "output": "[1, 2, 1, 2]", "testtype": "functional"}]),
         "metadata": json.dumps({"func_name": "twice"})}])
    assert [i.qid for i in lcb] == ["a", "b"] and lcb[0].messages[0]["role"] == "system"
    assert "starter code" in lcb[0].messages[1]["content"] and "stdin" in lcb[1].messages[1]["content"]
    assert lcb[1].check("```python\na, b = map(int, input().split())\nprint(a + b)\n```")[1]
    assert not lcb[1].check("```python\nprint(0)\n```")[1]
    assert lcb[0].check("```python\nclass Solution:\n    def twice(self, x):\n        return x + x\n```")[1]


class Flaky:
    """Fails twice with a 503, then answers; counts the requests per question."""

    def __init__(self, fail=2):
        self.calls, self.fail = {}, fail

    def post(self, path, body, timeout=None):
        q = body["messages"][-1]["content"]
        self.calls[q] = self.calls.get(q, 0) + 1
        if self.calls[q] <= self.fail:
            raise ApiError(503, "busy")
        return {"choices": [{"message": {"content": "Answer: A", "reasoning_content": "hm"}, "finish_reason": "stop"}],
                "usage": {"prompt_tokens": 5, "completion_tokens": 3}}


def test_retries_checkpoint_and_resume(tmp_path):
    items = ev.custom_items([{"question": f"q{i}", "choices": ["x", "y"], "answer": i % 2} for i in range(6)])
    naps = []
    r = ev.ask(Flaky(), "m", items[0], ev.Sampling(), None, sleep=naps.append)
    assert r.correct and r.attempts == 3 and naps == [2.0, 4.0] and r.completion_tokens == 3 and r.reasoning_chars == 2

    class Bad:
        def post(self, *a, **k):
            raise ApiError(400, "bad request")
    r = ev.ask(Bad(), "m", items[0], ev.Sampling(), None, sleep=naps.append)
    assert r.error and r.attempts == 1                        # a 4xx is not retried
    with pytest.raises(ev.InstanceFailed):
        ev.ask(Flaky(fail=9), "m", items[0], ev.Sampling(), None, healthy=lambda: False, sleep=naps.append)

    path = tmp_path / "ck.jsonl"
    c1 = Flaky(fail=0)
    first = ev.run_suite(c1, "m", items[:4], ev.Sampling(), 2, checkpoint=ev.Checkpoint(path))
    assert len(path.read_text().splitlines()) == 4 and sum(r.correct for r in first) == 2
    c2 = Flaky(fail=0)
    again = ev.run_suite(c2, "m", items, ev.Sampling(), 2, checkpoint=ev.Checkpoint(path))
    assert len(c2.calls) == 2 and [r.question_id for r in again] == [str(i) for i in range(6)]      # only the new questions were asked
    s = ev.summarise("custom", again, 2.0, 2)
    assert s["n"] == 6 and s["correct"] == 3 and s["accuracy"] == 0.5 and s["tokens_per_s"] == 9.0
    assert "50.0%" in ev.table([s])
    assert len(ev.run_suite(Flaky(fail=0), "m", items, ev.Sampling(), 1, checkpoint=ev.Checkpoint(path, fresh=True))) == 6
    assert ev.Sampling.preset(True).body()["temperature"] == 0.6 and "top_p" not in ev.Sampling.preset(False).body()


def test_load_rows_reads_jsonl_and_parquet(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    (tmp_path / "aime_2024.jsonl").write_text('{"id": 1, "problem": "p", "answer": 7}\n')
    assert ev.load_rows(tmp_path, "aime_2024") == [{"id": 1, "problem": "p", "answer": 7}]
    pq.write_table(pa.table({"question": ["q"], "options": [["a", "b"]], "answer_index": [1]}), tmp_path / "mmlu_pro.parquet")
    assert ev.mmlu_pro_items(ev.load_rows(tmp_path, "mmlu_pro"))[0].gold == "B"
    with pytest.raises(FileNotFoundError):
        ev.load_rows(tmp_path, "humaneval")
