"""Answer-quality evaluation of a model served by a running cluster.

Counterpart of the reference's ``bench/exo_eval.py``: the same six suites, scored the same way —

=================  ======  ==============================================================================
suite              kind    scoring
=================  ======  ==============================================================================
``gpqa_diamond``   mc      4 shuffled choices, last ``Answer: X`` line
``mmlu_pro``       mc      up to 10 choices, last ``Answer: X`` line
``aime_2024/25``   math    integer inside the last ``\\boxed{}``
``humaneval``      code    completed function + the problem's ``check`` run in a child interpreter
``livecodebench``  code    program run against every stdin/stdout (or call-based) test, per-test time limit
``custom``         mc/em   a JSONL file of ``{"question","choices","answer"}`` or ``{"prompt","answer"}``
=================  ======  ==============================================================================

Datasets are read from ``--data-dir`` (``<suite>.jsonl`` or ``<suite>.parquet``, one record per problem in the
published column layout); nothing is downloaded.  Requests go through ``/v1/chat/completions`` with ``--num-concurrent``
in flight, each retried with back-off while the instance stays healthy.  Every finished question is appended to a
checkpoint file at once, so an interrupted run resumes where it stopped (``--force`` starts over).  Reasoning models
get the reasoning preset (temperature 0.6, top-p 0.95, long outputs), others greedy decoding; every sampling knob can be
overridden.  ``--compare-concurrency 1,4`` repeats a suite at several concurrencies and prints accuracy and
throughput side by side.

Code suites run model-written programs: in a child process with CPU-time, address-space and wall-clock limits, an
empty environment and a scratch working directory.  Use a throw-away machine all the same.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import re
import string
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable

from .client import ApiError, ExoClient

LETTERS = string.ascii_uppercase


# ---------------------------------------------------------------------------------------------------------------------
# answer extraction
# ---------------------------------------------------------------------------------------------------------------------
def extract_choice(text: str, letters: str = "ABCD") -> str | None:
    """The letter of the last ``Answer: X`` in the reply; failing that, a reply that is just a letter."""
    found = re.findall(r"(?i)answer\s*[:：]\s*\**\s*\(?([%s])\)?" % letters, text)
    if found:
        return found[-1].upper()
    m = re.fullmatch(r"\s*\(?([%s])\)?[.)]?\s*" % letters, text.strip(), flags=re.I)
    return m.group(1).upper() if m else None


def extract_letter(text: str, n: int) -> int | None:
    """Index of the first stand-alone choice letter (short-answer prompts of the ``custom`` suite)."""
    m = re.search(r"\b([A-%s])\b" % LETTERS[n - 1], text.strip().upper())
    return LETTERS.index(m.group(1)) if m else None


def extract_boxed(text: str) -> str | None:
    """Content of the last ``\\boxed{...}`` with balanced braces."""
    at = text.rfind("\\boxed")
    if at < 0:
        return None
    i = text.find("{", at)
    if i < 0:
        return None
    depth = 0
    for j in range(i, len(text)):
        depth += text[j] == "{"
        depth -= text[j] == "}"
        if depth == 0:
            return text[i + 1:j].strip()
    return None


def integer_answer_matches(extracted: str | None, gold: int) -> bool:
    if extracted is None:
        return False
    s = re.sub(r"\\text\{[^}]*\}|\\[,;! ]|[$\s]", "", extracted).replace(",", "").lstrip("0") or "0"
    try:
        return int(float(s)) == int(gold) and float(s) == int(float(s))
    except ValueError:
        return False


def extract_code(text: str, keep_indent: bool = False) -> str | None:
    """The last fenced block (``python`` or untagged); a reply without fences counts as code in whole."""
    blocks = re.findall(r"```(?:python|py)?[ \t]*\n(.*?)```", text, flags=re.S | re.I)
    if blocks:
        return blocks[-1] if keep_indent else blocks[-1].strip("\n")
    return text if ("def " in text or "print(" in text or "input(" in text) else None


def normalise(s: str) -> str:
    return re.sub(r"\s+", " ", s.strip().lower().strip(string.punctuation))


# ---------------------------------------------------------------------------------------------------------------------
# running model-written code
# ---------------------------------------------------------------------------------------------------------------------
def _limits(cpu_s: int, mem_bytes: int) -> Callable[[], None]:
    def apply() -> None:
        import resource
        resource.setrlimit(resource.RLIMIT_CPU, (cpu_s, cpu_s + 1))
        resource.setrlimit(resource.RLIMIT_AS, (mem_bytes, mem_bytes))
        resource.setrlimit(resource.RLIMIT_NPROC, (64, 64)) if hasattr(resource, "RLIMIT_NPROC") else None
        os.setsid()
    return apply


def run_python(source: str, stdin: str = "", timeout: float = 10.0, mem_bytes: int = 2 << 30) -> tuple[bool, str, str]:
    """``(exited 0 in time, stdout, stderr tail)`` of ``source`` in a fresh interpreter under resource limits."""
    with tempfile.TemporaryDirectory(prefix="exo-eval-") as tmp:
        path = Path(tmp) / "prog.py"
        path.write_text(source)
        try:
            p = subprocess.run([sys.executable, "-I", str(path)], input=stdin, capture_output=True, text=True, cwd=tmp,
                               timeout=timeout, env={"PATH": "/usr/bin:/bin"}, preexec_fn=_limits(int(timeout) + 1, mem_bytes))
        except subprocess.TimeoutExpired:
            return False, "", "timeout"
        return p.returncode == 0, p.stdout, p.stderr[-2000:]


def run_humaneval(problem: dict[str, Any], completion: str, timeout: float = 10.0) -> tuple[bool, str]:
    """The prompt's signature + the model's body (or its full re-definition), then the problem's ``check``."""
    body = completion
    if re.search(r"^\s*def\s+%s\s*\(" % re.escape(problem["entry_point"]), completion, flags=re.M):
        program = completion                                      # the model re-wrote the whole function
        imports = "\n".join(ln for ln in problem["prompt"].splitlines() if ln.startswith(("import ", "from ")))
        program = imports + "\n" + program
    else:
        if body and not body.startswith((" ", "\t")):
            body = "\n".join("    " + ln if ln.strip() else ln for ln in body.splitlines())
        program = problem["prompt"] + body
    ok, _out, err = run_python(f"{program}\n\n{problem['test']}\n\ncheck({problem['entry_point']})\n", timeout=timeout)
    return ok, err


def run_io_tests(code: str, tests: list[dict[str, Any]], fn_name: str | None = None, timeout: float = 6.0) -> tuple[bool, str]:
    """LiveCodeBench style: every test must pass.  ``stdin`` tests compare whitespace-normalised stdout; ``functional``
    tests call ``Solution().fn_name(*args)`` with JSON-line arguments and compare the JSON result."""
    for k, t in enumerate(tests):
        if t.get("testtype", "stdin") == "functional" and fn_name:
            args = [json.loads(ln) for ln in t["input"].splitlines() if ln.strip()]
            harness = (f"{code}\n\nimport json\n_args = json.loads({json.dumps(json.dumps(args))})\n"
                       f"_f = Solution().{fn_name} if 'Solution' in globals() else {fn_name}\n"
                       f"print(json.dumps(_f(*_args)))\n")
            ok, out, err = run_python(harness, timeout=timeout)
            try:
                same = ok and json.loads(out.strip().splitlines()[-1]) == json.loads(t["output"])
            except (ValueError, IndexError):
                same = False
        else:
            ok, out, err = run_python(code, stdin=t["input"], timeout=timeout)
            same = ok and out.split() == t["output"].split()
        if not same:
            return False, f"test {k}: {err or 'wrong output'}"
    return True, ""


# ---------------------------------------------------------------------------------------------------------------------
# suites
# ---------------------------------------------------------------------------------------------------------------------
MC_TAIL = ("Answer the following multiple choice question. The last line of your response should be in the following "
           "format: 'Answer: {opts}' (e.g. 'Answer: A').")
AIME_HEAD = ("Solve the following math problem step by step. Put your answer inside \\boxed{}.\n"
             "Remember to put your answer inside \\boxed{}.")
HUMANEVAL_HEAD = ("Complete the following Python function. Return only the function body inside a ```python code block. "
                  "Do not include the function signature.")
LCB_SYSTEM = ("You are an expert Python programmer. You will be given a question (problem specification) and will "
              "generate a correct Python program that matches the specification and passes all tests.")
LCB_STARTER = ("### Question:\n{q}\n\n### Format: You will use the following starter code to write the solution to the "
               "problem and enclose your code within delimiters.\n```python\n{starter}\n```\n\n"
               "### Answer: (use the provided format with backticks)\n")
LCB_STDIN = ("### Question:\n{q}\n\n### Format: Read the inputs from stdin solve the problem and write the answer to "
             "stdout (do not directly test on the sample inputs). Enclose your code within delimiters as follows. Ensure "
             "that when the python program runs, it reads the inputs, runs the algorithm and writes output to STDOUT.\n"
             "```python\n# YOUR CODE HERE\n```\n\n### Answer: (use the provided format with backticks)\n")


@dataclass
class Item:
    qid: str
    messages: list[dict[str, str]]
    gold: str
    check: Callable[[str], tuple[str | None, bool, str]]       # reply -> (extracted answer, correct, note)


def _mc_item(qid: str, question: str, choices: list[str], gold_index: int) -> Item:
    letters = LETTERS[:len(choices)]
    body = "\n".join(f"{letters[i]}) {c}" for i, c in enumerate(choices))
    prompt = MC_TAIL.format(opts="/".join(letters)) + f"\n\n{question}\n\n{body}"
    gold = letters[gold_index]

    def check(reply: str):
        got = extract_choice(reply, letters)
        return got, got == gold, ""
    return Item(qid, [{"role": "user", "content": prompt}], gold, check)


def gpqa_items(rows: list[dict[str, Any]]) -> list[Item]:
    out = []
    for i, r in enumerate(rows):
        choices = [r["Correct Answer"], r["Incorrect Answer 1"], r["Incorrect Answer 2"], r["Incorrect Answer 3"]]
        order = list(range(4))
        random.Random(i).shuffle(order)                           # the same permutation on every run
        out.append(_mc_item(str(r.get("Record ID", i)), r["Question"].strip(), [choices[j].strip() for j in order], order.index(0)))
    return out


def mmlu_pro_items(rows: list[dict[str, Any]]) -> list[Item]:
    return [_mc_item(str(r.get("question_id", i)), r["question"], [o for o in r["options"] if o != "N/A"], int(r["answer_index"]))
            for i, r in enumerate(rows)]


def aime_items(rows: list[dict[str, Any]]) -> list[Item]:
    out = []
    for i, r in enumerate(rows):
        gold = int(r.get("answer", r.get("Answer")))

        def check(reply: str, gold=gold):
            got = extract_boxed(reply)
            return got, integer_answer_matches(got, gold), ""
        out.append(Item(str(r.get("id", r.get("problem_idx", i))),
                        [{"role": "user", "content": AIME_HEAD + "\n\n" + r.get("problem", r.get("Problem", ""))}], str(gold), check))
    return out


def humaneval_items(rows: list[dict[str, Any]]) -> list[Item]:
    out = []
    for r in rows:
        def check(reply: str, r=r):
            code = extract_code(reply, keep_indent=True)
            if code is None:
                return None, False, "no code block"
            ok, err = run_humaneval(r, code)
            return code, ok, err
        out.append(Item(r["task_id"], [{"role": "user", "content": HUMANEVAL_HEAD + "\n\n```python\n" + r["prompt"] + "\n```"}],
                        "pass", check))
    return out


def livecodebench_items(rows: list[dict[str, Any]]) -> list[Item]:
    out = []
    for r in sorted(rows, key=lambda r: str(r.get("question_id", ""))):
        tests = r.get("public_test_cases") or []
        tests = json.loads(tests) if isinstance(tests, str) else tests
        private = r.get("private_test_cases")
        if isinstance(private, list):
            tests = tests + private
        meta = r.get("metadata") or {}
        meta = json.loads(meta) if isinstance(meta, str) else meta
        starter = r.get("starter_code") or ""
        user = (LCB_STARTER.format(q=r["question_content"], starter=starter) if starter
                else LCB_STDIN.format(q=r["question_content"]))

        def check(reply: str, tests=tests, fn=meta.get("func_name")):
            code = extract_code(reply)
            if code is None:
                return None, False, "no code block"
            ok, err = run_io_tests(code, tests, fn)
            return code, ok, err
        out.append(Item(str(r.get("question_id")), [{"role": "system", "content": LCB_SYSTEM}, {"role": "user", "content": user}],
                        "pass", check))
    return out


def custom_items(rows: list[dict[str, Any]]) -> list[Item]:
    out = []
    for i, r in enumerate(rows):
        if "choices" in r:
            opts = "\n".join(f"{LETTERS[j]}. {c}" for j, c in enumerate(r["choices"]))

            def check(reply: str, r=r):
                got = extract_letter(reply, len(r["choices"]))
                return (None if got is None else LETTERS[got]), got == int(r["answer"]), ""
            out.append(Item(str(i), [{"role": "user", "content": f"{r['question']}\n{opts}\nAnswer with the letter only."}],
                            LETTERS[int(r["answer"])], check))
        else:
            def check(reply: str, r=r):
                return reply.strip(), normalise(reply) == normalise(str(r["answer"])), ""
            out.append(Item(str(i), [{"role": "user", "content": r["prompt"]}], str(r["answer"]), check))
    return out


@dataclass(frozen=True)
class Suite:
    name: str
    kind: str
    about: str
    items: Callable[[list[dict[str, Any]]], list[Item]]


SUITES = {s.name: s for s in (
    Suite("gpqa_diamond", "mc", "graduate-level science, 198 questions, 4 choices", gpqa_items),
    Suite("mmlu_pro", "mc", "multi-task understanding, 12k questions, up to 10 choices", mmlu_pro_items),
    Suite("aime_2024", "math", "olympiad 2024, 30 problems, integer answers", aime_items),
    Suite("aime_2025", "math", "olympiad 2025, 30 problems, integer answers", aime_items),
    Suite("humaneval", "code", "164 Python functions, pass@1", humaneval_items),
    Suite("livecodebench", "code", "competitive programming, pass@1", livecodebench_items),
    Suite("custom", "mc", "a JSONL file of your own", custom_items))}


def score(q: dict[str, Any], reply: str) -> bool:
    """One ``custom`` record against a reply."""
    return custom_items([q])[0].check(reply)[1]


def load_rows(data_dir: Path, suite: str, file: str | None = None) -> list[dict[str, Any]]:
    cands = [Path(file)] if file else [data_dir / f"{suite}.jsonl", data_dir / f"{suite}.json", data_dir / f"{suite}.parquet"]
    for p in cands:
        if not p.exists():
            continue
        if p.suffix == ".parquet":
            import pyarrow.parquet as pq
            return pq.read_table(p).to_pylist()
        text = p.read_text()
        if p.suffix == ".json":
            return json.loads(text)
        return [json.loads(ln) for ln in text.splitlines() if ln.strip()]
    raise FileNotFoundError(f"no dataset for {suite!r}: looked for {', '.join(str(c) for c in cands)}")


# ---------------------------------------------------------------------------------------------------------------------
# running a suite
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Sampling:
    temperature: float = 0.0
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    max_tokens: int = 16384
    reasoning_effort: str | None = None
    enable_thinking: bool | None = None

    @classmethod
    def preset(cls, reasoning: bool) -> "Sampling":
        return cls(0.6, 0.95, None, None, 65536, "high", None) if reasoning else cls()

    def body(self) -> dict[str, Any]:
        b = {k: v for k, v in asdict(self).items() if v is not None}
        return b


@dataclass
class Result:
    question_id: str
    gold: str
    extracted: str | None = None
    correct: bool = False
    error: str | None = None
    note: str = ""
    response: str = ""
    reasoning_chars: int = 0
    prompt_tokens: int = 0
    completion_tokens: int = 0
    finish_reason: str = ""
    elapsed_s: float = 0.0
    attempts: int = 1


class InstanceFailed(RuntimeError):
    pass


def ask(client: ExoClient, model: str, item: Item, sampling: Sampling, timeout: float | None, retries: int = 4,
        healthy: Callable[[], bool] | None = None, sleep: Callable[[float], None] = time.sleep) -> Result:
    """One question: the request (retried with back-off on transport and 5xx errors while the instance is healthy),
    then the suite's check."""
    res = Result(item.qid, item.gold)
    body = {"model": model, "messages": item.messages, **sampling.body()}
    t0 = time.time()
    for attempt in range(1, retries + 1):
        res.attempts = attempt
        try:
            r = client.post("/v1/chat/completions", body, timeout=timeout)
            msg = r["choices"][0]["message"]
            res.response = msg.get("content") or ""
            res.reasoning_chars = len(msg.get("reasoning_content") or "")
            res.finish_reason = r["choices"][0].get("finish_reason") or ""
            usage = r.get("usage") or {}
            res.prompt_tokens, res.completion_tokens = usage.get("prompt_tokens", 0), usage.get("completion_tokens", 0)
            res.error = None
            break
        except ApiError as e:
            res.error = str(e)
            if e.status < 500 and e.status != 429:
                break                                          # the request itself is wrong: retrying cannot help
        except (OSError, ValueError, KeyError) as e:
            res.error = f"{type(e).__name__}: {e}"
        if healthy is not None and not healthy():
            raise InstanceFailed(f"instance of {model} is gone ({res.error})")
        sleep(min(30.0, 2.0 ** attempt))
    res.elapsed_s = time.time() - t0
    if res.error is None:
        try:
            res.extracted, res.correct, res.note = item.check(res.response)
            if res.extracted is not None:
                res.extracted = res.extracted[:4000]
        except Exception as e:  # noqa: BLE001 - a checker that chokes on a reply scores it wrong, with the reason
            res.note = f"checker: {type(e).__name__}: {e}"
    return res


class Checkpoint:
    """Append-only JSONL of finished questions; reading it back gives the results to skip."""

    def __init__(self, path: Path | None, fresh: bool = False):
        self.path, self.lock = path, threading.Lock()
        self.done: dict[str, Result] = {}
        if path is None:
            return
        if fresh and path.exists():
            path.unlink()
        if path.exists():
            for ln in path.read_text().splitlines():
                if ln.strip():
                    d = json.loads(ln)
                    if not d.get("error"):                     # failed requests are asked again
                        self.done[d["question_id"]] = Result(**d)

    def add(self, r: Result) -> None:
        if self.path is None:
            return
        with self.lock:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            with self.path.open("a") as f:
                f.write(json.dumps(asdict(r)) + "\n")


def run_suite(client: ExoClient, model: str, items: list[Item], sampling: Sampling, concurrency: int = 1,
              timeout: float | None = None, checkpoint: Checkpoint | None = None, healthy: Callable[[], bool] | None = None,
              progress: Callable[[Result, int, int], None] | None = None) -> list[Result]:
    checkpoint = checkpoint or Checkpoint(None)
    results: dict[str, Result] = {it.qid: checkpoint.done[it.qid] for it in items if it.qid in checkpoint.done}
    todo = [it for it in items if it.qid not in results]
    n_done = [len(results)]

    def work(it: Item) -> Result:
        r = ask(client, model, it, sampling, timeout, healthy=healthy)
        checkpoint.add(r)
        n_done[0] += 1
        if progress:
            progress(r, n_done[0], len(items))
        return r
    with ThreadPoolExecutor(max_workers=max(1, concurrency)) as pool:
        for r in pool.map(work, todo):
            results[r.question_id] = r
    return [results[it.qid] for it in items]


def summarise(name: str, results: list[Result], wall_s: float, concurrency: int) -> dict[str, Any]:
    answered = [r for r in results if r.error is None]
    toks = sum(r.completion_tokens for r in answered)
    return {"suite": name, "n": len(results), "answered": len(answered), "errors": len(results) - len(answered),
            "correct": sum(r.correct for r in answered),
            "accuracy": (sum(r.correct for r in answered) / len(answered)) if answered else None,
            "no_answer": sum(r.extracted is None for r in answered),
            "truncated": sum(r.finish_reason == "length" for r in answered),
            "completion_tokens": toks, "mean_completion_tokens": toks / len(answered) if answered else 0.0,
            "wall_s": wall_s, "tokens_per_s": toks / wall_s if wall_s > 0 else 0.0, "concurrency": concurrency}


def table(rows: list[dict[str, Any]]) -> str:
    head = ("suite", "conc", "n", "acc", "err", "no-ans", "trunc", "tok/q", "tok/s", "wall")
    lines = [head] + [(r["suite"], str(r["concurrency"]), str(r["n"]),
                       "-" if r["accuracy"] is None else f"{100 * r['accuracy']:.1f}%", str(r["errors"]), str(r["no_answer"]),
                       str(r["truncated"]), f"{r['mean_completion_tokens']:.0f}", f"{r['tokens_per_s']:.1f}", f"{r['wall_s']:.0f}s")
                      for r in rows]
    w = [max(len(ln[i]) for ln in lines) for i in range(len(head))]
    return "\n".join("  ".join(c.ljust(w[i]) for i, c in enumerate(ln)) for ln in lines)


def looks_like_reasoning_model(client: ExoClient, model: str) -> bool:
    try:
        for m in client.get("/v1/models").get("data", []):
            if m.get("id") == model:
                return bool(m.get("supports_thinking") or "thinking" in (m.get("capabilities") or []))
    except (ApiError, OSError, ValueError):
        pass
    return any(k in model.lower() for k in ("thinking", "reason", "-r1", "qwq", "gpt-oss", "deepseek-v3.2", "deepseek-v4"))


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="exo-eval", description=__doc__.split("\n\n")[0])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=52415)
    ap.add_argument("--model", required=True)
    ap.add_argument("--tasks", required=True, help="comma-separated suites (%s), or a JSONL path for the custom suite" % ", ".join(SUITES))
    ap.add_argument("--data-dir", default=os.environ.get("EXO_EVAL_DATA", "eval_data"))
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--offset", type=int, default=0)
    g = ap.add_mutually_exclusive_group()
    g.add_argument("--reasoning", action="store_true", default=None, help="reasoning preset (temperature 0.6, top-p 0.95, 65536 tokens)")
    g.add_argument("--no-reasoning", action="store_true", help="greedy preset (temperature 0, 16384 tokens)")
    ap.add_argument("--temperature", type=float)
    ap.add_argument("--top-p", type=float)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--min-p", type=float)
    ap.add_argument("--max-tokens", type=int)
    ap.add_argument("--reasoning-effort", choices=["low", "medium", "high"])
    ap.add_argument("--enable-thinking", type=lambda v: v.lower() in ("1", "true", "yes"))
    ap.add_argument("--no-thinking", action="store_true")
    ap.add_argument("--num-concurrent", "--concurrency", type=int, default=1)
    ap.add_argument("--compare-concurrency", default=None, help="e.g. 1,4: repeat every suite at each level")
    ap.add_argument("--request-timeout", type=float, default=None)
    ap.add_argument("--difficulty", choices=["easy", "medium", "hard"], help="livecodebench only")
    ap.add_argument("--release-version", help="livecodebench only")
    ap.add_argument("--results-dir", default="eval_results")
    ap.add_argument("--force", action="store_true", help="discard checkpoints")
    ap.add_argument("--place", action="store_true", help="place an instance first and delete it afterwards")
    ap.add_argument("--sharding", default="Tensor")
    ap.add_argument("--min-nodes", type=int, default=1)
    a = ap.parse_args(argv)

    client = ExoClient(a.host, a.port)
    placed = None
    if a.place:
        client.place(a.model, a.sharding, a.min_nodes)
        placed = client.wait_ready(a.model)
    reasoning = a.reasoning if a.reasoning is not None else (False if a.no_reasoning else looks_like_reasoning_model(client, a.model))
    sampling = Sampling.preset(bool(reasoning))
    for k in ("temperature", "top_p", "top_k", "min_p", "max_tokens", "reasoning_effort", "enable_thinking"):
        if getattr(a, k) is not None:
            setattr(sampling, k, getattr(a, k))
    if a.no_thinking:
        sampling.enable_thinking = False

    def healthy() -> bool:
        try:
            return bool(client.instances_of(a.model))
        except (ApiError, OSError, ValueError):
            return False
    levels = [int(x) for x in a.compare_concurrency.split(",")] if a.compare_concurrency else [a.num_concurrent]
    out_dir = Path(a.results_dir)
    summaries = []
    try:
        for task in a.tasks.split(","):
            name, file = (task, None) if task in SUITES else ("custom", task)
            rows = load_rows(Path(a.data_dir), name, file)
            if a.difficulty:
                rows = [r for r in rows if r.get("difficulty") == a.difficulty]
            if a.release_version:
                rows = [r for r in rows if r.get("release_version") == a.release_version]
            items = SUITES[name].items(rows)[a.offset:]
            if a.limit:
                items = items[:a.limit]
            if SUITES[name].kind == "code":
                print("note: this suite executes model-written code in child processes", file=sys.stderr)
            for conc in levels:
                tag = f"{a.model.replace('/', '--')}_{name}_c{conc}"
                ck = Checkpoint(out_dir / f"{tag}.checkpoint.jsonl", fresh=a.force)
                t0 = time.time()
                res = run_suite(client, a.model, items, sampling, conc, a.request_timeout, ck, healthy,
                                lambda r, i, n: print(f"[{name} c{conc}] {i}/{n} {'ok ' if r.correct else ('ERR' if r.error else 'no ')}"
                                                      f" {r.question_id} {r.elapsed_s:.1f}s", file=sys.stderr))
                s = summarise(name, res, time.time() - t0, conc)
                summaries.append(s)
                out_dir.mkdir(parents=True, exist_ok=True)
                (out_dir / f"{tag}.json").write_text(json.dumps({"model": a.model, "sampling": asdict(sampling), "summary": s,
                                                                  "results": [asdict(r) for r in res]}, indent=1))
    except InstanceFailed as e:
        print(f"stopped: {e}", file=sys.stderr)
        return 2
    finally:
        if placed:
            client.delete_instance(placed)
    print(table(summaries))
    print(json.dumps({"model": a.model, "summaries": summaries}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
