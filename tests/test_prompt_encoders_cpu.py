"""DeepSeek-V3.2 / V4 prompt formats: golden strings of the published layout, round trips through the parser, and the
way ``render_prompt`` selects them."""
import json

import pytest

from exo_b200.shared.messages import InputMessage, TextGenerationTaskParams
from exo_b200.worker.engines.b200.prompt_encoders import (ASSISTANT, BOS, DSML, EOS, MAX_EFFORT_PREAMBLE, USER, V4, V32,
                                                          DeepSeekPromptEncoder, encoder_for)
from exo_b200.worker.engines.b200.tokenizer import (ByteTokenizer, known_eos_ids, render_prompt,
                                                    without_schema_length_guard)

WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "weather by city",
                                            "parameters": {"type": "object", "properties": {"city": {"type": "string"},
                                                                                            "days": {"type": "integer"}}}}}
CALL = {"id": "c1", "type": "function", "function": {"name": "get_weather", "arguments": json.dumps({"city": "Oslo", "days": 2})}}


def test_v4_plain_turns_thinking_and_chat():
    enc = DeepSeekPromptEncoder(V4)
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}]
    assert enc.encode(msgs, thinking=True) == f"{BOS}Be brief.{USER}Hi{ASSISTANT}<think>"
    assert enc.encode(msgs, thinking=False) == f"{BOS}Be brief.{USER}Hi{ASSISTANT}</think>"
    assert enc.encode(msgs, thinking=True, reasoning_effort="max").startswith(BOS + MAX_EFFORT_PREAMBLE + "Be brief.")
    assert MAX_EFFORT_PREAMBLE not in enc.encode(msgs, thinking=False, reasoning_effort="max")


def test_v4_history_drops_old_reasoning_but_not_with_tools():
    enc = DeepSeekPromptEncoder(V4)
    msgs = [{"role": "user", "content": "a"}, {"role": "assistant", "content": "A", "reasoning_content": "r1"},
            {"role": "user", "content": "b"}]
    got = enc.encode(msgs, thinking=True)
    assert got == f"{BOS}{USER}a{ASSISTANT}</think>A{EOS}{USER}b{ASSISTANT}<think>"
    with_tools = enc.encode(msgs, thinking=True, tools=[WEATHER])
    assert f"{USER}a{ASSISTANT}<think>r1</think>A{EOS}" in with_tools
    assert "### Available Tool Schemas" in with_tools and json.dumps(WEATHER["function"]) in with_tools
    assert f'"<{DSML}tool_calls>" block' in with_tools


def test_v4_tool_results_join_the_next_user_turn_in_call_order():
    enc = DeepSeekPromptEncoder(V4)
    call2 = {"id": "c2", "type": "function", "function": {"name": "get_weather", "arguments": '{"city": "Rome"}'}}
    msgs = [{"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "", "reasoning_content": "look it up", "tool_calls": [CALL, call2]},
            {"role": "tool", "tool_call_id": "c2", "content": "sunny"},
            {"role": "tool", "tool_call_id": "c1", "content": "rain"},
            {"role": "user", "content": "and?"}]
    got = enc.encode(msgs, thinking=True, tools=[WEATHER])
    block = (f'\n\n<{DSML}tool_calls>\n<{DSML}invoke name="get_weather">\n'
             f'<{DSML}parameter name="city" string="true">Oslo</{DSML}parameter>\n'
             f'<{DSML}parameter name="days" string="false">2</{DSML}parameter>\n</{DSML}invoke>\n'
             f'<{DSML}invoke name="get_weather">\n<{DSML}parameter name="city" string="true">Rome</{DSML}parameter>\n'
             f'</{DSML}invoke>\n</{DSML}tool_calls>')
    assert f"{ASSISTANT}<think>look it up</think>{block}{EOS}" in got
    assert got.endswith(f"{USER}<tool_result>rain</tool_result>\n\n<tool_result>sunny</tool_result>\n\nand?{ASSISTANT}<think>")


def test_v32_function_results_follow_the_assistant_turn():
    enc = DeepSeekPromptEncoder(V32)
    msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "", "reasoning_content": "think", "tool_calls": [CALL]},
            {"role": "tool", "tool_call_id": "c1", "content": "rain"}]
    got = enc.encode(msgs, thinking=True, tools=[WEATHER])
    assert f'<{DSML}function_calls>\n<{DSML}invoke name="get_weather">' in got
    assert got.endswith(f"</{DSML}function_calls>{EOS}\n\n<function_results>\n<result>rain</result>\n</function_results>\n\n<think>")
    assert "<functions>\n" + json.dumps(WEATHER["function"]) + "\n</functions>" in got
    chat = enc.encode(msgs, thinking=False, tools=[WEATHER])
    assert chat.endswith("</function_results>")
    # a turn without reasoning carries no think markers
    plain = enc.encode([{"role": "user", "content": "hi"}], thinking=False)
    assert plain == f"{BOS}{USER}hi{ASSISTANT}"
    hist = enc.encode([{"role": "user", "content": "a"}, {"role": "assistant", "content": "A", "reasoning_content": "r"},
                       {"role": "user", "content": "b"}], thinking=True)
    assert hist == f"{BOS}{USER}a{ASSISTANT}A{EOS}{USER}b{ASSISTANT}<think>"


@pytest.mark.parametrize("dialect", [V32, V4])
def test_completion_round_trip(dialect):
    enc = DeepSeekPromptEncoder(dialect)
    args = {"city": "Oslo", "days": 2, "opts": {"units": "C", "tags": ["a", "b"]}, "note": "line1\nline2"}
    turn = "because</think>On it." + enc.encode_calls([{"function": {"name": "get_weather", "arguments": json.dumps(args)}}]) + EOS
    msg = enc.parse_completion(turn, thinking=True)
    assert msg["reasoning_content"] == "because" and msg["content"] == "On it."
    (tc,) = msg["tool_calls"]
    assert tc["function"]["name"] == "get_weather" and json.loads(tc["function"]["arguments"]) == args
    assert enc.parse_completion("just text" + EOS, thinking=False) == {
        "role": "assistant", "content": "just text", "reasoning_content": "", "tool_calls": []}
    with pytest.raises(ValueError):
        enc.parse_completion("no close marker", thinking=True)
    with pytest.raises(ValueError):
        enc.parse_completion(f"</think>x\n\n{enc.block_open}\n", thinking=True)


def test_render_prompt_selects_the_encoder_by_model_id():
    assert encoder_for("deepseek-ai/DeepSeek-V4-Base").d is V4 and encoder_for("mlx-community/DeepSeek-V3.2-8bit").d is V32
    assert encoder_for("deepseek-ai/DeepSeek-V3.1") is None
    tok = ByteTokenizer(300)
    p = TextGenerationTaskParams(model="mlx-community/DeepSeek-V4-4bit", input=[InputMessage(role="user", content="Hi")],
                                 instructions="S", enable_thinking=False)
    assert render_prompt(tok, p) == (f"{BOS}S{USER}Hi{ASSISTANT}</think>", False)
    p = TextGenerationTaskParams(model="mlx-community/DeepSeek-V4-4bit", reasoning_effort="xhigh", input=[],
                                 chat_template_messages=[{"role": "user", "content": "Hi"},
                                                         {"role": "assistant", "content": "<think>old</think>Hello"},
                                                         {"role": "user", "content": "more"},
                                                         {"role": "assistant", "content": "Sure, "}])
    text, cont = render_prompt(tok, p)
    assert cont and text == f"{BOS}{MAX_EFFORT_PREAMBLE}{USER}Hi{ASSISTANT}</think>Hello{EOS}{USER}more{ASSISTANT}<think>Sure, "


def test_known_eos_ids_and_template_guard():
    assert known_eos_ids("moonshotai/Kimi-K2-Instruct") == (163586,)
    assert known_eos_ids("zai-org/GLM-5-Air") == (154820, 154827, 154829) and known_eos_ids("zai-org/GLM-4.7") == (151336, 151329, 151338)
    assert known_eos_ids("openai/gpt-oss-120b") == (200002, 200012) and known_eos_ids("meta-llama/Llama-3.1-8B") == ()
    tpl = "{% if inner_type == \"object | object\" or inner_type|length > 50 %}any[]{% endif %}"
    assert without_schema_length_guard(tpl) == "{% if inner_type == \"object | object\" %}any[]{% endif %}"
    assert without_schema_length_guard("{{ messages }}") is None
