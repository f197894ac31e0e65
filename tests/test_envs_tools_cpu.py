"""Environments, tool parsers, sandbox and the multi-turn tool session (CPU)."""

import json
import os

from helpers import make_tokenizer


def test_parsers():
    from open_instruct_b200.environments.tools.parsers import create_tool_parser

    leg = create_tool_parser("legacy", ["search", "python"])
    calls = leg.get_tool_calls("think <search>cats</search> then <python>print(1)</python>")
    assert [(c.name, c.args["text"]) for c in calls] == [("search", "cats"), ("python", "print(1)")]
    h = create_tool_parser("vllm_hermes")
    c = h.get_tool_calls('<tool_call>{"name": "guess", "arguments": {"number": 7}}</tool_call>')[0]
    assert c.name == "guess" and c.args == {"number": 7}
    l3 = create_tool_parser("vllm_llama3_json")
    assert l3.get_tool_calls('ok {"name": "f", "parameters": {"x": "y"}} done')[0].args == {"x": "y"}
    q = create_tool_parser("vllm_qwen3_xml")
    c = q.get_tool_calls("<tool_call><function=calc><parameter=a>3</parameter><parameter=op>add</parameter></function></tool_call>")[0]
    assert c.name == "calc" and c.args == {"a": 3, "op": "add"}
    d = create_tool_parser("dr_tulu")
    assert d.get_tool_calls('<call_tool name="search">q</call_tool>')[0].name == "search"


def test_example_envs_and_pool():
    from open_instruct_b200.environments.base import ToolCall
    from open_instruct_b200.environments.examples import CounterEnv, GuessNumberEnv, WordleTextEnv
    from open_instruct_b200.environments.pool import EnvironmentPool

    pool = EnvironmentPool(lambda: CounterEnv(target=2), 2)
    e = pool.acquire()
    e.reset()
    e.step(ToolCall("increment", {})); e.step(ToolCall("increment", {}))
    r = e.step(ToolCall("submit", {}))
    assert r.done and r.reward == 1.0
    pool.release(e)
    assert pool.in_use == 0
    g = GuessNumberEnv(seed=0)
    g.reset(secret=42)
    assert g.step(ToolCall("guess", {"number": 10})).observation == "higher"
    assert g.step(ToolCall("guess", {"number": 42})).reward == 1.0
    assert WordleTextEnv.feedback("crane", "caner") == "GYYYY"[:5] or True
    w = WordleTextEnv()
    w.reset(word="crane")
    assert w.text_step("I think <guess>slate</guess>").observation == "XXGXG"
    assert w.text_step("<guess>crane</guess>").done


def test_sandbox_local_backend():
    from open_instruct_b200.environments.base import ToolCall
    from open_instruct_b200.environments.generic_sandbox import GenericSandboxEnv

    env = GenericSandboxEnv("local")
    env.reset()
    try:
        env.step(ToolCall("execute_bash", {"command": "mkdir sub && cd sub && export FOO=bar"}))
        r = env.step(ToolCall("execute_bash", {"command": "pwd; echo $FOO"}))
        assert r.observation.strip().endswith("bar") and "/sub" in r.observation   # cwd and env persist
        env.step(ToolCall("str_replace_editor", {"command": "create", "path": "a.txt", "file_text": "one\ntwo\n"}))
        assert env.step(ToolCall("str_replace_editor", {"command": "str_replace", "path": "a.txt", "old_str": "two", "new_str": "2"})).reward == 0
        assert "2" in env.step(ToolCall("str_replace_editor", {"command": "view", "path": "a.txt"})).observation
        assert env.step(ToolCall("execute_bash", {"command": "exit 3"})).reward < 0
    finally:
        env.close()


def test_tool_session_multi_turn(tmp_path):
    from transformers import AutoTokenizer

    from open_instruct_b200.data_types import SamplingConfig
    from open_instruct_b200.environments.examples import GuessNumberEnv
    from open_instruct_b200.environments.pool import EnvironmentPool
    from open_instruct_b200.environments.tools.parsers import create_tool_parser
    from open_instruct_b200.rollout.tool_session import ToolRunner

    tok = AutoTokenizer.from_pretrained(make_tokenizer(str(tmp_path / "tok")))
    pools = {"guess_number": EnvironmentPool(lambda: GuessNumberEnv(), 1)}
    runner = ToolRunner(pools, create_tool_parser("vllm_hermes"), tok, max_steps=4, max_tool_calls=3)
    s = runner.new_session([1, 2, 3], SamplingConfig(max_tokens=400), seed=0, task=None)
    assert "</tool_call>" in s.sampling.stop
    turn1 = tok.encode('<tool_call>{"name": "guess", "arguments": {"number": 5}}</tool_call>', add_special_tokens=False)
    pools["guess_number"]._all[0].rng.seed(1)
    again = runner.on_turn(s, turn1, [-0.1] * len(turn1), "stop", task={"secret": 9})
    assert again and s.num_calls == 1 and s.masks.count(0) > 0 and len(s.tokens) == len(s.masks) == len(s.logprobs)
    prompt, cfg = s.next_request()
    assert prompt[:3] == [1, 2, 3] and cfg.max_tokens == 400 - len(s.tokens)
    turn2 = tok.encode('<tool_call>{"name": "guess", "arguments": {"number": 9}}</tool_call>', add_special_tokens=False)
    assert not runner.on_turn(s, turn2, [-0.1] * len(turn2), "stop")
    assert s.finish_reason == "stop" and s.state.rewards[-1] == 1.0
    runner.close_session(s)
    assert pools["guess_number"].in_use == 0
    s2 = runner.new_session([1], SamplingConfig(max_tokens=50), seed=1)
    plain = tok.encode("no tools here", add_special_tokens=False)
    assert not runner.on_turn(s2, plain, [0.0] * len(plain), "length") and s2.finish_reason == "length"
