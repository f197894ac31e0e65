"""Verifiers, GRPO loss math and RL packing (CPU)."""

import asyncio
import json
import math

import numpy as np
import torch


def test_verifiers_basic():
    from open_instruct_b200 import ground_truth_utils as g

    v = g.build_all_verifiers()
    for name in ("gsm8k", "math", "strict_math", "ifeval", "flan", "string_matcher", "string_f1", "puzzle", "re_search_f1",
                 "re_search", "max_length", "up_to_max_length", "passthrough", "code", "rubric", "general-quality"):
        assert name in v, name
    assert v["gsm8k"]([], "so the total is 1,234.", "1234").score == 1.0
    assert v["gsm8k"]([], "it is -5 then 7", "-5").score == 0.0
    assert v["math"]([], "thus \\boxed{\\frac{1}{2}}", "\\frac{1}{2}").score == 1.0
    assert v["math"]([], "the value is $0.5$", "\\frac{1}{2}").score == 1.0
    assert v["strict_math"]([], "\\boxed{3}", "3").score == 0.0
    assert v["strict_math"]([], "Final Answer: The final answer is $3$. I hope it is correct.", "3").score == 1.0
    assert v["string_matcher"]([], "<think>x</think><answer>The Cat</answer>", "cat").score == 1.0
    assert v["string_matcher"]([], "cat", "cat").score == 0.0
    assert abs(v["string_f1"]([], "the quick brown fox", ["quick fox", "zzz"]).score - 0.8) < 1e-6
    assert v["re_search_f1"]([], "<finish>nothing alike</finish>", "paris").score == 0.1
    assert v["re_search"]([], "<FINISH> Paris </finish>", json.dumps(["paris", "Paris, France"])).score == 1.0
    assert v["up_to_max_length"]([0] * 10, "", "20").score == 1.0
    assert abs(v["max_length"]([0] * 10, "", "20").score - (1 - 10 / 32768)) < 1e-9
    lab = json.dumps({"instruction_id": ["keywords:existence", "punctuation:no_comma"], "kwargs": [{"keywords": ["moon"]}, {}]})
    assert v["ifeval"]([], "the moon is bright", lab).score == 1.0
    assert v["ifeval"]([], "the moon, is bright", lab).score == 0.5
    assert v["ifeval_old"]([], "HELLO", json.dumps({"func_name": "validate_uppercase"})).score == 1.0


def test_code_and_judge_verifiers_with_fakes():
    from open_instruct_b200 import ground_truth_utils as g

    def poster(url, payload):
        assert "def f" in payload["program"]
        return {"results": [1, 1, 0, 1], "runtimes": [0.1] * 4}

    cv = g.CodeVerifier(g.CodeVerifierConfig(code_pass_rate_reward_threshold=0.5), poster=poster)
    assert cv([], "here\n```python\ndef f(): pass\n```", json.dumps(["assert True"] * 4)).score == 0.75
    assert cv([], "no code", "[]").score == 0.0

    async def judge(messages, **kw):
        return '```json\n{"REASONING": "fine", "SCORE": "7"}\n```'

    jv = g.LMJudgeVerifier("quality", g.LMJudgeVerifierConfig(llm_judge_client=judge))
    res = asyncio.run(jv.async_call([], "an answer", "ref", "q"))
    assert abs(res.score - 0.7) < 1e-9
    # a request that outgrows the judge's context window is cut to fit; when even the cut does not fit, the score is 0 without a call
    seen = []

    async def recording_judge(messages, **kw):
        seen.append(messages)
        return '{"REASONING": "ok", "SCORE": "5"}'

    long_answer = "word " * 5000
    fit = g.LMJudgeVerifier("quality", g.LMJudgeVerifierConfig(llm_judge_client=recording_judge, llm_judge_max_tokens=64, llm_judge_max_context_length=1500))
    assert abs(asyncio.run(fit.async_call([], long_answer, "ref", "q")).score - 0.5) < 1e-9
    assert len(seen) == 1 and len(seen[0][0]["content"]) < len(long_answer) / 2
    tiny = g.LMJudgeVerifier("quality", g.LMJudgeVerifierConfig(llm_judge_client=recording_judge, llm_judge_max_tokens=64, llm_judge_max_context_length=250))
    res = asyncio.run(tiny.async_call([], long_answer, "ref", "q"))
    assert res.score == 0.0 and "Context window" in res.reasoning and len(seen) == 1
    rv = g.RubricVerifier(g.RubricVerifierConfig(llm_judge_client=judge))
    lab = json.dumps({"query": "q", "rubrics": [{"description": "a", "weight": 1.0}, {"description": "b", "weight": -1.0}]})
    assert asyncio.run(rv.async_call([], "ans", lab)).score == 0.0


def test_reward_fn_aggregation():
    from open_instruct_b200 import ground_truth_utils as g
    from open_instruct_b200.data_types import RequestInfo

    cfg = g.RewardConfig(verifier_functions=g.build_all_verifiers(), non_stop_penalty=True, non_stop_penalty_value=-3.0)
    fn = cfg.build()
    infos = RequestInfo(rollout_states=[{}, {"rewards": [0.5, 0.25]}, {}])
    scores, metrics = asyncio.run(fn([[1], [2], [3]], ["ans 4", "ans 5", "ans 6"], ["4", "0", "6"], ["gsm8k"] * 3,
                                     ["stop", "stop", "length"], infos))
    assert scores == [10.0, 0.25, -3.0]
    assert abs(metrics["objective/verifiable_correct_rate"] - 2 / 3) < 1e-9
    cfg2 = g.RewardConfig(verifier_functions=g.build_all_verifiers(), apply_r1_style_format_reward=True, reward_aggregator="sum")
    s2, m2 = asyncio.run(cfg2.build()([[1], [2]], ["<think>a</think> <answer>4</answer>", "4"], ["4", "4"], ["gsm8k"] * 2,
                                      ["stop", "stop"], None))
    assert s2 == [10.0, 0] and m2["val/format_scores"] == 0.5


def test_grpo_loss_and_rho():
    from open_instruct_b200.grpo_utils import (GRPOExperimentConfig, compute_grpo_loss, compute_rho_correction, estimate_kl,
                                               masked_mean, resolve_old_logprob)

    cfg = GRPOExperimentConfig(clip_lower=0.2, clip_higher=0.2)
    new = torch.log(torch.tensor([[0.5, 0.9, 0.1]]))
    old = torch.log(torch.tensor([[0.5, 0.5, 0.5]]))
    ratio = torch.exp(new - old)
    adv = torch.tensor([[1.0, 1.0, -1.0]])
    pg, clipfrac, kl = compute_grpo_loss(new, ratio, adv, None, cfg, torch.ones_like(ratio))
    assert torch.allclose(pg, torch.tensor([[-1.0, -1.2, 0.8]]), atol=1e-6)
    assert clipfrac.tolist() == [[0.0, 1.0, 1.0]] and float(kl.abs().sum()) == 0.0
    cfg_c = GRPOExperimentConfig(loss_fn="cispo", clip_higher=0.2)
    pg_c, cf_c, _ = compute_grpo_loss(new, ratio, adv, None, cfg_c, torch.ones_like(ratio))
    assert torch.allclose(pg_c, -adv * torch.clamp(ratio, max=1.2) * new)
    ref = new - torch.tensor([[0.1, -0.2, 0.0]])
    _, _, kl2 = compute_grpo_loss(new, ratio, adv, ref, cfg, torch.ones_like(ratio))
    d = new - ref
    assert torch.allclose(kl2, torch.expm1(-d) + d)
    assert estimate_kl(d, ratio).shape[0] == 4
    mask = torch.tensor([[True, True, False]])
    vllm = old - torch.tensor([[0.0, math.log(4.0), 0.0]])
    rc = compute_rho_correction(old, vllm, mask, adv, cfg)
    assert torch.allclose(rc.weights, torch.tensor([[1.0, 2.0, 0.0]]))
    cfg_m = GRPOExperimentConfig(rho_mask_upper_bound=3.0)
    assert torch.allclose(compute_rho_correction(old, vllm, mask, adv, cfg_m).weights, torch.tensor([[1.0, 0.0, 0.0]]))
    assert float(masked_mean(torch.tensor([1.0, 3.0]), torch.tensor([False, False]))) == 0.0
    assert float(masked_mean(torch.tensor([1.0, 3.0]), torch.tensor([True, True]), denominator=4.0)) == 1.0
    cache = [None]
    x = torch.tensor([0.1], requires_grad=True)
    o = resolve_old_logprob(cache, 0, 0, 1, False, None, x)
    assert not o.requires_grad and resolve_old_logprob(cache, 0, 1, 1, False, None, x * 2) is o


def test_pack_sequences_contract():
    from open_instruct_b200.rl_utils import calculate_advantages, pack_sequences, reset_position_ids

    q = [[5, 6], [7], [8, 9, 10]]
    r = [[11, 12, 0], [13], [14, 15]]
    m = [[1, 1, 1], [1], [1, 0]]
    lp = [[-0.1, -0.2, 0.0], [-0.3], [-0.4, -0.5]]
    p = pack_sequences(q, r, m, pack_length=7, pad_token_id=0, vllm_logprobs=lp, mask_tool_use=True)
    assert [t.tolist() for t in p.query_responses] == [[5, 6, 11, 12, 7, 13], [8, 9, 10, 14, 15]]
    assert p.response_masks[0].tolist() == [0, 0, 1, 1, 0, 2] and p.response_masks[1].tolist() == [0, 0, 0, 3, 0]
    assert p.attention_masks[0].tolist() == [1, 1, 1, 1, 2, 2] and p.attention_masks[1].tolist() == [1] * 5
    assert p.position_ids[0].tolist() == [0, 1, 2, 3, 0, 1]
    assert torch.equal(p.position_ids[0], reset_position_ids(p.attention_masks[0][None])[0])
    assert p.dones[0].tolist() == [0, 0, 0, 1, 0, 2] and p.cu_seqlens[0].tolist() == [0, 4, 6]
    assert torch.isnan(p.vllm_logprobs[0][:2]).all() and abs(p.vllm_logprobs[0][5].item() + 0.3) < 1e-6
    p2 = pack_sequences(q, r, m, pack_length=100, pad_token_id=0, vllm_logprobs=lp, min_num_batches=2)
    assert len(p2.query_responses) >= 2
    adv, ret = calculate_advantages(np.zeros((1, 3)), np.array([[0.0, 0.0, 1.0]]), gamma=1.0, lam=1.0)
    assert adv.tolist() == [[1.0, 1.0, 1.0]]


def test_pass_at_k():
    from open_instruct_b200.grpo_utils import compute_pass_at_k_metrics

    out = compute_pass_at_k_metrics([10, 0, 0, 0, 0, 0, 0, 0], ["a"] * 4 + ["b"] * 4, k=2, max_possible_score=10)
    assert abs(out["eval/pass_at_2"] - 0.25) < 1e-9
