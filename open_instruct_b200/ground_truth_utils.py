"""Verifiable rewards: verifier functions, their registry and the reward function builder.

Interface and scoring rules follow the reference (``open_instruct/ground_truth_utils.py``):
``VerifierFunction.__call__(tokenized_prediction, prediction, label, query, rollout_state) -> VerificationResult``
(``:108-183``), one verifier per dataset-source name discovered through ``__subclasses__()`` (``:1188-1225``),
and ``RewardConfig.build()`` returning ``async reward_fn(responses, decoded, ground_truths, datasets,
finish_reasons, infos, queries) -> (scores, metrics)`` (``:1313-1418``): optional R1-style format reward,
verifiable reward x ``verification_reward`` (default 10), per-turn aggregation (last / sum), and the
non-stop penalty.  Verifiers that call out (LLM judge, code execution) take their transport from
the config so that tests inject a fake.
"""

from __future__ import annotations

import asyncio
import dataclasses
import json
import logging
import re
import string
from abc import ABC, abstractmethod
from collections import Counter, defaultdict
from typing import Any, Callable, Literal

import numpy as np

from .math_utils import (
    get_unnormalized_answer,
    hendrycks_is_equiv,
    is_equiv,
    last_boxed_only_string,
    normalize_final_answer,
    remove_boxed,
)

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class VerifierConfig:
    """Base configuration; ``from_args`` copies every field that any of the sources defines."""

    @classmethod
    def from_args(cls, *sources) -> "VerifierConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {}
        for src in sources:
            if src is None:
                continue
            for n in names:
                if hasattr(src, n):
                    kw[n] = getattr(src, n)
        return cls(**kw)


@dataclasses.dataclass
class LMJudgeVerifierConfig(VerifierConfig):
    llm_judge_model: str = "gpt-4o-mini"
    llm_judge_max_tokens: int = 2048
    llm_judge_max_context_length: int = 8192
    llm_judge_temperature: float = 1.0
    llm_judge_timeout: int = 60
    seed: int = 0
    llm_judge_base_url: str | None = None
    llm_judge_client: Any = None  # async callable(messages, **kw) -> str; tests inject one


@dataclasses.dataclass
class CodeVerifierConfig(VerifierConfig):
    code_api_url: str = "http://127.0.0.1:1234/test_program"
    code_max_execution_time: float = 1.0
    code_pass_rate_reward_threshold: float = 0.0
    code_apply_perf_penalty: bool = False


@dataclasses.dataclass
class MaxLengthVerifierConfig(VerifierConfig):
    max_length_verifier_max_length: int = 32768


@dataclasses.dataclass
class VerificationResult:
    score: float
    cost: float = 0.0
    reasoning: str | None = None


class VerifierFunction(ABC):
    def __init__(self, name: str, weight: float = 1.0, verifier_config: VerifierConfig | None = None) -> None:
        self.name, self.weight, self.verifier_config = name, weight, verifier_config

    @classmethod
    def get_config_class(cls) -> type:
        return VerifierConfig

    @abstractmethod
    def __call__(self, tokenized_prediction: list[int], prediction: str, label: Any, query: str | None = None,
                 rollout_state: dict | None = None) -> VerificationResult: ...

    async def async_call(self, tokenized_prediction, prediction, label, query=None, rollout_state=None) -> VerificationResult:
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, lambda: self(tokenized_prediction, prediction, label, query, rollout_state))

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(name={self.name}, weight={self.weight})"


# ---------------------------------------------------------------------------------- text helpers
def remove_thinking_section(prediction: str) -> str:
    prediction = prediction.replace("<|assistant|>", "").strip().split("</think>")[-1]
    return prediction.replace("<answer>", "").replace("</answer>", "").strip()


def normalize_answer(s: str) -> str:
    """SQuAD normalisation: lower-case, strip punctuation, articles and extra whitespace."""
    s = "".join(ch for ch in str(s).lower() if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def f1_score(prediction: str, ground_truth: str) -> dict[str, float]:
    p, g = normalize_answer(prediction).split(), normalize_answer(ground_truth).split()
    common = sum((Counter(p) & Counter(g)).values())
    if common == 0:
        return {"f1": 0.0, "precision": 0.0, "recall": 0.0}
    prec, rec = common / len(p), common / len(g)
    return {"f1": 2 * prec * rec / (prec + rec), "precision": prec, "recall": rec}


# ---------------------------------------------------------------------------------- verifiers
class GSM8KVerifier(VerifierFunction):
    """Last number of the prediction (thousands separators removed, sign kept) equals the label."""

    def __init__(self, verifier_config=None):
        super().__init__("gsm8k", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        text = re.sub(r"(\d),(\d)", r"\1\2", prediction)
        nums = re.findall(r"[-+]?(?:\d*\.\d+|\d+)", text)
        got = nums[-1] if nums else text
        return VerificationResult(float(str(got).lower() == str(label).lower()))


def _math_candidates(prediction: str, strict: bool) -> list[str]:
    cands = []
    if not strict:
        boxed = last_boxed_only_string(prediction)
        if boxed is not None:
            try:
                cands.append(remove_boxed(boxed))
            except ValueError:
                pass
    minerva = normalize_final_answer(get_unnormalized_answer(prediction))
    if minerva and minerva != "[invalidanswer]":
        cands.append(minerva)
    if strict:
        return cands
    if not cands:
        d = [m.start() for m in re.finditer(r"\$", prediction)]
        if len(d) > 1:
            cands.append(normalize_final_answer(prediction[d[-2] + 1:d[-1]]))
    if not cands:
        cands += [normalize_final_answer(prediction), prediction]
    return cands


class MathVerifier(VerifierFunction):
    """Boxed answer, Minerva 'final answer is', last $...$ span, or the whole output - any match wins."""

    def __init__(self, verifier_config=None):
        super().__init__("math", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        for ans in _math_candidates(prediction, strict=False):
            if is_equiv(ans, label) or hendrycks_is_equiv(ans, label):
                return VerificationResult(1.0)
        return VerificationResult(0.0)


class StrictMathVerifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("strict_math", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        for ans in _math_candidates(prediction, strict=True):
            if is_equiv(ans, label) or hendrycks_is_equiv(ans, label):
                return VerificationResult(1.0)
        return VerificationResult(0.0)


class IFEvalVerifier(VerifierFunction):
    """Instruction-following constraints: label = JSON with ``instruction_id`` list and ``kwargs`` list;
    score = fraction of constraints satisfied by the answer (thinking section removed)."""

    def __init__(self, verifier_config=None):
        super().__init__("ifeval", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        from .if_functions import check_instruction

        spec = label
        if isinstance(spec, str):
            try:
                spec = json.loads(spec)
            except ValueError:  # datasets store the label as a Python literal (``open_instruct/ground_truth_utils.py:332``)
                import ast

                spec = ast.literal_eval(spec)
        if isinstance(spec, list):
            spec = spec[0]
        if isinstance(spec, str):
            spec = json.loads(spec)
        ids, kws = spec.get("instruction_id", []), spec.get("kwargs", [])
        answer = remove_thinking_section(prediction)
        if not ids or not answer:
            return VerificationResult(0.0)
        ok = [check_instruction(i, answer, (kws[n] if n < len(kws) else None) or {}) for n, i in enumerate(ids)]
        return VerificationResult(sum(ok) / len(ok))


class IFEvalVerifierOld(VerifierFunction):
    """Single-constraint form: label = {"func_name": ..., other kwargs}; score 0/1."""

    def __init__(self, verifier_config=None):
        super().__init__("ifeval_old", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        from .if_functions import IF_FUNCTIONS_MAP

        c = json.loads(label) if isinstance(label, str) else dict(label)
        answer = remove_thinking_section(prediction)
        fn = IF_FUNCTIONS_MAP.get(c.pop("func_name", None))
        if fn is None or not answer:
            return VerificationResult(0.0)
        kw = {k: v for k, v in c.items() if v is not None}
        return VerificationResult(float(fn(answer, **kw)))


class FlanVerifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("flan", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        ans = prediction.split("The answer is: ")[-1].strip()
        return VerificationResult(float(normalize_answer(ans) == normalize_answer(label)))


class StringMatcherVerifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("string_matcher", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        if "<answer>" not in prediction or "</answer>" not in prediction:
            return VerificationResult(0.0)
        ans = prediction.split("<answer>")[-1].split("</answer>")[0]
        return VerificationResult(float(normalize_answer(ans) == normalize_answer(label)))


class F1Verifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("string_f1", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        pred = remove_thinking_section(prediction)
        labels = label if isinstance(label, list) else [label]
        return VerificationResult(max(f1_score(pred, str(x))["f1"] for x in labels))


class PuzzleMatcherVerifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("puzzle", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        return VerificationResult(float(normalize_answer(remove_thinking_section(prediction)) == normalize_answer(label)))


class ReSearchVerifierF1(VerifierFunction):
    """F1 of the text inside <finish>..</finish>; correct format with zero overlap still earns 0.1."""

    def __init__(self, verifier_config=None):
        super().__init__("re_search_f1", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        try:
            label = json.loads(label)
        except (json.JSONDecodeError, TypeError):
            label = str(label).strip()
        if "<finish>" not in prediction and "</finish>" not in prediction:
            return VerificationResult(0.0)
        ans = prediction.split("<finish>")[-1].split("</finish>")[0]
        if not ans:
            return VerificationResult(0.0)
        labels = label if isinstance(label, list) else [label]
        f1 = max(f1_score(ans, str(x))["f1"] for x in labels)
        return VerificationResult(0.1 if f1 == 0 else f1)


class R1SearchVerifier(VerifierFunction):
    TAG = re.compile(r"<finish>(.*?)</finish>", re.IGNORECASE | re.DOTALL)

    def __init__(self, verifier_config=None):
        super().__init__("re_search", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        try:
            parsed = json.loads(label)
            labels = parsed if isinstance(parsed, list) else [parsed]
        except (json.JSONDecodeError, TypeError):
            labels = label if isinstance(label, list) else [str(label).strip()]
        m = self.TAG.search(prediction)
        if not m or not m.group(1).strip():
            return VerificationResult(0.0)
        got = normalize_answer(m.group(1).strip())
        return VerificationResult(float(any(got == normalize_answer(str(x)) for x in labels)))


class MaxLenVerifier(VerifierFunction):
    """1 - |len - target| / max_length: rewards hitting a target length."""

    def __init__(self, verifier_config=None):
        super().__init__("max_length", verifier_config=verifier_config or MaxLengthVerifierConfig())

    @classmethod
    def get_config_class(cls):
        return MaxLengthVerifierConfig

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        diff = abs(len(tokenized_prediction) - float(label))
        return VerificationResult(1 - diff / self.verifier_config.max_length_verifier_max_length)


class UpToMaxLenVerifier(VerifierFunction):
    def __init__(self, verifier_config=None):
        super().__init__("up_to_max_length", verifier_config=verifier_config or MaxLengthVerifierConfig())

    @classmethod
    def get_config_class(cls):
        return MaxLengthVerifierConfig

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        diff = len(tokenized_prediction) - float(label)
        if diff < 0:
            return VerificationResult(1.0)
        return VerificationResult(1 - diff / self.verifier_config.max_length_verifier_max_length)


class PassthroughVerifier(VerifierFunction):
    """Environment-driven tasks: the per-turn rewards in the rollout state are the score; adds nothing."""

    def __init__(self, verifier_config=None):
        super().__init__("passthrough", verifier_config=verifier_config)

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        return VerificationResult(0.0)


class LMJudgeVerifier(VerifierFunction):
    """LLM-as-judge: prompt template by judge type, JSON {"REASONING", "SCORE"} answer, score scaled to [0, 1].
    The transport is ``verifier_config.llm_judge_client`` (async callable) or an OpenAI-compatible HTTP endpoint."""

    def __init__(self, judge_type: str = "quality", verifier_config: LMJudgeVerifierConfig | None = None):
        super().__init__(f"general-{judge_type}", verifier_config=verifier_config or LMJudgeVerifierConfig())
        self.judge_type = judge_type

    @classmethod
    def get_config_class(cls):
        return LMJudgeVerifierConfig

    def build_messages(self, prediction: str, label: str, query: str | None) -> list[dict]:
        from .judge_utils import JUDGE_PROMPT_MAP

        tpl = JUDGE_PROMPT_MAP.get(self.judge_type, JUDGE_PROMPT_MAP["quality"])
        return [{"role": "user", "content": tpl.format(input=query or "", output=remove_thinking_section(prediction), label=label)}]

    async def _ask(self, messages: list[dict]) -> str:
        cfg = self.verifier_config
        if cfg.llm_judge_client is not None:
            return await cfg.llm_judge_client(messages, model=cfg.llm_judge_model, max_tokens=cfg.llm_judge_max_tokens,
                                              temperature=cfg.llm_judge_temperature, seed=cfg.seed)
        if cfg.llm_judge_base_url is None:
            raise RuntimeError("no judge transport configured (llm_judge_client or llm_judge_base_url)")
        import aiohttp

        payload = {"model": cfg.llm_judge_model, "messages": messages, "max_tokens": cfg.llm_judge_max_tokens,
                   "temperature": cfg.llm_judge_temperature, "seed": cfg.seed}
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=cfg.llm_judge_timeout)) as s:
            async with s.post(cfg.llm_judge_base_url.rstrip("/") + "/chat/completions", json=payload) as r:
                data = await r.json()
        return data["choices"][0]["message"]["content"]

    async def async_call(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        from .judge_utils import extract_score_from_string

        messages = self.build_messages(prediction, str(label), query)
        # a judge request must fit the judge's context window: cut the messages to fit, give up (score 0) when even that
        # does not (``open_instruct/ground_truth_utils.py:773-797``)
        from . import context_window_checker as cwc

        cfg = self.verifier_config
        if not cwc.check_context_window_limit(messages, cfg.llm_judge_max_tokens, cfg.llm_judge_model, cfg.llm_judge_max_context_length, 150):
            messages = cwc.truncate_messages_to_fit_context(messages, cfg.llm_judge_max_tokens, cfg.llm_judge_model,
                                                            cfg.llm_judge_max_context_length, 200)
            if not messages or not cwc.check_context_window_limit(messages, cfg.llm_judge_max_tokens, cfg.llm_judge_model,
                                                                  cfg.llm_judge_max_context_length, 150):
                return VerificationResult(0.0, reasoning="Error: Context window exceeded")
        for attempt in range(3):
            try:
                reply = await self._ask(messages)
                reasoning, score = extract_score_from_string(reply)
                return VerificationResult(score=score, reasoning=reasoning)
            except Exception as e:  # noqa: BLE001
                logger.warning("LLM judge attempt %d failed: %s", attempt + 1, e)
                await asyncio.sleep(0.05 * 2 ** attempt)
        return VerificationResult(0.0, reasoning="judge unavailable")

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        return asyncio.run(self.async_call(tokenized_prediction, prediction, label, query, rollout_state))


class CodeVerifier(VerifierFunction):
    """Runs the extracted program against the label's test cases through the code-execution service
    (POST {program, tests, max_execution_time} -> {results: [0/1]}); score = pass rate above a threshold."""

    def __init__(self, verifier_config: CodeVerifierConfig | None = None, name: str = "code", poster: Callable | None = None):
        super().__init__(name, verifier_config=verifier_config or CodeVerifierConfig())
        self._post = poster

    @classmethod
    def get_config_class(cls):
        return CodeVerifierConfig

    @staticmethod
    def extract_python_code(text: str) -> str:
        blocks = re.findall(r"```(?:python)?\n(.*?)```", text, re.DOTALL)
        return blocks[-1].strip() if blocks else ""

    def _request(self, payload: dict) -> dict:
        if self._post is not None:
            return self._post(self.verifier_config.code_api_url, payload)
        import requests

        r = requests.post(self.verifier_config.code_api_url, json=payload, timeout=60)
        r.raise_for_status()
        return r.json()

    def __call__(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        code = self.extract_python_code(remove_thinking_section(prediction) if "</think>" in prediction else prediction)
        if not code:
            return VerificationResult(0.0)
        tests = json.loads(label) if isinstance(label, str) else label
        cfg = self.verifier_config
        try:
            out = self._request({"program": code, "tests": tests, "max_execution_time": cfg.code_max_execution_time})
        except Exception as e:  # noqa: BLE001
            logger.warning("code API call failed: %s", e)
            return VerificationResult(0.0)
        results = out.get("results", [])
        rate = sum(results) / len(results) if results else 0.0
        score = 0.0 if rate < cfg.code_pass_rate_reward_threshold else rate
        if cfg.code_apply_perf_penalty and results and "runtimes" in out:
            mean_rt = float(np.mean(out["runtimes"]))
            score *= max(0.0, 1.0 - mean_rt / max(cfg.code_max_execution_time, 1e-9))
        return VerificationResult(score)


class CodeStdioVerifier(CodeVerifier):
    def __init__(self, verifier_config: CodeVerifierConfig | None = None, poster: Callable | None = None):
        cfg = verifier_config or CodeVerifierConfig()
        cfg = dataclasses.replace(cfg, code_api_url=cfg.code_api_url.replace("/test_program", "/test_program_stdio")
                                  if not cfg.code_api_url.endswith("_stdio") else cfg.code_api_url)
        super().__init__(cfg, name="code_stdio", poster=poster)


@dataclasses.dataclass
class RubricVerifierConfig(LMJudgeVerifierConfig):
    rubric_aggregation: str = "weighted_mean"


class RubricVerifier(LMJudgeVerifier):
    """Label = JSON {"query", "rubrics": [{"description", "weight"}]}; every rubric is judged 0-1 and the
    scores are combined by their (signed) weights, normalised by the total positive weight."""

    def __init__(self, verifier_config: RubricVerifierConfig | None = None):
        VerifierFunction.__init__(self, "rubric", verifier_config=verifier_config or RubricVerifierConfig())
        self.judge_type = "rubric"

    @classmethod
    def get_config_class(cls):
        return RubricVerifierConfig

    async def async_call(self, tokenized_prediction, prediction, label, query=None, rollout_state=None):
        from .rubrics import score_rubrics

        spec = json.loads(label) if isinstance(label, str) else label
        score, detail = await score_rubrics(remove_thinking_section(prediction), spec, self._ask)
        return VerificationResult(score, reasoning=json.dumps(detail)[:2000])


# ---------------------------------------------------------------------------------- registry
def _all_subclasses(cls):
    for sub in cls.__subclasses__():
        yield sub
        yield from _all_subclasses(sub)


def build_all_verifiers(args=None, streaming_config=None) -> dict[str, VerifierFunction]:
    """One instance of every concrete verifier keyed by lower-cased name (+ one judge per judge type)."""
    out: dict[str, VerifierFunction] = {}
    for sub in _all_subclasses(VerifierFunction):
        if sub in (LMJudgeVerifier,) or getattr(sub, "__abstractmethods__", None):
            continue
        cfg_cls = sub.get_config_class()
        try:
            cfg = cfg_cls.from_args(args, streaming_config)
        except TypeError:
            cfg = cfg_cls()
        inst = sub(cfg) if cfg_cls is not VerifierConfig else sub()
        out[inst.name.lower()] = inst
    from .judge_utils import JUDGE_PROMPT_MAP

    jcfg = LMJudgeVerifierConfig.from_args(args, streaming_config)
    for jt in JUDGE_PROMPT_MAP:
        inst = LMJudgeVerifier(jt, jcfg)
        out[inst.name.lower()] = inst
    if args is not None and getattr(args, "remap_verifier", None):
        src, dst = args.remap_verifier.split("=")
        out[src.lower()] = out[dst.lower()]
    return out


# ---------------------------------------------------------------------------------- reward function
def soft_format_reward_func(responses: list[str], reward_scale: float = 1.0) -> list[float]:
    """R1-style format: '...</think> <answer>...</answer>' anywhere from the start."""
    pat = re.compile(r".*?</think>\s*<answer>.*?</answer>", re.DOTALL)
    return [reward_scale if pat.match(r) else 0.0 for r in responses]


async def apply_verifiable_reward(reward_fn_mapping: dict[str, VerifierFunction], responses, decoded_responses, ground_truths,
                                  datasets, reward_mult: float = 1.0, queries=None, rollout_states=None):
    n = len(responses)
    queries = queries or [None] * n
    rollout_states = rollout_states or [None] * n
    tasks, meta = [], []
    for i in range(n):
        gts = [ground_truths[i]] if isinstance(ground_truths[i], str) else list(ground_truths[i])
        dss = [datasets[i]] if isinstance(datasets[i], str) else list(datasets[i])
        if len(gts) != len(dss):
            raise ValueError("Ground truth and dataset list lengths do not match.")
        for gt, ds in zip(gts, dss):
            fn = reward_fn_mapping.get(str(ds).lower())
            if fn is None:
                logger.warning("No reward function found for dataset %s. Skipping reward.", ds)
                continue
            tasks.append(fn.async_call(responses[i], decoded_responses[i], gt, queries[i], rollout_states[i]))
            meta.append((i, fn.name, fn.weight))
    results = await asyncio.gather(*tasks) if tasks else []
    rewards = [0.0] * n
    per_fn = [dict() for _ in range(n)]
    for res, (i, name, w) in zip(results, meta):
        val = reward_mult * (res.score if hasattr(res, "score") else float(res)) * w
        rewards[i] += val
        per_fn[i][name] = per_fn[i].get(name, 0.0) + val
    return rewards, per_fn


@dataclasses.dataclass
class RewardConfig:
    apply_r1_style_format_reward: bool = False
    r1_style_format_reward: float = 1.0
    apply_verifiable_reward: bool = True
    verification_reward: float = 10.0
    non_stop_penalty: bool = False
    non_stop_penalty_value: float = -10.0
    only_reward_good_outputs: bool = False
    additive_format_reward: bool = False
    verifier_functions: dict[str, VerifierFunction] = dataclasses.field(default_factory=dict)
    reward_aggregator: Literal["last", "sum"] = "last"

    def build(self) -> Callable:
        aggregate = (lambda r: r[-1] if r else 0.0) if self.reward_aggregator == "last" else (lambda r: float(sum(r)))

        async def reward_fn(responses, decoded_responses, ground_truths, datasets, finish_reasons, infos, queries=None):
            n = len(decoded_responses)
            states = (getattr(infos, "rollout_states", None) or [{}] * n) if infos is not None else [{}] * n
            states = [s or {} for s in states]
            good = [True] * n
            if infos is not None and getattr(infos, "tool_outputs", None):
                good = [len(infos.tool_outputs[i]) > 0 and infos.tool_calleds[i] and not infos.timeouts[i] and not infos.tool_errors[i]
                        for i in range(len(infos.tool_outputs))]
            scores = [0.0] * n
            metrics: dict[str, Any] = {}
            fmt: list[float] = []
            if self.apply_r1_style_format_reward:
                fmt = soft_format_reward_func(decoded_responses, self.r1_style_format_reward)
                scores = [f + s for f, s in zip(fmt, scores)]
                metrics["val/format_scores"] = float(np.mean(fmt))
            if self.apply_verifiable_reward:
                vr, per_fn = await apply_verifiable_reward(self.verifier_functions, responses, decoded_responses, ground_truths,
                                                           datasets, self.verification_reward, queries, states)
                for i in range(n):
                    if self.only_reward_good_outputs and not good[i]:
                        continue
                    turns = list(states[i].get("rewards", []))
                    if turns:
                        turns[-1] += vr[i]
                    else:
                        turns = [vr[i]]
                    raw = aggregate(turns)
                    if self.apply_r1_style_format_reward and self.additive_format_reward:
                        scores[i] = raw + scores[i]
                    elif self.apply_r1_style_format_reward:
                        scores[i] = raw if fmt[i] == 1 else 0
                    else:
                        scores[i] = raw
                arr = np.array(vr, dtype=np.float64)
                metrics["objective/verifiable_reward"] = float(arr.mean()) if n else 0.0
                metrics["objective/verifiable_correct_rate"] = float((arr > 0).mean()) if n else 0.0
                by_fn = defaultdict(list)
                for d in per_fn:
                    for k, v in d.items():
                        by_fn[k].append(v)
                for k, v in by_fn.items():
                    a = np.array(v)
                    metrics[f"objective/{k}_reward"] = float(a.mean())
                    metrics[f"objective/{k}_correct_rate"] = float((a > 0).mean())
            if self.non_stop_penalty:
                for i, fr in enumerate(finish_reasons):
                    if fr != "stop":
                        scores[i] = self.non_stop_penalty_value
            return scores, metrics

        return reward_fn
