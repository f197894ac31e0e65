"""Preference pairs from an LLM judge: every pair of candidates of a prompt (reference answer included) is shown to
a chat-completions endpoint in random order; the judge answers ``Comparison: ... Preferred: 0|1``
(``open_instruct/rejection_sampling/synthetic_preference_dataset.py:114-185``).

The endpoint is any OpenAI-compatible ``/chat/completions`` URL; ``judge`` can also be injected as an async callable
``(messages) -> str`` (used by the tests).  Unlike the reference, whose swap condition can never hold, the pair is
actually swapped when the judge prefers the second candidate.
"""

from __future__ import annotations

import asyncio
import copy
import itertools
import json
import random
from collections import defaultdict
from dataclasses import dataclass

from .prompt_templates import PAIRWISE_TEMPLATE


@dataclass
class Args:
    input_filename: str = "completions.jsonl"
    save_filename: str = "synthetic_preferences.jsonl"
    num_completions: int = 1
    model: str = "gpt-4o-2024-08-06"
    base_url: str = "https://api.openai.com/v1"
    api_key_env: str = "OPENAI_API_KEY"
    max_parallel_requests: int = 100
    max_tries: int = 3
    seed: int = 0


def comparison_pairs(completions: list[dict], num_completions: int, with_reference: bool = True) -> list[tuple[dict, dict]]:
    pairs = []
    for i in range(0, len(completions), num_completions):
        group = list(completions[i:i + num_completions])
        if with_reference:
            ref = copy.deepcopy(completions[i])
            ref["messages"][-1]["content"] = completions[i]["reference_completion"]
            group.append(ref)
        pairs += list(itertools.combinations(group, 2))
    return pairs


def parse_judgement(text: str) -> tuple[str, int]:
    comparison = text.split("Comparison:")[1].split("Preferred:")[0].strip()
    preferred = text.split("Preferred:")[1].strip().strip('"').strip()[:1]
    if preferred not in ("0", "1"):
        raise ValueError(f"judge did not name a preference: {text[-80:]!r}")
    return comparison, int(preferred)


def http_judge(args: Args):
    import os

    import aiohttp

    async def call(messages):
        headers = {"Authorization": f"Bearer {os.environ.get(args.api_key_env, '')}"}
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=120)) as s:
            async with s.post(args.base_url.rstrip("/") + "/chat/completions", json={"model": args.model, "messages": messages},
                              headers=headers) as r:
                r.raise_for_status()
                return (await r.json())["choices"][0]["message"]["content"]

    return call


async def judge_all(pairs, judge, max_parallel: int, max_tries: int, seed: int):
    limiter = asyncio.Semaphore(max_parallel)
    rng = random.Random(seed)
    flips = [rng.randint(0, 1) for _ in pairs]

    async def one(pair, flip):
        task = pair[0]["messages"][:-1]
        shown = (pair[flip]["messages"][-1], pair[1 - flip]["messages"][-1])
        prompt = PAIRWISE_TEMPLATE.replace("{{task}}", str(task)).replace("{{response0}}", str(shown[0])).replace("{{response1}}", str(shown[1]))
        messages = [{"role": "user", "content": prompt}]
        async with limiter:
            for _ in range(max_tries):
                try:
                    reply = await judge(messages)
                    comparison, preferred = parse_judgement(reply)
                except Exception:  # noqa: BLE001 - malformed reply or transport error: try again
                    continue
                winner = flip if preferred == 0 else 1 - flip  # index into `pair`
                return pair[winner]["messages"], pair[1 - winner]["messages"], comparison, messages + [{"role": "assistant", "content": reply}]
        return None

    return await asyncio.gather(*[one(p, f) for p, f in zip(pairs, flips)])


def main(args: Args, judge=None) -> dict:
    with open(args.input_filename) as f:
        completions = [json.loads(line) for line in f if line.strip()]
    pairs = comparison_pairs(completions, args.num_completions)
    items = asyncio.run(judge_all(pairs, judge or http_judge(args), args.max_parallel_requests, args.max_tries, args.seed))
    table = defaultdict(list)
    for it in items:
        if it is None:
            continue
        for k, v in zip(("chosen", "rejected", "comparison", "whole_conversation"), it):
            table[k].append(v)
    from .rejection_sampling import save_jsonl

    save_jsonl(args.save_filename, table)
    return dict(table)


if __name__ == "__main__":
    from ..config.argparser import ArgumentParserPlus

    main(ArgumentParserPlus((Args,)).parse())
