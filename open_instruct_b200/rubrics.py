"""Rubric-based rewards: score an answer against weighted rubric items with an LLM judge, and
maintain an evolving rubric buffer.

Scoring rule (cf. ``open_instruct/rubrics/``): each rubric item is judged on [0, 1]; positive-weight
items reward, negative-weight items penalise; the total is divided by the sum of positive weights
and clipped to [0, 1].  ``RubricBuffer`` keeps per-prompt persistent and adaptive rubrics, retiring
adaptive items whose scores no longer separate samples (zero variance within a group).
"""

from __future__ import annotations

import asyncio
import json
import statistics
from dataclasses import dataclass, field

_ITEM_PROMPT = ("You are grading an answer against ONE rubric item.\n\n[Question]\n{query}\n\n[Answer]\n{answer}\n\n"
                "[Rubric item]\n{rubric}\n\nRespond in JSON format: {{\"REASONING\": \"...\", \"SCORE\": \"<0 to 10>\"}}")


async def score_rubrics(answer: str, spec: dict, ask) -> tuple[float, list[dict]]:
    """``spec`` = {"query": str, "rubrics": [{"description": str, "weight": float}, ...]};
    ``ask`` = async callable(messages) -> str (the judge transport)."""
    from .judge_utils import extract_score_from_string

    rubrics = spec.get("rubrics", [])
    if not rubrics:
        return 0.0, []

    async def one(item):
        msg = [{"role": "user", "content": _ITEM_PROMPT.format(query=spec.get("query", ""), answer=answer, rubric=item["description"])}]
        try:
            _, s = extract_score_from_string(await ask(msg))
        except Exception:  # noqa: BLE001
            s = 0.0
        return s

    scores = await asyncio.gather(*(one(r) for r in rubrics))
    pos = sum(max(0.0, float(r.get("weight", 1.0))) for r in rubrics)
    total = sum(float(r.get("weight", 1.0)) * s for r, s in zip(rubrics, scores))
    final = min(max(total / pos, 0.0), 1.0) if pos > 0 else 0.0
    return final, [{"description": r["description"], "weight": r.get("weight", 1.0), "score": s, "type": r.get("type", "persistent")}
                   for r, s in zip(rubrics, scores)]


@dataclass
class RubricItem:
    description: str
    weight: float = 1.0
    adaptive: bool = False
    history: list[float] = field(default_factory=list)
    title: str = ""

    @property
    def kind(self) -> str:
        return "evolving" if self.adaptive else "persistent"


class RubricBuffer:
    """Per-prompt rubric store: persistent items never leave; adaptive items are capped and retired."""

    def __init__(self, max_active_adaptive: int = 5, min_std: float = 1e-6):
        self.items: dict[str, list[RubricItem]] = {}
        self.inactive: dict[str, list[RubricItem]] = {}   # retired adaptive items, kept for inspection and never re-proposed
        self.max_active_adaptive, self.min_std = max_active_adaptive, min_std

    def add_persistent(self, prompt_id: str, descriptions: list[str], weight: float = 1.0) -> None:
        self.items.setdefault(prompt_id, []).extend(RubricItem(d, weight, False) for d in descriptions)

    def add_adaptive(self, prompt_id: str, proposals: list[dict]) -> None:
        cur = self.items.setdefault(prompt_id, [])
        known = {i.description for i in cur} | {i.description for i in self.inactive.get(prompt_id, [])}
        for p in proposals:
            if p["description"] not in known:
                cur.append(RubricItem(p["description"], float(p.get("weight", 1.0)), True, title=p.get("title", "")))
                known.add(p["description"])
        adaptive = [i for i in cur if i.adaptive]
        for extra in adaptive[: max(0, len(adaptive) - self.max_active_adaptive)]:
            cur.remove(extra)
            self.inactive.setdefault(prompt_id, []).append(extra)

    def record_group_scores(self, prompt_id: str, per_item_scores: list[list[float]]) -> None:
        """``per_item_scores[k]`` = scores of item k over the samples of one prompt group."""
        cur = self.items.get(prompt_id, [])
        retire = []
        for item, scores in zip(cur, per_item_scores):
            item.history.append(statistics.mean(scores) if scores else 0.0)
            if item.adaptive and len(scores) > 1 and statistics.pstdev(scores) <= self.min_std:
                retire.append(item)
        for it in retire:
            cur.remove(it)
            self.inactive.setdefault(prompt_id, []).append(it)

    def filter(self, stats: dict[tuple[str, str], dict], max_active: int | None = None) -> dict[str, int]:
        """Prune with per-item score statistics gathered over a training step (the reference's ``filter_rubric_buffer``,
        ``open_instruct/rubrics/metrics.py:79-148``): ``stats[(prompt_id, description)] = {"mean": ..., "std": ...}``.
        Adaptive items whose scores did not vary at all are retired; if a prompt still has more than ``max_active`` adaptive
        items, those with the largest spread are kept (items without statistics are not touched).  Returns the counts."""
        cap = self.max_active_adaptive if max_active is None else max_active
        zero_std = over_cap = 0
        for pid, cur in self.items.items():
            scored = []
            for it in [i for i in cur if i.adaptive]:
                st = stats.get((pid, it.description))
                if st is None:
                    continue
                if st["std"] <= self.min_std:
                    cur.remove(it)
                    self.inactive.setdefault(pid, []).append(it)
                    zero_std += 1
                else:
                    scored.append((st["std"], it))
            if sum(1 for i in cur if i.adaptive) > cap:
                scored.sort(key=lambda t: -t[0])
                for _, it in scored[cap:]:
                    cur.remove(it)
                    self.inactive.setdefault(pid, []).append(it)
                    over_cap += 1
        return {"zero_std": zero_std, "over_cap": over_cap}

    def counts(self) -> dict[str, float]:
        n = max(1, len(self.items))
        return {"evolving_rubrics/num_active_rubrics": sum(sum(1 for i in v if i.adaptive) for v in self.items.values()) / n,
                "evolving_rubrics/num_persistent_rubrics": sum(sum(1 for i in v if not i.adaptive) for v in self.items.values()) / n,
                "evolving_rubrics/num_inactive_rubrics": sum(len(v) for v in self.inactive.values()) / n}

    def spec_for(self, prompt_id: str, query: str) -> dict:
        return {"query": query, "rubrics": [{"description": i.description, "weight": i.weight, "type": i.kind} for i in self.items.get(prompt_id, [])]}

    def state_dict(self) -> dict:
        return {"active": {k: [vars(i) for i in v] for k, v in self.items.items()},
                "inactive": {k: [vars(i) for i in v] for k, v in self.inactive.items()}}

    def load_state_dict(self, sd: dict) -> None:
        if "active" not in sd:  # earlier format: the active items only
            sd = {"active": sd, "inactive": {}}
        self.items = {k: [RubricItem(**i) for i in v] for k, v in sd["active"].items()}
        self.inactive = {k: [RubricItem(**i) for i in v] for k, v in sd["inactive"].items()}

    def dumps(self) -> str:
        return json.dumps(self.state_dict())


def rubric_reward_metrics(per_response: list[list[dict]]) -> dict[str, float]:
    """Mean and spread of the weighted item scores, split by item type (``open_instruct/rubrics/metrics.py:19-56``).
    ``per_response[k]`` is the per-item list that ``score_rubrics`` returns for response k, each entry carrying ``score``,
    ``weight`` and ``type`` ("evolving" | "persistent"; missing = persistent)."""
    ev = [d["score"] * d["weight"] for items in per_response for d in items if d.get("type") == "evolving"]
    ps = [d["score"] * d["weight"] for items in per_response for d in items if d.get("type") != "evolving"]
    return {"evolving_rubrics/avg_evolving_reward": statistics.fmean(ev) if ev else 0.0,
            "evolving_rubrics/std_evolving_reward": statistics.pstdev(ev) if ev else 0.0,
            "evolving_rubrics/avg_persistent_reward": statistics.fmean(ps) if ps else 0.0,
            "evolving_rubrics/std_persistent_reward": statistics.pstdev(ps) if ps else 0.0}


def rubric_key_stats(prompt_ids: list[str], per_response: list[list[dict]]) -> dict[tuple[str, str], dict]:
    """(prompt id, item description) -> {"mean", "std"} of the item's scores over the responses of a step: the input of
    ``RubricBuffer.filter``."""
    acc: dict[tuple[str, str], list[float]] = {}
    for pid, items in zip(prompt_ids, per_response):
        for d in items:
            acc.setdefault((pid, d["description"]), []).append(float(d["score"]))
    return {k: {"mean": statistics.fmean(v), "std": statistics.pstdev(v) if len(v) > 1 else 0.0} for k, v in acc.items()}


_EVOLVE_PROMPT = ("You maintain grading rubrics for the question below. Here are several sampled answers. Propose rubric items that "
                  "separate good answers from bad ones and are NOT already covered by the existing rubrics: 'positive' items describe "
                  "what strong answers do, 'negative' items describe failure patterns.\n\n[Question]\n{query}\n\n[Existing rubrics]\n{existing}\n\n"
                  "[Answers]\n{answers}\n\nRespond in JSON: {{\"positive_rubrics\": [{{\"description\": \"...\", \"title\": \"...\"}}], "
                  "\"negative_rubrics\": [{{\"description\": \"...\", \"title\": \"...\"}}]}}")


def extract_json_from_response(text: str) -> dict | None:
    """First JSON object in a model reply (code fences tolerated)."""
    import re

    m = re.search(r"\{.*\}", text.replace("```json", "").replace("```", ""), re.S)
    if not m:
        return None
    try:
        out = json.loads(m.group(0))
        return out if isinstance(out, dict) else None
    except json.JSONDecodeError:
        return None


class RubricManager:
    """One evolving-rubric step per training step (the role of ``open_instruct/rubrics/evolving_rubric_step.py:26-160``):
    for every prompt group, show the judge a few sampled answers and the current rubrics, parse its proposals, add them to
    the buffer as adaptive items (positive weight +1, negative weight -1), cap the active adaptive items, and return
    (metrics, ground-truth overrides keyed by dataset index).  ``ask`` is an async callable ``messages -> str``."""

    def __init__(self, ask, max_active_rubrics: int = 5, answers_shown: int = 4, answer_length_limit_in_words: int | None = 400,
                 cache_dir: str | None = None):
        self.ask, self.answers_shown, self.word_limit, self.cache_dir = ask, answers_shown, answer_length_limit_in_words, cache_dir
        self.buffer = RubricBuffer(max_active_adaptive=max_active_rubrics)

    def initialize(self, prompt_id: str, ground_truth: dict) -> None:
        if prompt_id not in self.buffer.items:
            self.buffer.add_persistent(prompt_id, [r["description"] for r in ground_truth.get("rubrics", []) if r.get("weight", 1.0) >= 0])
            neg = [r for r in ground_truth.get("rubrics", []) if r.get("weight", 1.0) < 0]
            self.buffer.items[prompt_id].extend(RubricItem(r["description"], float(r["weight"]), False) for r in neg)

    async def _propose(self, query: str, prompt_id: str, answers: list[str]) -> list[dict] | None:
        shown = answers[: self.answers_shown]
        if self.word_limit:
            shown = [" ".join(a.split()[: self.word_limit]) for a in shown]
        existing = "\n".join(f"- {i.description}" for i in self.buffer.items.get(prompt_id, [])) or "(none)"
        body = _EVOLVE_PROMPT.format(query=query, existing=existing, answers="\n\n".join(f"[Answer {k + 1}]\n{a}" for k, a in enumerate(shown)))
        try:
            parsed = extract_json_from_response(await self.ask([{"role": "user", "content": body}]))
        except Exception:  # noqa: BLE001 - transport error counts as an invalid proposal
            parsed = None
        if parsed is None:
            return None
        out = [{"description": r["description"], "weight": 1.0, "title": r.get("title", "")} for r in parsed.get("positive_rubrics", []) if r.get("description")]
        out += [{"description": r["description"], "weight": -1.0, "title": r.get("title", "")} for r in parsed.get("negative_rubrics", []) if r.get("description")]
        return out

    def step(self, decoded_responses: list[str], ground_truths: list[dict], indices: list[int], num_samples: int, training_step: int = 0):
        groups = [(indices[g] if indices else g // num_samples, ground_truths[g], decoded_responses[g:g + num_samples])
                  for g in range(0, len(decoded_responses), num_samples)]
        for idx, gt, _ in groups:
            self.initialize(str(idx), gt)

        async def run():
            return await asyncio.gather(*(self._propose(gt.get("query", ""), str(idx), answers) for idx, gt, answers in groups))

        proposals = asyncio.run(run())
        overrides, n_new, valid = {}, 0, 0
        for (idx, gt, _), prop in zip(groups, proposals):
            if prop is not None:
                valid += 1
                before = len(self.buffer.items[str(idx)])
                self.buffer.add_adaptive(str(idx), prop)
                n_new += max(0, len(self.buffer.items[str(idx)]) - before)
            overrides[idx] = {**gt, **self.buffer.spec_for(str(idx), gt.get("query", ""))}
        n = max(1, len(groups))
        active = [sum(1 for i in self.buffer.items[str(idx)] if i.adaptive) for idx, _, _ in groups]
        metrics = {"evolving_rubrics/valid_rate": valid / n, "evolving_rubrics/avg_new_rubrics": n_new / n,
                   "evolving_rubrics/avg_active_buffer": sum(active) / n, "evolving_rubrics/num_overrides": len(overrides),
                   "evolving_rubrics/skipped": len(groups) - valid, "evolving_rubrics/num_new_rubrics": n_new / n, **self.buffer.counts()}
        if self.cache_dir:
            import os

            os.makedirs(self.cache_dir, exist_ok=True)
            tmp = os.path.join(self.cache_dir, f".step_{training_step}.json.tmp")
            with open(tmp, "w") as f:
                json.dump({"step": training_step, "buffer": self.buffer.state_dict(), "proposals": proposals}, f)
            os.replace(tmp, os.path.join(self.cache_dir, f"step_{training_step}.json"))
        return metrics, overrides
