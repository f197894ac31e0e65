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
    return final, [{"description": r["description"], "weight": r.get("weight", 1.0), "score": s} for r, s in zip(rubrics, scores)]


@dataclass
class RubricItem:
    description: str
    weight: float = 1.0
    adaptive: bool = False
    history: list[float] = field(default_factory=list)


class RubricBuffer:
    """Per-prompt rubric store: persistent items never leave; adaptive items are capped and retired."""

    def __init__(self, max_active_adaptive: int = 5, min_std: float = 1e-6):
        self.items: dict[str, list[RubricItem]] = {}
        self.max_active_adaptive, self.min_std = max_active_adaptive, min_std

    def add_persistent(self, prompt_id: str, descriptions: list[str], weight: float = 1.0) -> None:
        self.items.setdefault(prompt_id, []).extend(RubricItem(d, weight, False) for d in descriptions)

    def add_adaptive(self, prompt_id: str, proposals: list[dict]) -> None:
        cur = self.items.setdefault(prompt_id, [])
        known = {i.description for i in cur}
        for p in proposals:
            if p["description"] not in known:
                cur.append(RubricItem(p["description"], float(p.get("weight", 1.0)), True))
        adaptive = [i for i in cur if i.adaptive]
        for extra in adaptive[: max(0, len(adaptive) - self.max_active_adaptive)]:
            cur.remove(extra)

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

    def spec_for(self, prompt_id: str, query: str) -> dict:
        return {"query": query, "rubrics": [{"description": i.description, "weight": i.weight} for i in self.items.get(prompt_id, [])]}

    def state_dict(self) -> dict:
        return {k: [vars(i) for i in v] for k, v in self.items.items()}

    def load_state_dict(self, sd: dict) -> None:
        self.items = {k: [RubricItem(**i) for i in v] for k, v in sd.items()}

    def dumps(self) -> str:
        return json.dumps(self.state_dict())
