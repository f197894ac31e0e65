"""Acceptance rates, win rates and annotator agreement from pairwise annotation records.

Semantics follow the reference's annotation app (``human_eval/app.py:147-265``, ``human_eval/compute_metrics.py``):
several annotators may judge the same instance; rates use the LATEST judgement per instance, agreement compares the last
two judgements of every instance that has more than one.  A record is a mapping with ``instance_id``, ``model_a``,
``model_b``, ``completion_a_is_acceptable``, ``completion_b_is_acceptable`` ("yes"/"no") and ``preference``
("a-is-better", "a-is-slightly-better", "tie", "b-is-slightly-better", "b-is-better").
"""

from __future__ import annotations

from collections import Counter, defaultdict

PREFERENCES = ("a-is-better", "a-is-slightly-better", "tie", "b-is-slightly-better", "b-is-better")


def _get(rec, key):
    return rec[key] if isinstance(rec, dict) else getattr(rec, key)


def acceptance_results(records, model_a: str, model_b: str) -> dict:
    per_model: dict[str, dict[str, list[str]]] = {model_a: defaultdict(list), model_b: defaultdict(list)}
    for r in records:
        per_model[_get(r, "model_a")][_get(r, "instance_id")].append(_get(r, "completion_a_is_acceptable"))
        per_model[_get(r, "model_b")][_get(r, "instance_id")].append(_get(r, "completion_b_is_acceptable"))
    multi = [i for i, v in per_model[model_a].items() if len(v) > 1]
    agreement = {"num_instances_with_multiple_annotations": len(multi), "acceptance_agreement": None}
    if multi:
        same = {m: sum(len(set(per_model[m][i][-2:])) == 1 for i in multi) for m in (model_a, model_b)}
        agreement["acceptance_agreement"] = (same[model_a] + same[model_b]) / (2 * len(multi))
        for m in (model_a, model_b):
            agreement[f"{m}_acceptance_agreement"] = same[m] / len(multi)
    out = {m: (sum(v[-1] == "yes" for v in per_model[m].values()) / len(per_model[m]) if per_model[m] else 0.0)
           for m in (model_a, model_b)}
    out["agreement"] = agreement
    return out


def comparison_results(records, model_a: str, model_b: str) -> dict:
    per_instance: dict[str, list[tuple[str, str]]] = defaultdict(list)   # (winner or "tie", strength)
    for r in records:
        a, b, pref = _get(r, "model_a"), _get(r, "model_b"), _get(r, "preference")
        if pref == "tie":
            per_instance[_get(r, "instance_id")].append(("tie", ""))
        elif pref in PREFERENCES:
            per_instance[_get(r, "instance_id")].append((a if pref.startswith("a-") else b, "slightly" if "slightly" in pref else "clearly"))
    latest = [v[-1] for v in per_instance.values()]
    n = max(len(latest), 1)
    counts = Counter("tie" if w == "tie" else f"{w} is {s} better" for w, s in latest)
    rates = {k: c / n for k, c in counts.items()}
    rates[f"{model_a}_wins"] = sum(w == model_a for w, _ in latest) / n
    rates[f"{model_b}_wins"] = sum(w == model_b for w, _ in latest) / n
    multi = [v for v in per_instance.values() if len(v) > 1]
    agreement = {"num_instances_with_multiple_annotations": len(multi), "comparison_agreement": None,
                 "relaxed_comparison_agreement": None}
    if multi:
        strict = relaxed = 0.0
        for v in multi:
            last_two = [w for w, _ in v[-2:]]
            if last_two[0] == last_two[1]:
                strict += 1
                relaxed += 1
            elif "tie" in last_two:
                relaxed += 0.5   # a tie against a preference counts as half an agreement
        agreement["comparison_agreement"] = strict / len(multi)
        agreement["relaxed_comparison_agreement"] = relaxed / len(multi)
    rates["agreement"] = agreement
    return rates


def summarize(records, users: list[str] | None = None, num_instances: int | None = None) -> dict:
    """Everything the summary page shows: contributions per annotator, progress, and per model pair the acceptance,
    comparison and feedback results."""
    judgements = [r for r in records if not _get(r, "instance_quality")]
    out = {"user_contributions": dict(Counter(_get(r, "evaluator") for r in judgements))}
    for u in users or []:
        out["user_contributions"].setdefault(u, 0)
    out["user_contributions"]["all"] = len(judgements)
    done = {_get(r, "instance_index") for r in judgements}
    out["progress"] = {"completed": len(done), "total": num_instances,
                       "missing_indices": sorted(set(range(num_instances or 0)) - done)}
    pairs = sorted({tuple(sorted((_get(r, "model_a"), _get(r, "model_b")))) for r in records})
    out["model_pairs"] = [list(p) for p in pairs]
    out["results"] = {}
    for a, b in pairs:
        mine = [r for r in records if {_get(r, "model_a"), _get(r, "model_b")} == {a, b}]
        feedback = defaultdict(list)
        for r in mine:
            if _get(r, "instance_quality"):
                feedback[_get(r, "instance_quality")].append(_get(r, "instance_index"))
        cmp_records = [r for r in mine if not _get(r, "instance_quality")]
        out["results"][f"{a}_vs_{b}"] = {"acceptance_results": acceptance_results(cmp_records, a, b),
                                         "comparison_results": comparison_results(cmp_records, a, b),
                                         "feedback_records": dict(feedback)}
    return out
