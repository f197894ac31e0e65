"""Find evaluation examples that leak into training data, and drop the contaminated training rows.

The reference indexes training sets in Elasticsearch and queries it with exact, n-gram and embedding matches
(``decontamination/index.py``, ``decontamination/search.py:41-190``).  This module does the text part without a search
server: an in-memory inverted index from word n-grams (default 8) to training rows.

* ``exact``  : a training field equals the evaluation text after whitespace/case normalisation;
* ``ngram``  : the share of the evaluation text's n-grams that occur in one training row is at least ``threshold``
  (the reference's match score, ``search.py:68-140``).

    python -m open_instruct_b200.decontamination.search --train train.jsonl --eval eval.jsonl --field text \\
        --ngram_size 8 --threshold 0.5 --output_dir out [--decontaminate]

With ``--es_url`` the training side is an Elasticsearch index filled by ``open_instruct_b200.decontamination.index`` (for
training sets that do not fit in one process); ``--train`` then names the indexed dataset, scores are the reference's
(exact: every field found as a phrase; ngram: share of the query's tokens inside matching n-grams), and
``--decontaminate`` still writes the training rows whose best score stays below ``--threshold``.
"""

from __future__ import annotations

import argparse
import json
import os
import re
from collections import Counter, defaultdict

_WS = re.compile(r"\s+")


def normalise(text: str) -> str:
    return _WS.sub(" ", text.strip().lower())


def ngrams(text: str, n: int) -> list[tuple[str, ...]]:
    toks = normalise(text).split(" ")
    return [tuple(toks[i:i + n]) for i in range(max(0, len(toks) - n + 1))]


def row_text(row: dict, fields: list[str]) -> str:
    parts = []
    for f in fields:
        v = row.get(f)
        if isinstance(v, list):  # chat messages
            parts += [m.get("content", "") if isinstance(m, dict) else str(m) for m in v]
        elif v is not None:
            parts.append(str(v))
    return "\n".join(parts)


class NgramIndex:
    def __init__(self, n: int = 8):
        self.n = n
        self.postings: dict[tuple[str, ...], set[int]] = defaultdict(set)
        self.exact: dict[str, list[int]] = defaultdict(list)
        self.size = 0

    def add(self, text: str) -> int:
        i = self.size
        self.size += 1
        self.exact[normalise(text)].append(i)
        for g in set(ngrams(text, self.n)):
            self.postings[g].add(i)
        return i

    def exact_match(self, text: str) -> list[int]:
        return list(self.exact.get(normalise(text), []))

    def ngram_match(self, text: str) -> dict[int, float]:
        """training row -> share of the query's n-grams found in it."""
        grams = ngrams(text, self.n)
        if not grams:
            return {}
        hits: Counter = Counter()
        for g in grams:
            for i in self.postings.get(g, ()):
                hits[i] += 1
        return {i: c / len(grams) for i, c in hits.items()}


def find_contamination(train_rows: list[dict], eval_rows: list[dict], train_fields: list[str], eval_fields: list[str], n: int = 8,
                       threshold: float = 0.5, mode: str = "ngram") -> dict:
    idx = NgramIndex(n)
    for r in train_rows:
        idx.add(row_text(r, train_fields))
    contaminated_train: set[int] = set()
    matches = []
    for j, e in enumerate(eval_rows):
        q = row_text(e, eval_fields)
        if mode == "exact":
            m = {i: 1.0 for i in idx.exact_match(q)}
        else:
            m = {i: s for i, s in idx.ngram_match(q).items() if s >= threshold}
        if m:
            matches.append({"eval_index": j, "train_matches": sorted(m.items(), key=lambda kv: -kv[1])[:20]})
            contaminated_train.update(m)
    return {"eval_contaminated": len(matches), "eval_total": len(eval_rows), "train_contaminated": sorted(contaminated_train), "matches": matches}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--train", required=True)
    ap.add_argument("--eval", required=True)
    ap.add_argument("--field", nargs="+", default=["text"], help="evaluation fields")
    ap.add_argument("--train_field", nargs="+", default=["messages"])
    ap.add_argument("--ngram_size", type=int, default=8)
    ap.add_argument("--threshold", type=float, default=0.5)
    ap.add_argument("--index_type", choices=["exact", "ngram", "vector"], default="ngram")
    ap.add_argument("--model", default=None, help="vector search: folder of the Hugging Face model that embedded the index")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--decontaminate", action="store_true")
    ap.add_argument("--es_url", default=None, help="query an Elasticsearch index of --train instead of indexing it in this process")
    ap.add_argument("--search_size", type=int, default=100, help="hits fetched per Elasticsearch query")
    a = ap.parse_args(argv)
    load = lambda p: [json.loads(line) for line in open(p) if line.strip()]
    if a.es_url:
        return _main_elasticsearch(a, load(a.eval))
    if a.index_type == "vector":
        raise SystemExit("vector search runs against an Elasticsearch index: give --es_url")
    train, ev = load(a.train), load(a.eval)
    rep = find_contamination(train, ev, a.train_field, a.field, a.ngram_size, a.threshold, a.index_type)
    os.makedirs(a.output_dir, exist_ok=True)
    with open(os.path.join(a.output_dir, "contamination_report.json"), "w") as f:
        json.dump(rep, f, indent=1)
    if a.decontaminate:
        bad = set(rep["train_contaminated"])
        with open(os.path.join(a.output_dir, "train_decontaminated.jsonl"), "w") as f:
            for i, r in enumerate(train):
                if i not in bad:
                    f.write(json.dumps(r) + "\n")
    return rep


def _main_elasticsearch(a, eval_rows: list[dict]) -> dict:
    from . import es as es_mod

    client = es_mod.ElasticClient(a.es_url)
    index = es_mod.index_name_for(a.train, "text")
    queries = [[row.get(f) for f in a.field] for row in eval_rows]
    if a.index_type == "vector":
        if not a.model:
            raise SystemExit("--index_type vector needs --model")
        index = es_mod.index_name_for(a.train, "vector")
        scores, report, train_scores = es_mod.vector_match(client, index, queries, es_mod.Embedder(a.model), a.search_size)
    elif a.index_type == "exact":
        scores, report, ids = es_mod.exact_match(client, index, queries, a.search_size)
        train_scores = {i: 1.0 for i in ids}
    else:
        scores, report, train_scores = es_mod.ngram_match(client, index, queries, a.ngram_size, a.search_size)
    bad = sorted(i for i, sc in train_scores.items() if sc >= a.threshold)
    rep = {"eval_contaminated": sum(1 for sc in scores if sc >= a.threshold), "eval_total": len(scores), "train_contaminated": bad,
           "mean_match_score": sum(scores) / max(1, len(scores)), "matches": report}
    os.makedirs(a.output_dir, exist_ok=True)
    with open(os.path.join(a.output_dir, "contamination_report.json"), "w") as f:
        json.dump(rep, f, indent=1)
    if a.decontaminate:
        from ..data.mixer import _load_any

        drop = set(bad)
        with open(os.path.join(a.output_dir, "train_decontaminated.jsonl"), "w") as f:
            for i, r in enumerate(_load_any(a.train, "train", None)):
                if i not in drop:
                    f.write(json.dumps(r) + "\n")
    return rep


if __name__ == "__main__":
    main()
