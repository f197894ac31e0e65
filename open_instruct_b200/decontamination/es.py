"""Elasticsearch as the store of the decontamination index, over its REST interface (no client library).

The reference keeps one text index per training set in an Elasticsearch server and asks it phrase queries
(``decontamination/index.py:14-79``, ``decontamination/search.py:41-140``).  This module speaks the same four requests with
``urllib``: create an index with the reference's pattern analyzer (splits on blanks and a few punctuation marks only, so
that equations and code survive), count its documents, bulk-add ``{"text", "original_id"}`` documents, and run a
``bool / filter / match_phrase`` search.  ``open_instruct_b200.decontamination.index`` fills an index,
``open_instruct_b200.decontamination.search --es_url`` queries it; without a server the in-process ``NgramIndex`` does
the same work for sets that fit in memory.

Embedding search (``index_type vector``): documents carry an L2-normalised ``vector`` (``dense_vector``, dot-product
similarity) made by ``Embedder`` - any Hugging Face encoder or decoder loaded from a local folder, mean-pooled over the tokens
(the reference hard-wires one 4096-wide embedding model and its own ``encode`` method) - and queries use the server's kNN search.

``tokenize`` restates the analyzer on the client: the n-grams sent as phrases and the token-coverage score are computed
over the same tokens the server matches (the reference tokenises queries with a spaCy model, which this image has not).
"""

from __future__ import annotations

import base64
import json
import os
import re
import urllib.error
import urllib.request

ANALYZER_PATTERN = '[ ,.?!:;()"-]|\\n|\\\\'   # what separates tokens; everything else (operators, digits, brackets) stays
_SPLIT = re.compile(ANALYZER_PATTERN)


def tokenize(text: str) -> list[str]:
    return [t for t in _SPLIT.split(text.lower()) if t]


def index_name_for(dataset: str, index_type: str = "text") -> str:
    """One index per training set and kind, named like the reference names them (``decontamination/index.py:190``)."""
    return re.sub(r"[^a-z0-9_.-]", "_", dataset.replace("/", "_").lower()) + f"_{index_type}"


class ElasticClient:
    """The handful of REST calls the decontamination tools need.  Credentials: ``ELASTIC_PASSWORD`` (user ``elastic``), as
    the reference reads them; none are sent when the variable is unset."""

    def __init__(self, url: str = "http://localhost:9200", password: str | None = None, timeout: float = 60.0):
        self.url = url.rstrip("/")
        self.timeout = timeout
        password = password if password is not None else os.environ.get("ELASTIC_PASSWORD")
        self.auth = "Basic " + base64.b64encode(f"elastic:{password}".encode()).decode() if password else None

    def _request(self, method: str, path: str, body=None, ndjson: bool = False):
        data = None
        if body is not None:
            data = ("".join(json.dumps(x) + "\n" for x in body) if ndjson else json.dumps(body)).encode()
        req = urllib.request.Request(self.url + path, data=data, method=method)
        req.add_header("Content-Type", "application/x-ndjson" if ndjson else "application/json")
        if self.auth:
            req.add_header("Authorization", self.auth)
        try:
            with urllib.request.urlopen(req, timeout=self.timeout) as r:
                raw = r.read()
        except urllib.error.HTTPError as e:
            if e.code == 404:
                return None
            raise RuntimeError(f"Elasticsearch {method} {path}: HTTP {e.code}: {e.read()[:300]!r}") from e
        return json.loads(raw) if raw else {}

    def index_exists(self, name: str) -> bool:
        return self._request("HEAD", f"/{name}") is not None

    def create_text_index(self, name: str) -> None:
        self._request("PUT", f"/{name}", {
            "settings": {"analysis": {"analyzer": {"tulu_analyzer": {"type": "pattern", "pattern": ANALYZER_PATTERN, "lowercase": True}}}},
            "mappings": {"properties": {"text": {"type": "text", "index": True, "analyzer": "tulu_analyzer"},
                                        "original_id": {"type": "integer"}}}})

    def create_vector_index(self, name: str, dims: int) -> None:
        self._request("PUT", f"/{name}", {"mappings": {"properties": {
            "text": {"type": "text"}, "original_id": {"type": "integer"},
            "vector": {"type": "dense_vector", "dims": dims, "index": True, "similarity": "dot_product"}}}})

    def knn(self, name: str, vector: list[float], k: int = 10) -> list[dict]:
        """The ``k`` documents whose vectors are closest to ``vector``: [{"_id", "_score", "_source"}], best first."""
        out = self._request("POST", f"/{name}/_search", {"knn": {"field": "vector", "query_vector": vector, "k": k, "num_candidates": 10 * k},
                                                          "_source": ["text", "original_id"]})
        if out is None:
            raise RuntimeError(f"Elasticsearch index {name} does not exist: build it with open_instruct_b200.decontamination.index")
        return list(out["hits"]["hits"])

    def count(self, name: str) -> int:
        out = self._request("GET", f"/{name}/_count")
        return int(out["count"]) if out else 0

    def bulk_add(self, name: str, docs: list[dict]) -> None:
        lines = []
        for d in docs:
            src = {"text": d["text"], "original_id": d["original_id"]}
            if "vector" in d:
                src["vector"] = d["vector"]
            lines += [{"index": {"_index": name}}, src]
        out = self._request("POST", "/_bulk?refresh=true", lines, ndjson=True)
        if out and out.get("errors"):
            raise RuntimeError(f"Elasticsearch bulk request into {name} reported errors")

    def search_phrases(self, name: str, phrases: list[str], size: int = 100) -> tuple[int, list[dict]]:
        """Documents whose text contains EVERY phrase.  Returns (total hits, [{"_id", "_source"}])."""
        out = self._request("POST", f"/{name}/_search?rest_total_hits_as_int=true&search_type=query_then_fetch",
                            {"size": size, "query": {"bool": {"filter": [{"match_phrase": {"text": p}} for p in phrases]}}})
        if out is None:
            raise RuntimeError(f"Elasticsearch index {name} does not exist: build it with open_instruct_b200.decontamination.index")
        return int(out["hits"]["total"]), list(out["hits"]["hits"])


def messages_to_index(rows: list[dict], messages_field: str = "messages", query_filter: str = "role:user", query_field: str = "content") -> list[dict]:
    """One document per message that passes ``query_filter`` (``key:value``), remembering the row it came from."""
    key, value = query_filter.split(":", 1)
    return [{"text": m[query_field], "original_id": i} for i, row in enumerate(rows) for m in row[messages_field] if m.get(key) == value]


def index_text(es: ElasticClient, name: str, docs: list[dict], batch_size: int = 1000) -> int:
    """Add ``docs`` to index ``name`` (created if missing).  A run that was interrupted resumes where the index's document
    count says it stopped, as the reference's does.  Returns the number of documents added."""
    if not es.index_exists(name):
        es.create_text_index(name)
    start = es.count(name)
    for i in range(start, len(docs), batch_size):
        es.bulk_add(name, docs[i:i + batch_size])
    return max(0, len(docs) - start)


def exact_match(es: ElasticClient, name: str, queries: list[list[str]], size: int = 100):
    """Per evaluation example (a list of field texts): 1 if some training document contains every field as a phrase.
    Returns (scores, report rows, matching training row ids)."""
    scores, report, train_ids = [], [], set()
    for fields in queries:
        if any(f is None for f in fields):
            continue
        total, hits = es.search_phrases(name, fields, size)
        scores.append(1 if total > 0 else 0)
        if total > 0:
            docs = [h["_source"] for h in hits]
            train_ids.update(d["original_id"] for d in docs)
            report.append({"query": fields, "num_hits": total, "train_docs": docs})
    return scores, report, train_ids


def ngram_match(es: ElasticClient, name: str, queries: list[list[str]], ngram_size: int = 8, size: int = 100):
    """The reference's n-gram score (``decontamination/search.py:68-140``): for every field, the share of its TOKENS that lie
    inside an n-gram found (as a phrase) in a training document; averaged over the fields; an example's score is its best
    document's.  Returns (scores, report rows, {training row id: highest score against any example})."""
    scores, report, train_best = [], [], {}
    for fields in queries:
        if any(f is None for f in fields):
            continue
        per_field, sources = [], {}
        for text in fields:
            toks = tokenize(text)
            covered: dict[str, set] = {}
            asked: dict[str, list] = {}   # a repeated n-gram is asked once
            for i in range(len(toks) - ngram_size + 1):
                gram = " ".join(toks[i:i + ngram_size])
                if gram not in asked:
                    asked[gram] = es.search_phrases(name, [gram], size)[1]
                for h in asked[gram]:
                    covered.setdefault(h["_id"], set()).update(range(i, i + ngram_size))
                    sources[h["_id"]] = h["_source"]
            per_field.append({doc: len(ix) / max(1, len(toks)) for doc, ix in covered.items()})
        if not sources:
            scores.append(0)
            continue
        agg = {doc: sum(f.get(doc, 0.0) for f in per_field) / len(fields) for doc in sources}
        ranked = sorted(agg.items(), key=lambda kv: -kv[1])
        for doc, sc in ranked:
            oid = sources[doc]["original_id"]
            train_best[oid] = max(train_best.get(oid, 0.0), sc)
        scores.append(ranked[0][1])
        report.append({"query": fields, "score": ranked[0][1], "matches": [{"doc_id": d, "source": sources[d], "score": sc} for d, sc in ranked]})
    return scores, report, train_best


class Embedder:
    """Sentence vectors from a local Hugging Face model: mean of the last hidden states over the real tokens, L2-normalised.
    Texts are batched by a token budget (``max_batch_tokens`` = longest text of the batch x batch size); a single text longer
    than the budget is skipped (None in the result), as the reference does."""

    def __init__(self, model_name_or_path: str, max_batch_tokens: int = 10000, device: str | None = None, prefix: str = ""):
        import torch
        from transformers import AutoModel, AutoTokenizer

        self.torch = torch
        self.tok = AutoTokenizer.from_pretrained(model_name_or_path)
        if self.tok.pad_token is None:
            self.tok.pad_token = self.tok.eos_token or self.tok.unk_token
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.model = AutoModel.from_pretrained(model_name_or_path).eval().to(self.device)
        self.dims = int(self.model.config.hidden_size)
        self.max_batch_tokens, self.prefix = max_batch_tokens, prefix

    def __call__(self, texts: list[str]) -> list[list[float] | None]:
        torch = self.torch
        lens = [len(self.tok.tokenize(self.prefix + t)) for t in texts]
        out: list = [None] * len(texts)
        i = 0
        while i < len(texts):
            if lens[i] > self.max_batch_tokens:
                i += 1
                continue
            j, longest = i, 0
            while j < len(texts) and lens[j] <= self.max_batch_tokens and max(longest, lens[j]) * (j - i + 1) <= self.max_batch_tokens:
                longest = max(longest, lens[j])
                j += 1
            enc = self.tok([self.prefix + t for t in texts[i:j]], return_tensors="pt", padding=True).to(self.device)
            with torch.no_grad():
                h = self.model(**enc).last_hidden_state.float()
            mask = enc["attention_mask"].unsqueeze(-1).float()
            v = torch.nn.functional.normalize((h * mask).sum(1) / mask.sum(1).clamp(min=1), dim=1)
            for k, row in enumerate(v.cpu().tolist()):
                out[i + k] = row
            i = j
        return out


def index_vectors(es: ElasticClient, name: str, docs: list[dict], embed: Embedder, batch_size: int = 256) -> int:
    """Like ``index_text`` with a ``vector`` per document; documents too long to embed are left out."""
    if not es.index_exists(name):
        es.create_vector_index(name, embed.dims)
    start, added = es.count(name), 0
    for i in range(start, len(docs), batch_size):
        chunk = docs[i:i + batch_size]
        vecs = embed([d["text"] for d in chunk])
        ready = [{**d, "vector": v} for d, v in zip(chunk, vecs) if v is not None]
        if ready:
            es.bulk_add(name, ready)
        added += len(ready)
    return added


def vector_match(es: ElasticClient, name: str, queries: list[list[str]], embed: Embedder, size: int = 10):
    """Per evaluation example (its fields joined by a blank): similarity of the closest training document.  Returns (scores,
    report rows with the five best documents, {training row id: highest score against any example})."""
    texts = [" ".join(f for f in fields if f is not None) for fields in queries]
    scores, report, train_best = [], [], {}
    for text, vec in zip(texts, embed(texts)):
        if vec is None:
            continue
        hits = es.knn(name, vec, size)[:5]
        scores.append(hits[0]["_score"] if hits else 0.0)
        for h in hits:
            oid = h["_source"]["original_id"]
            train_best[oid] = max(train_best.get(oid, 0.0), h["_score"])
        report.append({"query": text, "results": [{"score": h["_score"], "id": h["_id"], "text": h["_source"]["text"],
                                                   "original_id": h["_source"]["original_id"]} for h in hits]})
    return scores, report, train_best
