"""Test fixtures: a tiny fast tokenizer and small chat datasets built on the fly (no network)."""

import json
import os


def free_port() -> int:
    """A rendezvous port that is free right now (fixed port numbers collide on shared machines)."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def make_tokenizer(path: str, vocab_size: int = 300):
    from tokenizers import Tokenizer, models, pre_tokenizers, trainers, decoders
    from transformers import PreTrainedTokenizerFast

    corpus = [
        "hello world this is a tiny corpus for a tiny tokenizer",
        "the quick brown fox jumps over the lazy dog 0123456789",
        "user assistant system what is the answer to two plus two it is four",
        "<|user|> <|assistant|> <|system|> \n question answer reasoning step by step",
    ] * 4
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<unk>", "<s>", "</s>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(corpus, trainer)
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    os.makedirs(path, exist_ok=True)
    fast.save_pretrained(path)
    return path


def make_sft_jsonl(path: str, n: int = 40):
    rows = []
    for i in range(n):
        rows.append({"messages": [
            {"role": "user", "content": f"what is {i} plus {i + 1}"},
            {"role": "assistant", "content": f"the answer is {2 * i + 1}"},
            {"role": "user", "content": "and doubled"},
            {"role": "assistant", "content": f"it is {4 * i + 2}"},
        ]})
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    return path


def make_pref_jsonl(path: str, n: int = 32):
    with open(path, "w") as fh:
        for i in range(n):
            prompt = [{"role": "user", "content": f"say the number {i}"}]
            fh.write(json.dumps({
                "chosen": prompt + [{"role": "assistant", "content": f"the number is {i}"}],
                "rejected": prompt + [{"role": "assistant", "content": "i do not know"}],
            }) + "\n")
    return path


def make_rlvr_jsonl(path: str, n: int = 16):
    with open(path, "w") as fh:
        for i in range(n):
            fh.write(json.dumps({
                "messages": [{"role": "user", "content": f"what is {i} plus 1"}],
                "ground_truth": str(i + 1), "dataset": "gsm8k",
            }) + "\n")
    return path


class FakeElasticsearch:
    """An in-process HTTP server that answers the REST calls of the decontamination tools the way Elasticsearch does: index
    creation (the analyzer's split pattern is read from the settings), HEAD, _count, _bulk and _search with
    ``bool / filter / match_phrase`` (a phrase matches when its tokens occur contiguously in the analysed text)."""

    def __init__(self):
        import http.server
        import json
        import re
        import threading
        from urllib.parse import urlparse

        store = self.indices = {}
        log = self.requests = []

        def analyse(index, text):
            return [t for t in store[index]["split"].split(text.lower()) if t]

        def contains(hay, needle):
            n = len(needle)
            return n > 0 and any(hay[i:i + n] == needle for i in range(len(hay) - n + 1))

        class Handler(http.server.BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def _reply(self, code, body=None):
                raw = json.dumps(body).encode() if body is not None else b""
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                if self.command != "HEAD":
                    self.wfile.write(raw)

            def _body(self):
                return self.rfile.read(int(self.headers.get("Content-Length") or 0)).decode()

            def do_HEAD(self):
                name = urlparse(self.path).path.strip("/")
                log.append(("HEAD", name))
                self._reply(200 if name in store else 404)

            def do_PUT(self):
                name = urlparse(self.path).path.strip("/")
                body = json.loads(self._body())
                pat = body.get("settings", {}).get("analysis", {}).get("analyzer", {}).get("tulu_analyzer", {}).get("pattern", r"\s+")
                store[name] = {"split": re.compile(pat), "docs": [], "dims": body["mappings"]["properties"].get("vector", {}).get("dims")}
                log.append(("PUT", name))
                self._reply(200, {"acknowledged": True})

            def do_GET(self):
                parts = urlparse(self.path).path.strip("/").split("/")
                if len(parts) == 2 and parts[1] == "_count" and parts[0] in store:
                    return self._reply(200, {"count": len(store[parts[0]]["docs"])})
                self._reply(404, {"error": "no such index"})

            def do_POST(self):
                path = urlparse(self.path).path.strip("/")
                if path == "_bulk":
                    lines = [json.loads(x) for x in self._body().splitlines() if x.strip()]
                    for action, doc in zip(lines[0::2], lines[1::2]):
                        idx = store[action["index"]["_index"]]
                        idx["docs"].append({"_id": f"d{len(idx['docs'])}", "_source": doc, "tokens": None})
                    log.append(("BULK", len(lines) // 2))
                    return self._reply(200, {"errors": False})
                name, op = path.split("/")
                if op != "_search" or name not in store:
                    return self._reply(404, {"error": "no such index"})
                q = json.loads(self._body())
                if "knn" in q:   # brute-force dot products, best first
                    qv = q["knn"]["query_vector"]
                    assert len(qv) == store[name]["dims"]
                    scored = sorted(((sum(a * b for a, b in zip(qv, d["_source"]["vector"])), d) for d in store[name]["docs"]), key=lambda t: -t[0])
                    hits = [{"_id": d["_id"], "_score": sc, "_source": {k: v for k, v in d["_source"].items() if k != "vector"}} for sc, d in scored[: q["knn"]["k"]]]
                    log.append(("KNN", name))
                    return self._reply(200, {"hits": {"total": {"value": len(hits)}, "hits": hits}})
                phrases = [analyse(name, f["match_phrase"]["text"]) for f in q["query"]["bool"]["filter"]]
                hits = []
                for d in store[name]["docs"]:
                    if d["tokens"] is None:
                        d["tokens"] = analyse(name, d["_source"]["text"])
                    if all(contains(d["tokens"], p) for p in phrases):
                        hits.append({"_id": d["_id"], "_source": d["_source"]})
                log.append(("SEARCH", name))
                self._reply(200, {"hits": {"total": len(hits), "hits": hits[: q.get("size", 10)]}})

        self.server = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Handler)
        self.url = f"http://127.0.0.1:{self.server.server_address[1]}"
        self.thread = threading.Thread(target=self.server.serve_forever, daemon=True)
        self.thread.start()

    def close(self):
        self.server.shutdown()
        self.server.server_close()
