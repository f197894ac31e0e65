"""Dataset builders and inspection helpers (the generic part of the reference's ``scripts/data/**``).

* ``qa_to_messages`` / ``gsm8k_to_rlvr``: question-answer rows -> chat ``messages`` (``scripts/data/gsm8k.py``) and ->
  RLVR rows (``messages`` + ``ground_truth`` + ``dataset``) with the final number after ``####`` as ground truth;
* ``counter_env_samples`` / ``guess_number_env_samples``: prompts for the two example tool environments with their
  per-sample ``env_config`` (``scripts/data/create_test_env_datasets.py``);
* ``messages_statistics``: turn / prompt / response / total token statistics and length-threshold counts
  (``scripts/data/get_statistics.py``);
* ``token_length_histogram``: bucketed token-length distribution of a column (``scripts/data/get_token_distribution.py``
  plots it; here the buckets are returned and optionally written as JSON).

* ``fill_identity_placeholders``: "who are you" seed conversations with ``<|MODEL_NAME|>``-style placeholders -> rows for one
  model (``scripts/data/build_hardcoded.py``), optionally only the rows tagged for a model family.

Everything works on lists of dicts or JSONL files: no hub access is needed.

    python -m open_instruct_b200.data.builders stats --data train.jsonl --tokenizer /path/to/tokenizer
    python -m open_instruct_b200.data.builders env --kind counter --num 100 --out counter.jsonl
    python -m open_instruct_b200.data.builders identity --data seed.jsonl --out hardcoded.jsonl --model_name "OLMo 2" --license "Apache 2.0"
"""

from __future__ import annotations

import argparse
import json
import re

import numpy as np

LENGTH_THRESHOLDS = (512, 768, 1024, 1536, 2048, 4096)


def read_jsonl(path: str) -> list[dict]:
    with open(path) as fh:
        return [json.loads(line) for line in fh if line.strip()]


def write_jsonl(rows: list[dict], path: str) -> None:
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")


# ---------------------------------------------------------------------------------------------- conversions
def qa_to_messages(rows: list[dict], question_key: str = "question", answer_key: str = "answer") -> list[dict]:
    return [{"messages": [{"role": "user", "content": r[question_key]}, {"role": "assistant", "content": r[answer_key]}],
             question_key: r[question_key], answer_key: r[answer_key]} for r in rows]


def gsm8k_final_answer(answer: str) -> str:
    """The number after the last ``####`` marker, thousands separators removed."""
    tail = answer.split("####")[-1].strip()
    m = re.search(r"-?[\d,]*\.?\d+", tail)
    return (m.group(0) if m else tail).replace(",", "")


def gsm8k_to_rlvr(rows: list[dict], dataset_name: str = "gsm8k", suffix: str = "") -> list[dict]:
    return [{"messages": [{"role": "user", "content": r["question"] + suffix}], "ground_truth": gsm8k_final_answer(r["answer"]),
             "dataset": dataset_name} for r in rows]


def counter_env_samples(num_samples: int = 100, nothink: bool = False) -> list[dict]:
    tail = " /nothink" if nothink else ""
    system = ("You are playing a counter game. Use the provided tools to increment or decrement the counter to reach the "
              "target value, then submit your answer.")
    out = []
    for i in range(num_samples):
        target = str(i % 10 + 1)
        out.append({"messages": [{"role": "system", "content": system},
                                 {"role": "user", "content": f"The counter starts at 0. Reach the target value of {target} and submit.{tail}"}],
                    "ground_truth": target, "dataset": "passthrough",
                    "env_config": {"env_configs": [{"env_name": "counter", "target": target}]}})
    return out


def guess_number_env_samples(num_samples: int = 100, nothink: bool = False) -> list[dict]:
    system = ("You are playing a number guessing game. Use the guess tool to find the secret number between 1 and 100. "
              "You will be told if your guess is too high or too low.")
    user = "Guess the secret number. Use binary search strategy for efficiency." + (" /nothink" if nothink else "")
    out = []
    for i in range(num_samples):
        secret = str(i % 100 + 1)
        out.append({"messages": [{"role": "system", "content": system}, {"role": "user", "content": user}],
                    "ground_truth": secret, "dataset": "passthrough",
                    "env_config": {"env_configs": [{"env_name": "guess_number", "number": secret}]}})
    return out


# ---------------------------------------------------------------------------------------------- statistics
def _describe(xs) -> dict:
    a = np.asarray(xs, dtype=np.float64)
    if a.size == 0:
        return {"count": 0}
    q = np.percentile(a, [25, 50, 75])
    return {"count": int(a.size), "mean": float(a.mean()), "std": float(a.std(ddof=1)) if a.size > 1 else 0.0, "min": float(a.min()),
            "25%": float(q[0]), "50%": float(q[1]), "75%": float(q[2]), "max": float(a.max())}


def messages_statistics(rows: list[dict], tokenizer, messages_key: str = "messages") -> dict:
    """System messages are ignored; lengths are token counts of the message contents without special tokens."""
    def ntok(text: str) -> int:
        return len(tokenizer(text, truncation=False, add_special_tokens=False)["input_ids"])

    turns, user_len, asst_len, total_len = [], [], [], []
    for r in rows:
        msgs = [m for m in r[messages_key] if m["role"] != "system"]
        turns.append(len(msgs))
        tot = 0
        for m in msgs:
            if m["role"] == "user":
                user_len.append(ntok(m["content"]))
                tot += user_len[-1]
            elif m["role"] == "assistant":
                asst_len.append(ntok(m["content"]))
                tot += asst_len[-1]
        total_len.append(tot)
    tl = np.asarray(total_len)
    longest = np.argsort(tl)[-100:][::-1].tolist()
    res = {"num_instances": len(rows), "turns_summary": _describe(turns), "user_prompt_lengths_summary": _describe(user_len),
           "assistant_response_lengths_summary": _describe(asst_len), "total_lengths_summary": _describe(total_len),
           "top_100_longest_instances": [rows[i]["id"] for i in longest] if rows and "id" in rows[0] else None}
    for t in LENGTH_THRESHOLDS:
        res[f"num_instances_with_total_length_gt_{t}"] = int((tl > t).sum())
    return res


def token_length_histogram(rows: list[dict], tokenizer, column: str = "messages", bucket: int = 256, max_len: int | None = None) -> dict:
    """Token lengths of ``column`` (chat messages are rendered with the tokenizer's template when it has one, else joined)
    counted in buckets of ``bucket`` tokens."""
    lens = []
    for r in rows:
        v = r[column]
        if isinstance(v, list):
            if getattr(tokenizer, "chat_template", None):
                ids = tokenizer.apply_chat_template(v, tokenize=True)
                ids = ids["input_ids"] if isinstance(ids, dict) else ids
                lens.append(len(ids))
                continue
            v = "\n".join(m["content"] for m in v)
        lens.append(len(tokenizer(v, add_special_tokens=False)["input_ids"]))
    a = np.asarray(lens)
    top = int(max_len or (a.max() if a.size else 0))
    edges = list(range(0, top + bucket, bucket))
    counts = np.histogram(a, bins=edges)[0].tolist() if a.size and len(edges) > 1 else []
    return {"bucket": bucket, "edges": edges, "counts": counts, "summary": _describe(lens),
            "over_max": int((a > top).sum()) if a.size else 0}


IDENTITY_PLACEHOLDERS = {"model_name": "<|MODEL_NAME|>", "posttrain_recipe": "<|POSTTRAIN_RECIPE|>", "context_length": "<|CONTEXT_LENGTH|>",
                         "base_model": "<|BASE_MODEL|>", "date_cutoff": "<|DATE_CUTOFF|>", "license": "<|LICENSE|>",
                         "weights_link": "<|WEIGHTS_LINK|>"}


def fill_identity_placeholders(rows: list[dict], values: dict, filter_tags: list[str] | None = None, messages_key: str = "messages") -> list[dict]:
    """Seed conversations about the model itself, with placeholders such as ``<|MODEL_NAME|>`` in any turn, made concrete for one
    model.  ``values`` maps the names in ``IDENTITY_PLACEHOLDERS`` (or raw placeholder strings) to text; ``filter_tags`` drops
    rows whose ``tags`` list shares an entry with it (rows written for another family).  A row that still holds a known
    placeholder afterwards is an error: better no identity data than one that says ``<|MODEL_NAME|>``."""
    table = {IDENTITY_PLACEHOLDERS.get(k, k): str(v) for k, v in values.items() if v is not None}
    out = []
    for row in rows:
        if filter_tags and set(filter_tags) & set(row.get("tags") or []):
            continue
        new = dict(row)
        msgs = []
        for m in row[messages_key]:
            text = m["content"]
            for ph, val in table.items():
                text = text.replace(ph, val)
            left = [ph for ph in IDENTITY_PLACEHOLDERS.values() if ph in text]
            if left:
                raise ValueError(f"no value given for {left} (row: {text[:80]!r})")
            msgs.append({**m, "content": text})
        new[messages_key] = msgs
        out.append(new)
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("stats")
    s.add_argument("--data", required=True)
    s.add_argument("--tokenizer", required=True)
    s.add_argument("--histogram_column", default=None)
    e = sub.add_parser("env")
    e.add_argument("--kind", choices=["counter", "guess_number"], required=True)
    e.add_argument("--num", type=int, default=100)
    e.add_argument("--nothink", action="store_true")
    e.add_argument("--out", required=True)
    g = sub.add_parser("gsm8k")
    g.add_argument("--data", required=True)
    g.add_argument("--out", required=True)
    g.add_argument("--rlvr", action="store_true")
    h = sub.add_parser("identity")
    h.add_argument("--data", required=True, help="seed conversations (.jsonl) with placeholders")
    h.add_argument("--out", required=True)
    h.add_argument("--filter_tags", nargs="*", default=None)
    for name in IDENTITY_PLACEHOLDERS:
        h.add_argument(f"--{name}", default=None)
    args = ap.parse_args(argv)
    if args.cmd == "identity":
        write_jsonl(fill_identity_placeholders(read_jsonl(args.data), {k: getattr(args, k) for k in IDENTITY_PLACEHOLDERS}, args.filter_tags), args.out)
    elif args.cmd == "env":
        write_jsonl((counter_env_samples if args.kind == "counter" else guess_number_env_samples)(args.num, args.nothink), args.out)
    elif args.cmd == "gsm8k":
        rows = read_jsonl(args.data)
        write_jsonl(gsm8k_to_rlvr(rows) if args.rlvr else qa_to_messages(rows), args.out)
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
        rows = read_jsonl(args.data)
        out = {"statistics": messages_statistics(rows, tok)}
        if args.histogram_column:
            out["histogram"] = token_length_histogram(rows, tok, args.histogram_column)
        print(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
