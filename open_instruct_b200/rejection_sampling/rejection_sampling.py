"""Best-of-n / worst-of-n selection: score every completion with one or more scorers, pick per prompt, vote.

Pipeline of ``open_instruct/rejection_sampling/rejection_sampling.py:231-330``: the input jsonl holds
``num_completions`` consecutive rows per prompt; the reference completion is inserted as candidate 0 of every
group; every scorer yields one score per candidate; per scorer the arg-max / arg-min candidate of each group is
found; scorers then vote (majority, random among a full tie); output rows carry ``chosen`` / ``rejected`` message
lists with their scores, and a second file carries every candidate with all its scores.

A scorer is any callable ``list[list[message]] -> list[float]``; ``RewardModelScorer`` wraps a trained reward model
(transformer + scalar head read at the last token).
"""

from __future__ import annotations

import copy
import json
import random
from collections import Counter, defaultdict
from dataclasses import dataclass, field

import torch


@dataclass
class Args:
    model_names_or_paths: list[str] = field(default_factory=list)
    input_filename: str = "completions.jsonl"
    save_filename: str = "rejected_sampling_completions.jsonl"
    save_filename_scores: str = "completion_scores.jsonl"
    num_completions: int = 1
    max_forward_batch_size: int = 64
    include_reference_completion_for_rejection_sampling: bool = True
    seed: int = 0


class RewardModelScorer:
    def __init__(self, model_dir: str, tokenizer, device=None, max_batch_tokens: int = 16384):
        import os

        from ..ckpt.hf_io import load_hf_checkpoint
        from ..models.llama import LlamaModel
        from ..models.spec import get_spec

        self.tok, self.max_batch_tokens = tokenizer, max_batch_tokens
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        spec = get_spec(model_dir)
        fused = device != "cpu" and spec.head_dim == 128 and not spec.post_norm
        self.model = LlamaModel(spec, device=device, dtype=torch.bfloat16 if fused else torch.float32, ops="fused" if fused else "ref",
                                with_lm_head=False)
        load_hf_checkpoint(model_dir, self.model.flat, spec, self.model.layout, strict=False)
        from ..reward_modeling import load_score_weight

        w = load_score_weight(model_dir)
        if w is None:
            raise FileNotFoundError(f"{model_dir} holds no score.weight: not a reward model")
        self.score = w.to(device).float()

    @torch.no_grad()
    def __call__(self, conversations: list[list[dict]]) -> list[float]:
        from ..data.collate import flatten_examples

        out: list[float] = []
        ids = [list(self.tok.apply_chat_template(c, tokenize=True)) for c in conversations]
        i = 0
        while i < len(ids):
            j, tokens = i, 0
            while j < len(ids) and (j == i or tokens + len(ids[j]) <= self.max_batch_tokens):
                tokens += len(ids[j])
                j += 1
            b = flatten_examples(ids[i:j])
            dev = self.model.device
            h = self.model.hidden_states(b["input_ids"].to(dev), b["position_ids"].to(dev), b["cu_seq_lens_q"].to(dev))
            last = b["cu_seq_lens_q"][1:].long().to(dev) - 1
            out += (h[last].float() @ self.score.t()).squeeze(-1).tolist()
            i = j
        return out


def insert_reference_candidates(completions: list[dict], num_completions: int) -> list[dict]:
    out = []
    for i, c in enumerate(completions):
        if i % num_completions == 0:
            ref = copy.deepcopy(c)
            ref["messages"][-1]["content"] = ref["reference_completion"]
            ref["model_completion"] = ref["reference_completion"]
            out.append(ref)
        out.append(c)
    return out


def majority_vote(offsets_per_model: dict[str, torch.Tensor], rng: random.Random | None = None) -> torch.Tensor:
    rng = rng or random
    names = list(offsets_per_model)
    n = offsets_per_model[names[0]].numel()
    out = torch.zeros(n, dtype=torch.long)
    for i in range(n):
        votes = [int(offsets_per_model[m][i]) for m in names]
        counts = Counter(votes)
        out[i] = counts.most_common(1)[0][0] if len(counts) != len(names) else votes[rng.randrange(len(votes))]
    return out


def select(completions: list[dict], scorers: dict, num_completions: int, include_reference: bool = True, seed: int = 0):
    """Returns (preference table, per-candidate table)."""
    cands = insert_reference_candidates(completions, num_completions)
    k = num_completions + 1
    best, worst, ref_scores = {}, {}, {}
    for name, scorer in scorers.items():
        scores = torch.tensor(scorer([c["messages"] for c in cands]), dtype=torch.float32).view(-1, k)
        ref_scores[name] = scores[:, 0].tolist()
        for i, c in enumerate(cands):
            c.setdefault("score", {})[name] = float(scores.view(-1)[i])
            c.setdefault("reference_completion_score", {})[name] = float(scores[i // k, 0])
        pool = scores if include_reference else scores[:, 1:]
        shift = 0 if include_reference else 1
        base = torch.arange(0, scores.shape[0] * k, k)
        best[name] = base + pool.argmax(1) + shift
        worst[name] = base + pool.argmin(1) + shift
    rng = random.Random(seed)
    b, w = majority_vote(best, rng), majority_vote(worst, rng)
    table = defaultdict(list)
    for i, (bi, wi) in enumerate(zip(b.tolist(), w.tolist())):
        cb, cw = cands[bi], cands[wi]
        if cb["messages"][:-1] != cw["messages"][:-1]:
            raise ValueError("chosen and rejected candidates belong to different prompts: input is not grouped by prompt")
        table["chosen"].append(cb["messages"])
        table["rejected"].append(cw["messages"])
        table["reference_completion"].append(cw["reference_completion"])
        table["reference_completion_score"].append({m: ref_scores[m][i] for m in ref_scores})
        table["chosen_score"].append(cb["score"])
        table["rejected_score"].append(cw["score"])
    kept = cands if include_reference else [c for i, c in enumerate(cands) if i % k]
    per_cand = defaultdict(list)
    for c in kept:
        for key in kept[0]:
            per_cand[key].append(c[key])
    return dict(table), dict(per_cand)


def save_jsonl(path: str, table: dict[str, list]) -> None:
    keys = list(table)
    with open(path, "w") as f:
        for i in range(len(table[keys[0]]) if keys else 0):
            f.write(json.dumps({k: table[k][i] for k in keys}) + "\n")


def main(args: Args, scorers: dict | None = None):
    with open(args.input_filename) as f:
        completions = [json.loads(line) for line in f if line.strip()]
    if scorers is None:
        from ..data.tokenize import TokenizerConfig

        scorers = {}
        for path in args.model_names_or_paths:
            tc = TokenizerConfig(tokenizer_name_or_path=path)
            scorers[path] = RewardModelScorer(path, tc.tokenizer, max_batch_tokens=args.max_forward_batch_size * 512)
    table, per_cand = select(completions, scorers, args.num_completions, args.include_reference_completion_for_rejection_sampling, args.seed)
    save_jsonl(args.save_filename, table)
    save_jsonl(args.save_filename_scores, per_cand)
    return table


if __name__ == "__main__":
    from ..config.argparser import ArgumentParserPlus

    main(ArgumentParserPlus((Args,)).parse())
