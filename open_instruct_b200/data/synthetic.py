"""Synthetic workloads of the benchmark shapes (no dataset or checkpoint is needed).

SFT: packed rows of ``seq_len`` tokens; example lengths log-uniform in ``[min_len, seq_len]``; the
first ``prompt_frac`` of every example is a masked prompt; token ids uniform in the vocabulary.
DPO: pairs sharing a prompt of 64-512 tokens with independent responses of 64-1024 tokens.
"""

from __future__ import annotations

import math

import torch

from .collate import IGNORE, flatten_examples


def sft_pack(seq_len: int, vocab: int, gen: torch.Generator, min_len: int = 128, prompt_frac: float = 0.3) -> dict:
    """One packed row of exactly ``seq_len`` tokens (the last example is cut to fit)."""
    ids, labels = [], []
    used = 0
    while used < seq_len:
        u = torch.rand((), generator=gen).item()
        n = int(round(math.exp(math.log(min_len) + u * (math.log(seq_len) - math.log(min_len)))))
        n = max(2, min(n, seq_len - used))
        x = torch.randint(0, vocab, (n,), generator=gen)
        lab = x.clone()
        lab[: int(n * prompt_frac)] = IGNORE
        ids.append(x)
        labels.append(lab)
        used += n
    return flatten_examples(ids, labels)


def sft_step_batches(n_packs: int, seq_len: int, vocab: int, seed: int, packs_per_micro: int = 1) -> list[dict]:
    """``n_packs`` packed rows grouped into micro-batches of ``packs_per_micro`` rows each."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(0, n_packs, packs_per_micro):
        rows = [sft_pack(seq_len, vocab, gen) for _ in range(packs_per_micro)]
        if packs_per_micro == 1:
            out.append(rows[0])
        else:
            ids = [r["input_ids"][a:b] for r in rows for a, b in zip(r["cu_seq_lens_q"][:-1], r["cu_seq_lens_q"][1:])]
            labs = [r["labels"][a:b] for r in rows for a, b in zip(r["cu_seq_lens_q"][:-1], r["cu_seq_lens_q"][1:])]
            out.append(flatten_examples(ids, labs))
    return out


def dpo_pairs(n_pairs: int, vocab: int, seed: int, max_len: int = 2048) -> list[dict]:
    gen = torch.Generator().manual_seed(seed)
    rows = []
    for i in range(n_pairs):
        p = int(torch.randint(64, 513, (), generator=gen))
        prompt = torch.randint(0, vocab, (p,), generator=gen)
        row = {"index": i}
        for side in ("chosen", "rejected"):
            r = int(torch.randint(64, 1025, (), generator=gen))
            resp = torch.randint(0, vocab, (r,), generator=gen)
            ids = torch.cat([prompt, resp])[:max_len]
            lab = ids.clone()
            lab[:p] = IGNORE
            row[f"{side}_input_ids"] = ids
            row[f"{side}_labels"] = lab
        rows.append(row)
    return rows
