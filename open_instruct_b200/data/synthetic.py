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


def make_byte_tokenizer(path: str, vocab_size: int = 320) -> str:
    """A small byte-level BPE tokenizer written to ``path`` (benchmarks and tests run without network access;
    random-init models only need token ids below their vocabulary size)."""
    import os

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast

    corpus = ["what is 1234 + 5678 - 90 * 12 ?", "the answer is 0123456789", "user assistant system compute the value of the expression",
              "<|user|> <|assistant|> <|system|> \n step by step reasoning result"] * 4
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<unk>", "<s>", "</s>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(corpus, trainer)
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    os.makedirs(path, exist_ok=True)
    fast.save_pretrained(path)
    return path


def arithmetic_rlvr_jsonl(path: str, n: int, seed: int = 0) -> str:
    """Seeded synthetic arithmetic prompts: two to four integers in [0, 10^4] joined by + - *; the ground truth is the
    exact value; verifier ``gsm8k`` (last integer of the response must equal it)."""
    import json
    import random

    rng = random.Random(seed)
    with open(path, "w") as fh:
        for _ in range(n):
            k = rng.randint(2, 4)
            nums = [rng.randint(0, 10**4) for _ in range(k)]
            ops = [rng.choice("+-*") for _ in range(k - 1)]
            expr = str(nums[0]) + "".join(f" {o} {v}" for o, v in zip(ops, nums[1:]))
            fh.write(json.dumps({"messages": [{"role": "user", "content": f"Compute the value of the expression: {expr}. Give the final integer."}],
                                 "ground_truth": str(eval(expr)), "dataset": "gsm8k"}) + "\n")  # noqa: S307 - digits and + - * only
    return path
