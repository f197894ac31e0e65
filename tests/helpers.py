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
