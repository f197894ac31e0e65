"""Teacher top-k log-probabilities for every position of a tokenised dataset, written as compressed parquet shards.

The reference asks vLLM for ``prompt_logprobs=k`` and streams rows into parquet
(``open_instruct/sample_logits_vllm.py:60-342``).  Here the teacher is this framework's own model: one packed forward per
batch gives the logits, ``topk`` + ``log_softmax`` the sorted distribution, ``distill/compression.py`` the bytes.

    python -m open_instruct_b200.distill.sample_logits --model <hf dir | preset> --dataset_mixer_list data.jsonl 1.0 --output_dir out
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch

from .compression import QuantizationConfig, compress_logprobs, pack_bits


@dataclass
class Args:
    model: str = "tiny"
    dataset_mixer_list: list[str] = field(default_factory=list)
    dataset_mixer_list_splits: list[str] = field(default_factory=lambda: ["train"])
    output_dir: str = "teacher_logits"
    top_k: int = 64
    max_seq_length: int = 4096
    max_batch_tokens: int = 16384
    rows_per_shard: int = 2048
    max_samples: int | None = None
    temperature: float = 1.0


@torch.no_grad()
def topk_logprobs(model, input_ids: torch.Tensor, position_ids: torch.Tensor, cu: torch.Tensor, k: int, temperature: float = 1.0):
    """(values [T, k] sorted descending, ids [T, k]) of the next-token distribution at every packed position."""
    logits = model.logits(input_ids, position_ids, cu).float() / temperature
    lse = torch.logsumexp(logits, dim=-1, keepdim=True)
    vals, ids = torch.topk(logits, k, dim=-1)
    return vals - lse, ids


class ParquetShardWriter:
    def __init__(self, out_dir: str, rows_per_shard: int):
        os.makedirs(out_dir, exist_ok=True)
        self.out_dir, self.rows_per_shard, self.rows, self.shard = out_dir, rows_per_shard, [], 0

    def add(self, row: dict) -> None:
        self.rows.append(row)
        if len(self.rows) >= self.rows_per_shard:
            self.flush()

    def flush(self) -> None:
        if not self.rows:
            return
        import pyarrow as pa
        import pyarrow.parquet as pq

        table = pa.Table.from_pylist(self.rows)
        pq.write_table(table, os.path.join(self.out_dir, f"part-{self.shard:05d}.parquet"), compression="zstd")
        self.shard += 1
        self.rows = []


def process_dataset(model, rows, cfg: QuantizationConfig, args: Args, writer: ParquetShardWriter) -> int:
    from ..data.collate import flatten_examples

    dev = model.device
    n, i = 0, 0
    rows = [r for r in rows]
    while i < len(rows):
        j, tokens = i, 0
        while j < len(rows) and (j == i or tokens + len(rows[j]["input_ids"]) <= args.max_batch_tokens):
            tokens += len(rows[j]["input_ids"])
            j += 1
        b = flatten_examples([r["input_ids"][: args.max_seq_length] for r in rows[i:j]])
        vals, ids = topk_logprobs(model, b["input_ids"].to(dev), b["position_ids"].to(dev), b["cu_seq_lens_q"].to(dev), cfg.k, args.temperature)
        comp = compress_logprobs(vals.cpu(), cfg)
        pid = pack_bits(ids.cpu(), cfg.id_bits)
        cu = b["cu_seq_lens_q"].tolist()
        for r, a, e in zip(rows[i:j], cu[:-1], cu[1:]):
            writer.add({"input_ids": list(r["input_ids"][: args.max_seq_length]), "compressed_logprobs": comp[a:e].numpy().tobytes(),
                        "packed_indices": pid[a:e].numpy().tobytes(), "num_positions": e - a})
            n += 1
        i = j
    writer.flush()
    return n


def main(args: Args) -> int:
    from ..ckpt.hf_io import load_hf_checkpoint
    from ..data.mixer import get_cached_dataset_tulu
    from ..data.tokenize import TokenizerConfig
    from ..models.llama import LlamaModel
    from ..models.spec import get_spec

    spec = get_spec(args.model)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    fused = dev == "cuda" and spec.head_dim == 128 and not spec.qk_norm and not spec.attention_bias
    model = LlamaModel(spec, device=dev, dtype=torch.bfloat16 if fused else torch.float32, ops="fused" if fused else "ref")
    if os.path.isdir(args.model):
        load_hf_checkpoint(args.model, model.flat.detach(), spec, strict=False)
    tc = TokenizerConfig(tokenizer_name_or_path=args.model)
    ds = get_cached_dataset_tulu(args.dataset_mixer_list, args.dataset_mixer_list_splits, tc, ["sft_tulu_tokenize_and_truncate_v1"],
                                 [{"max_seq_length": args.max_seq_length}], target_columns=["input_ids", "labels", "attention_mask"])
    rows = [ds[i] for i in range(len(ds) if args.max_samples is None else min(len(ds), args.max_samples))]
    cfg = QuantizationConfig(k=args.top_k, vocab_size=spec.vocab_size)
    return process_dataset(model, rows, cfg, args, ParquetShardWriter(args.output_dir, args.rows_per_shard))


if __name__ == "__main__":
    from ..config.argparser import ArgumentParserPlus

    main(ArgumentParserPlus((Args,)).parse())
