"""Tokenised SFT mixes as flat numpy shards, and a reader that serves fixed-length packed windows.

On-disk layout (same as the reference's converter, ``open_instruct/numpy_dataset_conversion.py:1-10``):

    token_ids_part_XXXX.npy      raw token ids, uint8/16/32/64 chosen from the vocabulary size
    labels_mask_part_XXXX.npy    raw bool, 1 = trainable position
    token_ids_part_XXXX.csv.gz   "start,end" per document, relative to the shard
    tokenizer/                   tokenizer snapshot
    dataset_statistics.json/.txt

The files are headerless (np.memmap), sharded at ``max_shard_gb``.  Conversion is resumable: samples are
appended to three ``*.partial.bin`` files and the boundaries file is the commit log - after a crash the
token and label files are truncated to the end of the last complete (start, end) pair
(``numpy_dataset_conversion.py:105-134``).
"""

from __future__ import annotations

import gzip
import json
import os
import pathlib
from dataclasses import dataclass

import numpy as np

TOKEN_IDS_NPY_GLOB = "token_ids_part_*.npy"
LABELS_MASK_NPY_GLOB = "labels_mask_part_*.npy"
TOKEN_IDS_METADATA_GLOB = "token_ids_part_*.csv.gz"
_PAIR = np.dtype(np.int64).itemsize * 2


def select_token_dtype(vocab_size: int):
    for dt in (np.uint8, np.uint16, np.uint32, np.uint64):
        if vocab_size - 1 <= np.iinfo(dt).max:
            return dt
    raise ValueError(f"vocab size {vocab_size} does not fit an unsigned numpy integer")


class ShardWriter:
    """Append-only writer with a commit log; ``finalize()`` cuts the stream into shards."""

    def __init__(self, output_dir: str | os.PathLike, vocab_size: int, resume: bool = False, sync_every: int = 1000):
        self.dir = pathlib.Path(output_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.dtype = select_token_dtype(vocab_size)
        self.item = np.dtype(self.dtype).itemsize
        self.paths = {k: self.dir / f"_{k}.partial.bin" for k in ("tokens", "labels", "boundaries")}
        self.num_samples, self.position = self._recover() if resume else self._reset()
        self.fh = {k: open(p, "ab") for k, p in self.paths.items()}
        self.sync_every, self._since_sync = sync_every, 0

    def _reset(self) -> tuple[int, int]:
        for p in self.paths.values():
            p.unlink(missing_ok=True)
        return 0, 0

    def _recover(self) -> tuple[int, int]:
        if not all(p.exists() for p in self.paths.values()):
            return self._reset()
        b = self.paths["boundaries"]
        whole = (b.stat().st_size // _PAIR) * _PAIR
        os.truncate(b, whole)
        n = whole // _PAIR
        pos = int(np.memmap(b, mode="r", dtype=np.int64, shape=(n, 2))[-1, 1]) if n else 0
        os.truncate(self.paths["tokens"], pos * self.item)
        os.truncate(self.paths["labels"], pos)
        return n, pos

    def append(self, input_ids, labels) -> None:
        ids = np.asarray(input_ids)
        if ids.size and int(ids.max()) > np.iinfo(self.dtype).max:
            raise ValueError("token id outside the range of the shard dtype")
        mask = np.asarray(labels) != -100
        if mask.shape != ids.shape:
            raise ValueError("labels and input_ids differ in length")
        # data first, commit record last
        self.fh["tokens"].write(ids.astype(self.dtype).tobytes())
        self.fh["labels"].write(mask.astype(np.bool_).tobytes())
        end = self.position + ids.size
        self._since_sync += 1
        if self._since_sync >= self.sync_every:
            self.sync()
        self.fh["boundaries"].write(np.array([self.position, end], dtype=np.int64).tobytes())
        self.position, self.num_samples = end, self.num_samples + 1

    def sync(self) -> None:
        for k in ("tokens", "labels", "boundaries"):
            self.fh[k].flush()
            os.fsync(self.fh[k].fileno())
        self._since_sync = 0

    def finalize(self, max_shard_gb: float = 1.0) -> list[tuple[int, int]]:
        self.sync()
        for f in self.fh.values():
            f.close()
        total = self.position
        bounds = np.memmap(self.paths["boundaries"], mode="r", dtype=np.int64, shape=(self.num_samples, 2)) if self.num_samples else np.zeros((0, 2), np.int64)
        per_shard = max(1, int(max_shard_gb * 1024**3) // self.item)
        chunks = [(s, min(s + per_shard, total)) for s in range(0, total, per_shard)]
        for name, src_key, dt in (("token_ids", "tokens", self.dtype), ("labels_mask", "labels", np.bool_)):
            if total == 0:
                continue
            src = np.memmap(self.paths[src_key], mode="r", dtype=dt, shape=(total,))
            for i, (s, e) in enumerate(chunks):
                dst = np.memmap(self.dir / f"{name}_part_{i:04d}.npy", mode="w+", dtype=dt, shape=(e - s,))
                dst[:] = src[s:e]
                dst.flush()
        starts, ends = bounds[:, 0], bounds[:, 1]
        for i, (s, e) in enumerate(chunks):
            lo, hi = np.searchsorted(ends, s, side="right"), np.searchsorted(starts, e, side="left")
            with gzip.open(self.dir / f"token_ids_part_{i:04d}.csv.gz", "wt", encoding="utf-8") as f:
                for ds, de in bounds[lo:hi]:
                    f.write(f"{max(0, int(ds) - s)},{min(e - s, int(de) - s)}\n")
        for p in self.paths.values():
            p.unlink(missing_ok=True)
        return chunks


def convert_hf_to_numpy_sft(output_dir, dataset_mixer_list, dataset_mixer_list_splits, tc, dataset_transform_fn, transform_fn_args,
                            dataset_target_columns, max_seq_length: int | None = None, dataset_local_cache_dir: str = "local_dataset_cache",
                            dataset_skip_cache: bool = False, dataset_config_hash: str | None = None, shuffle_seed: int = 42,
                            resume: bool = False, tokenizer_config_only: bool = False, num_examples: int = 0, max_shard_gb: float = 1.0) -> dict:
    """Mix + tokenise (through the dataset cache), shuffle, stream into shards.  Returns the statistics dict."""
    from .mixer import get_cached_dataset_tulu_with_statistics

    out = pathlib.Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    tok = tc.tokenizer
    tok.save_pretrained(str(out / "tokenizer"))
    if tokenizer_config_only:
        return {}
    ds, stats = get_cached_dataset_tulu_with_statistics(
        dataset_mixer_list, dataset_mixer_list_splits, tc, dataset_transform_fn, transform_fn_args, target_columns=dataset_target_columns,
        dataset_local_cache_dir=dataset_local_cache_dir, dataset_skip_cache=dataset_skip_cache, dataset_config_hash=dataset_config_hash)
    ds = ds.shuffle(seed=shuffle_seed)
    if num_examples > 0:
        ds = ds.select(range(num_examples))
    w = ShardWriter(out, tok.vocab_size if len(tok) <= tok.vocab_size else len(tok), resume=resume)
    trainable = total = truncated = 0
    for i in range(w.num_samples, len(ds)):
        row = ds[i]
        ids, labels = row["input_ids"], row["labels"]
        if max_seq_length is not None and len(ids) > max_seq_length:
            ids, labels, truncated = ids[:max_seq_length], labels[:max_seq_length], truncated + 1
        w.append(ids, labels)
        total += len(ids)
        trainable += sum(1 for x in labels if x != -100)
    chunks = w.finalize(max_shard_gb)
    stats = dict(stats or {})
    stats["overall_statistics"] = {"total_instances": w.num_samples, "total_tokens": w.position, "trainable_tokens_this_run": trainable,
                                   "truncated_instances": truncated, "num_shards": len(chunks), "token_dtype": np.dtype(w.dtype).name}
    write_dataset_statistics(out, stats)
    return stats


def write_dataset_statistics(output_dir, stats: dict) -> None:
    out = pathlib.Path(output_dir)
    (out / "dataset_statistics.json").write_text(json.dumps(stats, indent=2, default=str))
    lines = ["Dataset statistics", "=" * 40]
    for k, v in stats.get("overall_statistics", {}).items():
        lines.append(f"{k}: {v}")
    for d in stats.get("per_dataset_statistics", []):
        lines.append("-" * 40)
        lines += [f"{k}: {v}" for k, v in d.items()]
    (out / "dataset_statistics.txt").write_text("\n".join(lines) + "\n")


@dataclass
class PackedWindow:
    input_ids: np.ndarray
    label_mask: np.ndarray
    cu_seqlens: np.ndarray  # document starts inside the window, plus the window length


class NumpyPackedFSLDataset:
    """Fixed-sequence-length view over the shards: window ``i`` covers tokens ``[i*L, (i+1)*L)`` of a shard,
    documents are cut at window edges, and ``cu_seqlens`` marks the document starts so attention does not cross them
    (the role of olmo-core's packed FSL dataset in ``open_instruct/olmo_core_finetune.py:232-243``)."""

    def __init__(self, data_dir: str | os.PathLike, sequence_length: int, vocab_size: int):
        self.L = sequence_length
        d = pathlib.Path(data_dir)
        dt = select_token_dtype(vocab_size)
        self.shards = []
        for p in sorted(d.glob(TOKEN_IDS_NPY_GLOB)):
            n = p.stat().st_size // np.dtype(dt).itemsize
            toks = np.memmap(p, mode="r", dtype=dt, shape=(n,))
            mask = np.memmap(p.with_name(p.name.replace("token_ids", "labels_mask")), mode="r", dtype=np.bool_, shape=(n,))
            with gzip.open(d / (p.stem + ".csv.gz"), "rt") as f:
                starts = np.array([int(line.split(",")[0]) for line in f if line.strip()], dtype=np.int64)
            self.shards.append((toks, mask, starts, n // self.L))
        self.offsets = np.cumsum([0] + [s[3] for s in self.shards])

    def __len__(self) -> int:
        return int(self.offsets[-1])

    def __getitem__(self, i: int) -> PackedWindow:
        if not 0 <= i < len(self):
            raise IndexError(i)
        s = int(np.searchsorted(self.offsets, i, side="right") - 1)
        toks, mask, starts, _ = self.shards[s]
        lo = (i - int(self.offsets[s])) * self.L
        hi = lo + self.L
        inner = starts[(starts > lo) & (starts < hi)] - lo
        cu = np.concatenate([[0], inner, [self.L]]).astype(np.int32)
        return PackedWindow(np.asarray(toks[lo:hi]).astype(np.int64), np.asarray(mask[lo:hi]), cu)
