"""Padding-free collators: examples are concatenated into one packed row with document
boundaries, never padded to a common length.

Behaviour follows ``open_instruct/padding_free_collator.py:19-163`` (``TensorDataCollatorWithFlattening``
and its DPO variant): the first token of every document gets label -100 so that no token
predicts across a boundary, ``cu_seq_lens`` are int32 prefix sums, ``position_ids`` restart at 0
per document and ``seq_idx`` holds the document index of every token.  What differs is the
hand-off: the batch is also given in the 1-D form the packed model consumes
(``labels_shifted[t]`` = target of position ``t``), so the model never shifts or pads.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

IGNORE = -100


def shift_labels(labels: torch.Tensor) -> torch.Tensor:
    """``out[t] = labels[t + 1]`` (last position ignored).  With -100 on every document's first
    token, a global shift is exactly the per-document causal shift."""
    out = torch.full_like(labels, IGNORE)
    out[:-1] = labels[1:]
    return out


def flatten_examples(input_ids: list, labels: list | None = None, pad_to: int | None = None,
                     pad_token_id: int = 0) -> dict:
    """Concatenate token lists into one packed batch (dict of 1-D tensors + boundaries)."""
    ids, labs, pos, seq_idx, cu = [], [], [], [], [0]
    for i, x in enumerate(input_ids):
        x = torch.as_tensor(x, dtype=torch.long)
        n = x.numel()
        if n == 0:
            continue
        lab = torch.as_tensor(labels[i], dtype=torch.long).clone() if labels is not None else x.clone()
        lab[0] = IGNORE
        ids.append(x)
        labs.append(lab)
        pos.append(torch.arange(n, dtype=torch.long))
        seq_idx.append(torch.full((n,), len(cu) - 1, dtype=torch.int32))
        cu.append(cu[-1] + n)
    if not ids:
        raise ValueError("empty batch")
    ids_t, labs_t, pos_t, idx_t = torch.cat(ids), torch.cat(labs), torch.cat(pos), torch.cat(seq_idx)
    max_len = max(b - a for a, b in zip(cu[:-1], cu[1:]))
    if pad_to is not None and ids_t.numel() < pad_to:
        # padding becomes one extra, fully masked document so attention never mixes it in
        n = pad_to - ids_t.numel()
        ids_t = torch.cat([ids_t, torch.full((n,), pad_token_id, dtype=torch.long)])
        labs_t = torch.cat([labs_t, torch.full((n,), IGNORE, dtype=torch.long)])
        pos_t = torch.cat([pos_t, torch.arange(n, dtype=torch.long)])
        idx_t = torch.cat([idx_t, torch.full((n,), len(cu) - 1, dtype=torch.int32)])
        cu.append(cu[-1] + n)
        max_len = max(max_len, n)
    cu_t = torch.tensor(cu, dtype=torch.int32)
    return {
        "input_ids": ids_t,
        "labels": labs_t,
        "labels_shifted": shift_labels(labs_t),
        "position_ids": pos_t,
        "seq_idx": idx_t,
        "cu_seq_lens_q": cu_t,
        "cu_seq_lens_k": cu_t,
        "max_length_q": max_len,
        "max_length_k": max_len,
    }


@dataclass
class TensorDataCollatorWithFlattening:
    """SFT collator.  ``features``: dicts with ``input_ids`` and optional ``labels``.

    ``max_seq_length`` pads the packed row up to a fixed length (one extra masked document).
    ``return_batch_dim`` adds the leading batch dimension of 1 that the reference emits.
    """

    return_position_ids: bool = True
    return_seq_idx: bool = True
    max_seq_length: int | None = None
    pad_token_id: int = 0
    return_batch_dim: bool = False
    native: bool = False  # pack with the C++ host runtime (``data/native_pack.py``) when no padding is requested

    def __call__(self, features: list[dict]) -> dict:
        has_labels = "labels" in features[0]
        batch = None
        if self.native and self.max_seq_length is None and all(len(f["input_ids"]) > 0 for f in features):
            from . import native_pack

            if native_pack.available():
                batch = native_pack.pack_examples([f["input_ids"] for f in features], [f["labels"] for f in features] if has_labels else None,
                                                  budget=1 << 30)[0]
                lens = (batch["cu_seq_lens_q"][1:] - batch["cu_seq_lens_q"][:-1]).long()
                batch["seq_idx"] = torch.repeat_interleave(torch.arange(lens.numel(), dtype=torch.int32), lens)
        if batch is None:
            batch = flatten_examples([f["input_ids"] for f in features],
                                     [f["labels"] for f in features] if has_labels else None,
                                     pad_to=self.max_seq_length, pad_token_id=self.pad_token_id)
        if "index" in features[0]:
            batch["index"] = torch.tensor([int(f["index"]) for f in features], dtype=torch.long)
        if not self.return_position_ids:
            batch.pop("position_ids")
        if not self.return_seq_idx:
            batch.pop("seq_idx")
        if self.return_batch_dim:
            for k in ("input_ids", "labels", "labels_shifted", "position_ids", "seq_idx"):
                if k in batch:
                    batch[k] = batch[k].unsqueeze(0)
        return batch


@dataclass
class TensorDataCollatorWithFlatteningDPO:
    """Preference collator: chosen and rejected sides flattened separately, keys prefixed
    ``chosen_`` / ``rejected_`` (``open_instruct/padding_free_collator.py:145-163``)."""

    max_seq_length: int | None = None
    pad_token_id: int = 0

    def __call__(self, features: list[dict]) -> dict:
        out = {}
        for side in ("chosen", "rejected"):
            b = flatten_examples([f[f"{side}_input_ids"] for f in features], [f[f"{side}_labels"] for f in features],
                                 pad_to=self.max_seq_length, pad_token_id=self.pad_token_id)
            for k, v in b.items():
                out[f"{side}_{k}"] = v
        if "index" in features[0]:
            out["index"] = torch.tensor([int(f["index"]) for f in features], dtype=torch.long)
        return out


def concatenated_inputs(batch: dict) -> tuple[dict, int]:
    """Chosen‖rejected along the sequence axis with offset boundaries
    (``open_instruct/padding_free_collator.py:166-199``).  Returns (packed batch, number of chosen docs)."""
    c_cu, r_cu = batch["chosen_cu_seq_lens_q"], batch["rejected_cu_seq_lens_q"]
    n_chosen = c_cu.numel() - 1
    cu = torch.cat([c_cu, r_cu[1:] + c_cu[-1]])
    cat = lambda k: torch.cat([batch[f"chosen_{k}"], batch[f"rejected_{k}"]])
    labels = cat("labels")
    return {
        "input_ids": cat("input_ids"),
        "labels": labels,
        "labels_shifted": shift_labels(labels),
        "position_ids": cat("position_ids"),
        "cu_seq_lens_q": cu,
        "cu_seq_lens_k": cu,
        "seq_idx": torch.cat([batch["chosen_seq_idx"], batch["rejected_seq_idx"] + n_chosen]),
    }, n_chosen


def get_batch_logps(per_token_logps: torch.Tensor, labels_shifted: torch.Tensor, cu_seq_lens: torch.Tensor,
                    average_log_prob: bool = False) -> torch.Tensor:
    """Per-document sum (or mean) of token log-probs over positions whose target is not -100
    (``open_instruct/padding_free_collator.py:202-229``): a segment reduction, no Python loop."""
    mask = (labels_shifted != IGNORE).to(per_token_logps.dtype)
    n_docs = cu_seq_lens.numel() - 1
    T = per_token_logps.numel()
    seg = torch.bucketize(torch.arange(T, device=per_token_logps.device), cu_seq_lens[1:].to(torch.long), right=True)
    seg = seg.clamp(max=n_docs - 1)
    sums = torch.zeros(n_docs, dtype=per_token_logps.dtype, device=per_token_logps.device).scatter_add_(0, seg, per_token_logps * mask)
    if not average_log_prob:
        return sums
    counts = torch.zeros_like(sums).scatter_add_(0, seg, mask)
    return sums / counts.clamp(min=1)


def count_features_within_token_budget(lengths: list[int], budget: int) -> int:
    """How many leading examples fit into ``budget`` tokens (at least one)
    (``open_instruct/padding_free_collator.py:123-142``)."""
    total, n = 0, 0
    for ln in lengths:
        if n > 0 and total + ln > budget:
            break
        total += ln
        n += 1
    return max(n, 1)


def to_device(batch: dict, device, non_blocking: bool = True) -> dict:
    return {k: (v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v) for k, v in batch.items()}


def pin(batch: dict) -> dict:
    if not torch.cuda.is_available():
        return batch
    return {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in batch.items()}
