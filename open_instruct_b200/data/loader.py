"""Deterministic, resumable, rank-sharded loader over a tokenised ``datasets.Dataset``.

Semantics follow ``HFDataLoader`` in the reference (``open_instruct/data_loader.py:72-390``):
* every epoch is a ``randperm`` seeded with ``seed + epoch``; ``exclude_index`` drops rows from later epochs;
* without packing, each global batch of ``batch_size`` rows is dealt to ranks with a stride
  (rank r takes positions r, r + world, ...), so all ranks see the same number of batches;
* with packing (collator with ``max_seq_length``), rows are first packed GLOBALLY into token-budgeted
  batches (for preference data both the chosen and the rejected stream must fit) and whole packed
  batches are dealt round-robin, which again guarantees equal batch counts on all ranks; with
  ``drop_last=False`` the tail is padded by repeating the last batch and flagged ``is_padding``;
* ``state_dict`` = epoch, batches processed, excluded indices; ``prompt_id`` = ``"{epoch}_{index}"``.
"""

from __future__ import annotations

from typing import Any, Callable

import numpy as np
import torch

from .collate import to_device


class HFDataLoader:
    def __init__(self, dataset, batch_size: int, seed: int, dp_rank: int = 0, dp_world_size: int = 1,
                 collator: Callable[[list[dict]], dict] | None = None, device=None, drop_last: bool = True,
                 automatic_reshuffle: bool = False, max_seq_length: int = 1, work_dir: str | None = None):
        if "index" not in dataset.column_names:
            raise ValueError("Dataset must have an 'index' column (added by get_cached_dataset_tulu); "
                             "for a custom dataset use dataset.add_column('index', range(len(dataset))).")
        if batch_size % dp_world_size:
            raise ValueError(f"global batch size {batch_size} must be divisible by the data-parallel world size {dp_world_size}")
        self._full = dataset
        self._batch_size = batch_size
        self._per_rank = batch_size // dp_world_size
        self.seed = seed
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self._collator = collator or (lambda ex: {"examples": ex, "index": [e["index"] for e in ex]})
        self._device = device
        self._drop_last = drop_last
        self._auto = automatic_reshuffle
        self.max_seq_length = max_seq_length
        self._excluded: set[int] = set()
        self._epoch = -1
        self.batches_processed = 0
        self._overflow: list[dict] = []
        self._plan: list[list[int]] = []  # dataset row numbers per local batch
        self._num_padding = 0
        self.reshuffle(0)

    # ------------------------------------------------------------------ planning
    def _packing_budget(self) -> int | None:
        return getattr(self._collator, "max_seq_length", None)

    def reshuffle(self, epoch: int | None = None, **_: Any) -> None:
        self._epoch = self._epoch + 1 if epoch is None else epoch
        self.batches_processed = 0
        g = torch.Generator().manual_seed(self.seed + self._epoch)
        order = torch.randperm(len(self._full), generator=g).numpy()
        if self._excluded:
            idx_col = np.asarray(self._full["index"])
            order = order[~np.isin(idx_col[order], list(self._excluded))]
        budget = self._packing_budget()
        self._num_padding = 0
        if budget is None:
            n_batches = len(order) // self._batch_size
            usable = n_batches * self._batch_size
            if not self._drop_last and usable < len(order):
                pad = order[: self._batch_size - (len(order) - usable)]
                order = np.concatenate([order, pad])
                n_batches += 1
                usable = n_batches * self._batch_size
            grid = order[:usable].reshape(n_batches, self._batch_size)[:, self.dp_rank :: self.dp_world_size]
            self._plan = [row.tolist() for row in grid]
            return
        cols = self._full.column_names
        if "chosen_input_ids" in cols:
            c, r = self._full["chosen_input_ids"], self._full["rejected_input_ids"]
            lens = [(len(c[i]), len(r[i])) for i in order.tolist()]
        else:
            ids = self._full["input_ids"]
            lens = [(len(ids[i]),) for i in order.tolist()]
        batches, cur, tot = [], [], [0] * len(lens[0])
        for pos, ln in enumerate(lens):
            new = [a + b for a, b in zip(tot, ln)]
            if cur and (any(t > budget for t in new) or len(cur) >= self._per_rank):
                batches.append(cur)
                cur, tot = [pos], list(ln)
            else:
                cur.append(pos)
                tot = new
        if cur:
            batches.append(cur)
        n_real = len(batches)
        if self._drop_last:
            batches = batches[: (len(batches) // self.dp_world_size) * self.dp_world_size]
        elif len(batches) % self.dp_world_size:
            batches += [batches[-1]] * (self.dp_world_size - len(batches) % self.dp_world_size)
        mine = list(range(self.dp_rank, len(batches), self.dp_world_size))
        self._num_padding = sum(1 for gi in mine if gi >= n_real)
        self._plan = [[int(order[p]) for p in batches[gi]] for gi in mine]

    # ------------------------------------------------------------------ iteration
    @property
    def total_batches(self) -> int:
        return len(self._plan)

    def __len__(self) -> int:
        return self.total_batches

    def __iter__(self):
        n_real = len(self._plan) - self._num_padding
        while self.batches_processed < len(self._plan):
            b = self.batches_processed
            rows = [self._full[i] for i in self._plan[b]]
            for ex in rows:
                ex["prompt_id"] = f"{self._epoch}_{ex['index']}"
            batch = self._collator(rows)
            if isinstance(batch, dict):
                batch["is_padding"] = b >= n_real
                if self._device is not None:
                    batch = to_device(batch, self._device)
            self.batches_processed += 1
            yield batch
        if self._auto:
            self.reshuffle()

    def get_mock_batch(self):
        rows = [self._full[i] for i in self._plan[0]] if self._plan else [self._full[0]]
        return self._collator(rows)

    def global_num_tokens_in_batch(self, batch: dict) -> int:
        n = sum(int(v.numel()) for k, v in batch.items() if "input_ids" in k and torch.is_tensor(v))
        if n == 0:
            raise ValueError("no input_ids tensors in the batch")
        return n * self.dp_world_size

    # ------------------------------------------------------------------ state
    def exclude_index(self, index: int) -> None:
        self._excluded.add(int(index))

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "batches_processed": self.batches_processed, "excluded_indices": sorted(self._excluded)}

    def load_state_dict(self, sd: dict) -> None:
        self._excluded = set(sd.get("excluded_indices", []))
        self.reshuffle(sd["epoch"])
        self.batches_processed = sd["batches_processed"]
