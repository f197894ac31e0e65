"""Packing of tokenised examples into padding-free rows by the C++ host runtime (``ops/csrc/host/host_runtime.cpp``).

``pack_plan`` assigns consecutive examples to rows under a token budget; ``pack_row`` copies one row's examples into
(pinned) output buffers and writes labels with the first token of every document masked, shifted labels, per-document
position ids and ``cu_seqlens`` in one pass - the work of the Python loops in ``data/collate.py:flatten_examples`` (and of
the reference's ``padding_free_collator.py:36-47`` / ``rl_utils.py:289-353``) without per-example tensor objects.
Falls back to the Python collator when the host library is not built.
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from ..ops import lib
from .collate import flatten_examples

_h = None


def _host():
    global _h
    if _h is None:
        h = lib.load_host()
        i32, p = ctypes.c_int, ctypes.c_void_p
        h.b200_pack_plan.argtypes = [p, i32, i32, i32, p]
        h.b200_pack_plan.restype = i32
        h.b200_pack_row.argtypes = [p, p, p, i32, i32, p, p, p, p, p]
        h.b200_pack_row.restype = i32
        _h = h
    return _h


def available() -> bool:
    try:
        _host()
        return True
    except Exception:  # noqa: BLE001
        return False


def pack_plan(lengths: list[int], budget: int, max_per_row: int = 0) -> list[int]:
    """Row index of every example (greedy, in order)."""
    lens = np.asarray(lengths, dtype=np.int32)
    out = np.empty(len(lens), dtype=np.int32)
    _host().b200_pack_plan(lens.ctypes.data, len(lens), budget, max_per_row, out.ctypes.data)
    return out.tolist()


def pack_examples(input_ids: list, labels: list | None, budget: int, max_per_row: int = 0, pin: bool = False) -> list[dict]:
    """Packed rows (same keys as ``flatten_examples``) for a list of tokenised examples."""
    if not available():
        rows, cur, used = [], [], 0
        for i, x in enumerate(input_ids):
            if cur and (used + len(x) > budget or (max_per_row and len(cur) >= max_per_row)):
                rows.append(cur)
                cur, used = [], 0
            cur.append(i)
            used += len(x)
        if cur:
            rows.append(cur)
        return [flatten_examples([input_ids[i] for i in r], [labels[i] for i in r] if labels is not None else None) for r in rows]
    h = _host()
    lens = [len(x) for x in input_ids]
    starts = np.zeros(len(lens) + 1, dtype=np.int64)
    np.cumsum(lens, out=starts[1:])
    tokens = np.concatenate([np.asarray(x, dtype=np.int64) for x in input_ids]) if lens else np.zeros(0, np.int64)
    labs = np.concatenate([np.asarray(x, dtype=np.int64) for x in labels]) if labels is not None else None
    row_of = pack_plan(lens, budget, max_per_row)
    out = []
    first = 0
    pin = pin and torch.cuda.is_available()
    while first < len(lens):
        last = first
        while last < len(lens) and row_of[last] == row_of[first]:
            last += 1
        n = int(starts[last] - starts[first])
        mk = lambda dt: torch.empty(n, dtype=dt, pin_memory=pin)
        ids_t, lab_t, sh_t, pos_t = mk(torch.int64), mk(torch.int64), mk(torch.int64), mk(torch.int64)
        cu_t = torch.empty(last - first + 1, dtype=torch.int32, pin_memory=pin)
        h.b200_pack_row(tokens.ctypes.data, labs.ctypes.data if labs is not None else None, starts.ctypes.data, first, last, ids_t.data_ptr(),
                        lab_t.data_ptr(), sh_t.data_ptr(), pos_t.data_ptr(), cu_t.data_ptr())
        mx = int((cu_t[1:] - cu_t[:-1]).max()) if last > first else 0
        out.append({"input_ids": ids_t, "labels": lab_t, "labels_shifted": sh_t, "position_ids": pos_t, "cu_seq_lens_q": cu_t, "cu_seq_lens_k": cu_t,
                    "max_length_q": mx, "max_length_k": mx})
        first = last
    return out
