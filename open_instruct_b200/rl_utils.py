"""RL-side packing, advantages (GAE) and rollout traces.

``pack_sequences`` has the contract of the reference (``open_instruct/rl_utils.py:227-375``): query+response
pairs are packed greedily, in arrival order, into rows of at most ``pack_length`` tokens (shrunk to
``total_tokens // min_num_batches`` so that every data-parallel rank gets at least one row); query
tokens carry response-mask 0, response tokens carry their 1-based sample id (0 for tool output when
``mask_tool_use``); the attention mask holds the per-row document id, position ids restart per
document, engine log-probs are NaN on query tokens, ``dones`` marks the last token of every sample.
The implementation is array-based (one pass to plan the rows, numpy fills) instead of per-token
Python loops, and additionally returns ``cu_seqlens`` per row for the packed attention kernel.
"""

from __future__ import annotations

import json
import os
import threading
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .utils.common import Timer  # noqa: F401  (re-exported: the reference exposes Timer here)


@dataclass
class PackedSequences:
    query_responses: list[torch.Tensor]
    attention_masks: list[torch.Tensor]
    response_masks: list[torch.Tensor]
    original_responses: list[list[int]]
    advantages: list[torch.Tensor] | None = None
    num_actions: list[torch.Tensor] | None = None
    position_ids: list[torch.Tensor] | None = None
    packed_seq_lens: list[torch.Tensor] | None = None
    vllm_logprobs: list[torch.Tensor] | None = None
    dones: list[torch.Tensor] | None = None
    rewards: list[torch.Tensor] | None = None
    cu_seqlens: list[torch.Tensor] | None = None


def reset_position_ids(attention_mask: torch.Tensor) -> torch.Tensor:
    """Positions restarting at 0 for every document id (> 0) of each row; id 0 (padding) gets 0."""
    out = torch.zeros_like(attention_mask, dtype=torch.long)
    for i in range(attention_mask.size(0)):
        row = attention_mask[i]
        for doc in range(1, int(row.max().item()) + 1):
            sel = row == doc
            out[i, sel] = torch.arange(int(sel.sum().item()), device=row.device)
    return out


def pack_sequences(queries: list[list[int]], responses: list[list[int]], masks: list[list[int]], pack_length: int,
                   pad_token_id: int, vllm_logprobs: list[list[float]], min_num_batches: int = 1,
                   mask_tool_use: bool = False) -> PackedSequences:
    n = len(queries)
    # pad tokens are stripped from queries as from responses (``open_instruct/rl_utils.py:294``): an already padded prompt,
    # or a tokenizer whose pad id equals eos, packs fine instead of stopping the data-preparation thread
    q_arr = [np.asarray(q, dtype=np.int64) for q in queries]
    q_arr = [q[q != pad_token_id] for q in q_arr]
    r_arr, m_arr, lp_arr = [], [], []
    for i in range(n):
        r = np.asarray(responses[i], dtype=np.int64)
        lp = np.asarray(vllm_logprobs[i], dtype=np.float32)
        if len(lp) != len(r):
            raise ValueError(f"Response {i}: logprobs length ({len(lp)}) != response length ({len(r)})")
        keep = r != pad_token_id
        r_arr.append(r[keep])
        m_arr.append(np.asarray(masks[i], dtype=np.int64)[keep])
        lp_arr.append(lp[keep])
    lens = np.array([len(q_arr[i]) + len(r_arr[i]) for i in range(n)], dtype=np.int64)
    total = int(lens.sum())
    eff = min(total // min_num_batches, pack_length) if (total > 0 and min_num_batches > 1) else pack_length
    # plan: greedy first-fit in arrival order
    rows: list[list[int]] = []
    cur, used = [], 0
    for i in range(n):
        if cur and used + lens[i] > eff:
            rows.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += int(lens[i])
    if cur:
        rows.append(cur)
    out = PackedSequences([], [], [], original_responses=responses, num_actions=[], position_ids=[], packed_seq_lens=[],
                          vllm_logprobs=[], dones=[], cu_seqlens=[])
    for members in rows:
        T = int(lens[members].sum())
        qr = np.empty(T, dtype=np.int64)
        rmask = np.zeros(T, dtype=np.int64)
        amask = np.empty(T, dtype=np.int64)
        pos = np.empty(T, dtype=np.int64)
        lps = np.full(T, np.nan, dtype=np.float32)
        dones = np.zeros(T, dtype=np.int64)
        cu = [0]
        o = 0
        for k, i in enumerate(members):
            lq, lr = len(q_arr[i]), len(r_arr[i])
            qr[o:o + lq] = q_arr[i]
            qr[o + lq:o + lq + lr] = r_arr[i]
            rmask[o + lq:o + lq + lr] = np.where(m_arr[i] != 0, i + 1, 0) if mask_tool_use else i + 1
            amask[o:o + lq + lr] = k + 1
            pos[o:o + lq + lr] = np.arange(lq + lr)
            lps[o + lq:o + lq + lr] = lp_arr[i]
            if lq + lr > 0:
                dones[o + lq + lr - 1] = i + 1
            o += lq + lr
            cu.append(o)
        out.query_responses.append(torch.from_numpy(qr))
        out.response_masks.append(torch.from_numpy(rmask))
        out.attention_masks.append(torch.from_numpy(amask))
        out.position_ids.append(torch.from_numpy(pos))
        out.vllm_logprobs.append(torch.from_numpy(lps))
        out.dones.append(torch.from_numpy(dones))
        out.num_actions.append(torch.tensor([len(r_arr[i]) for i in members]))
        out.packed_seq_lens.append(torch.tensor([int(lens[i]) for i in members]))
        out.cu_seqlens.append(torch.tensor(cu, dtype=torch.int32))
    return out


def calculate_advantages(values: np.ndarray, rewards: np.ndarray, gamma: float, lam: float):
    """Generalised advantage estimation over ``[B, T]`` arrays; returns (advantages, returns)."""
    T = values.shape[1]
    adv = np.zeros_like(rewards, dtype=np.float64)
    last = np.zeros(values.shape[0])
    for t in reversed(range(T)):
        nxt = values[:, t + 1] if t < T - 1 else 0.0
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lam * last
        adv[:, t] = last
    return adv, adv + values


def calculate_advantages_packed(values: np.ndarray, rewards: np.ndarray, gamma: float, lam: float, dones: np.ndarray,
                                response_masks: np.ndarray):
    """GAE over packed rows: the recursion is cut at sample boundaries (``dones`` > 0) and skips
    non-response tokens."""
    resp = response_masks.astype(bool)
    T = values.shape[1]
    adv = np.zeros_like(rewards, dtype=np.float64)
    last = np.zeros(values.shape[0])
    nxt = np.zeros(values.shape[0])
    for t in reversed(range(T)):
        nonterminal = (dones[:, t] == 0).astype(np.float64)
        nv = nxt * nonterminal
        last_t = last * nonterminal
        delta = rewards[:, t] + gamma * nv - values[:, t]
        cand = delta + gamma * lam * last_t
        last = np.where(resp[:, t], cand, last_t)
        nxt = np.where(resp[:, t], values[:, t], nv)
        adv[:, t] = np.where(resp[:, t], cand, 0.0)
    return adv, adv + values


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis: int | None = None, denominator: float | None = None):
    from .grpo_utils import masked_mean as _mm

    return _mm(values, mask, axis, denominator)


# ---------------------------------------------------------------------------------- rollout traces
class RolloutTraceWriter:
    """Sharded JSONL dump of rollouts (prompt, response, reward, finish reason) for offline inspection."""

    def __init__(self, out_dir: str, shard_size: int = 10000):
        self.dir, self.shard_size = out_dir, shard_size
        os.makedirs(out_dir, exist_ok=True)
        self._lock = threading.Lock()
        self._n, self._shard, self._fh = 0, 0, None

    def write(self, records: list[dict]) -> None:
        with self._lock:
            for rec in records:
                if self._fh is None or self._n >= self.shard_size:
                    if self._fh is not None:
                        self._fh.close()
                        self._shard += 1
                    self._fh = open(os.path.join(self.dir, f"rollouts_{self._shard:05d}.jsonl"), "a")
                    self._n = 0
                rec = {"time": time.time(), **rec}
                self._fh.write(json.dumps(rec, default=str) + "\n")
                self._n += 1
            if self._fh is not None:
                self._fh.flush()

    def close(self) -> None:
        with self._lock:
            if self._fh is not None:
                self._fh.close()
                self._fh = None
