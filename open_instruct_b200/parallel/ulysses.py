"""Sequence parallelism (Ulysses): batch splitting on the host, and the head <-> sequence exchange plan.

``UlyssesSPSplitter.split_collated_batch`` gives every rank of a sequence-parallel group its contiguous chunk of each
micro-batch tensor: all ranks agree on the longest row through one ``all_gather`` of lengths, pad to a multiple of the
group size (token pad id for ids, the invalid-logprob marker for rollout log-probs, 0 elsewhere) and slice
(``open_instruct/utils.py:2713-2761``).

``ExchangePlan`` describes, for a fused ``[q | k | v]`` projection, which rank owns which 128-wide head column after
the sequence -> head exchange; the column-scatter GEMM epilogue and the row-scatter exchange kernel both read it.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..utils.common import INVALID_LOGPROB


@dataclass
class UlyssesSPSplitter:
    sp_rank: int
    sp_group: object
    sp_world_size: int
    device: torch.device
    pad_token_id: int

    def split_collated_batch(self, data):
        local = torch.tensor([max(t.shape[-1] for t in data.query_responses)], dtype=torch.int64, device=self.device)
        if self.sp_world_size > 1 and dist.is_initialized():
            lens = [torch.zeros_like(local) for _ in range(self.sp_world_size)]
            dist.all_gather(lens, local, group=self.sp_group)
            longest = max(int(x.item()) for x in lens)
        else:
            longest = int(local.item())
        n = self.sp_world_size
        longest = -(-longest // n) * n
        chunk = longest // n
        lo, hi = chunk * self.sp_rank, chunk * (self.sp_rank + 1)
        out = {}
        for f in dataclasses.fields(data):
            col = getattr(data, f.name)
            if col is None or f.name == "cu_seqlens":
                out[f.name] = None  # document boundaries are rebuilt per chunk by the consumer
                continue
            fill = self.pad_token_id if f.name == "query_responses" else (INVALID_LOGPROB if f.name == "vllm_logprobs" else 0)
            out[f.name] = [F.pad(t, (0, longest - t.shape[-1]), value=fill)[..., lo:hi] for t in col]
        return type(data)(**out)


@dataclass
class ExchangePlan:
    """Head ownership for sequence parallel degree ``sp``: rank ``r`` holds query heads ``[r*Hq/sp, (r+1)*Hq/sp)`` and
    KV heads ``[r*Hkv/sp, (r+1)*Hkv/sp)``; its local fused row is ``[q_local | k_local | v_local]``."""

    sp: int
    num_heads: int
    num_kv_heads: int
    head_dim: int = 128

    def __post_init__(self):
        if self.num_heads % self.sp or self.num_kv_heads % self.sp:
            raise ValueError(f"heads ({self.num_heads}/{self.num_kv_heads}) must be divisible by the sequence-parallel size {self.sp}")

    @property
    def local_cols(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) // self.sp * self.head_dim

    def column_map(self) -> tuple[torch.Tensor, torch.Tensor]:
        """For every global head column block (q heads, then k, then v): (destination rank, destination column offset)."""
        hq, hk, sp, d = self.num_heads // self.sp, self.num_kv_heads // self.sp, self.sp, self.head_dim
        ranks, offs = [], []
        for h in range(self.num_heads):
            ranks.append(h // hq)
            offs.append((h % hq) * d)
        for which in range(2):
            for h in range(self.num_kv_heads):
                ranks.append(h // hk)
                offs.append((hq + which * hk + h % hk) * d)
        return torch.tensor(ranks, dtype=torch.int32), torch.tensor(offs, dtype=torch.int32)
