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


class UlyssesContext:
    """Symmetric buffers, destination tables and the four exchanges of one sequence-parallel group.

    Per decoder layer, with ``T`` tokens in the packed batch and ``T_l = T / sp`` of them on this rank:

    ==========  =======================================  ==============================================
    direction   what moves                               how
    ==========  =======================================  ==============================================
    forward     q/k/v of my tokens -> head owners        column-scatter epilogue of the QKV GEMM
    forward     attention output -> token owners         ``a2a_heads`` kernel (peer stores)
    backward    d(attention output) -> head owners       column-scatter epilogue of the o_proj dgrad GEMM
    backward    dq/dk/dv -> token owners                 ``a2a_heads`` kernel
    ==========  =======================================  ==============================================

    Each exchange ends with a device-side barrier on the launching stream (bounded wait, status word on timeout).
    ``qkv`` and the received attention output are kept per layer (the backward pass reads them in place).
    (The reference gets the same data movement from DeepSpeed's ``UlyssesSPAttentionHF`` all-to-alls,
    ``open_instruct/finetune.py:379-394``.)
    """

    def __init__(self, spec, max_tokens: int, device, group=None, peer_timeout_ms: int = 20000):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import lib
        from .symm import _ptr_array

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.sp = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.plan = ExchangePlan(self.sp, spec.num_heads, spec.num_kv_heads, spec.head_dim)
        if spec.head_dim != 128:
            raise ValueError("the exchange kernels move 128-wide head blocks")
        if max_tokens % self.sp:
            raise ValueError("max_tokens must divide by the sequence-parallel size")
        self.spec, self.device, self.max_tokens = spec, torch.device(device), max_tokens
        self.peer_timeout_ms = peer_timeout_ms
        sp, L, d = self.sp, spec.num_layers, spec.head_dim
        self.hq_l, self.hk_l = spec.num_heads // sp, spec.num_kv_heads // sp
        self.cols_l, self.q_l = self.plan.local_cols, self.hq_l * d
        self.t_l_max = max_tokens // sp
        sizes = {"qkv": L * max_tokens * self.cols_l, "attn_recv": L * self.t_l_max * spec.q_dim,
                 "d_attn": max_tokens * self.q_l, "dqkv_recv": self.t_l_max * spec.qkv_dim}
        self.off, n = {}, 0
        for k, v in sizes.items():
            self.off[k] = n
            n += (v + 127) // 128 * 128
        self.buf = symm_mem.empty(n, dtype=torch.bfloat16, device=self.device)
        self.buf.zero_()
        h = symm_mem.rendezvous(self.buf, self.group)
        self._h = h
        self.ptrs = [int(p) for p in h.buffer_ptrs]
        self._pads = _ptr_array(h.signal_pad_ptrs)
        self._epoch = 0
        # destination tables
        ranks, offs = self.plan.column_map()
        per_layer = max_tokens * self.cols_l
        tab = [[self.ptrs[int(r)] + 2 * (self.off["qkv"] + i * per_layer + int(o)) for r, o in zip(ranks, offs)] for i in range(L)]
        self.qkv_table = torch.tensor(tab, dtype=torch.int64, device=self.device)
        self.d_attn_table = torch.tensor([self.ptrs[hd // self.hq_l] + 2 * (self.off["d_attn"] + (hd % self.hq_l) * d)
                                          for hd in range(spec.num_heads)], dtype=torch.int64, device=self.device)
        self.attn_cols = torch.tensor([self.rank * self.q_l + b * d for b in range(self.hq_l)], dtype=torch.int32, device=self.device)
        q0, k0, v0 = 0, spec.q_dim, spec.q_dim + spec.kv_dim
        cols = [q0 + (self.rank * self.hq_l + b) * d for b in range(self.hq_l)]
        cols += [k0 + (self.rank * self.hk_l + b) * d for b in range(self.hk_l)]
        cols += [v0 + (self.rank * self.hk_l + b) * d for b in range(self.hk_l)]
        self.dqkv_cols = torch.tensor(cols, dtype=torch.int32, device=self.device)
        # full-width column index of every element of a local [q | k | v] row (for per-column parameters such as the bias)
        self.local_cols_index = (self.dqkv_cols.long()[:, None] + torch.arange(d, device=self.device)[None, :]).reshape(-1)
        _P, _I, _L, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
        _PP = ctypes.POINTER(ctypes.c_void_p)
        lib._SIGNATURES.update({
            "b200_gemm2_bf16_scatter": [_P, _P, _I, _I, _I, _L, _L, _I, _I, _P, _I, _L, _P, _P, _P],
            "b200_a2a_heads": [_P, _L, _PP, _I, _L, _P, _I, _I, _I, _P],
            "b200_symm_barrier": [_PP, _I, _I, _U, _I, _P, _P],
        })
        so = lib.load_ops()
        for name in ("b200_gemm2_bf16_scatter", "b200_a2a_heads", "b200_symm_barrier"):
            fn = getattr(so, name)
            fn.argtypes, fn.restype = lib._SIGNATURES[name], ctypes.c_int
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------ helpers
    def _view(self, region: str, offset: int, rows: int, cols: int) -> torch.Tensor:
        a = self.off[region] + offset
        return self.buf[a:a + rows * cols].view(rows, cols)

    def _region_ptrs(self, region: str, offset: int = 0):
        from .symm import _ptr_array

        return _ptr_array([p + 2 * (self.off[region] + offset) for p in self.ptrs])

    def barrier(self) -> None:
        from ..ops import lib
        from ..ops.lib import ptr, status_word, stream_ptr

        self._epoch += 1
        lib.call("b200_symm_barrier", self._pads, self.rank, self.sp, self._epoch, self.peer_timeout_ms, ptr(status_word(self.device)),
                 stream_ptr())

    def local_tokens(self, T: int) -> tuple[int, int]:
        if T % self.sp or T > self.max_tokens:
            raise ValueError(f"{T} tokens: need a multiple of {self.sp} and at most {self.max_tokens}")
        t_l = T // self.sp
        return self.rank * t_l, (self.rank + 1) * t_l

    def _gemm_scatter(self, a: torch.Tensor, b: torch.Tensor, b_mn: bool, table: torch.Tensor, row_off: int, ld_dst: int) -> None:
        from ..ops import lib
        from ..ops.lib import ptr, status_word, stream_ptr

        M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        lib.call("b200_gemm2_bf16_scatter", ptr(a), ptr(b), M, N, K, a.stride(0), b.stride(0), 0, int(b_mn), ptr(table), row_off, ld_dst,
                 ptr(status_word(self.device)), stream_ptr(), None)

    def _a2a(self, src: torch.Tensor, region: str, offset: int, ld_dst: int, cols: torch.Tensor, T: int) -> None:
        from ..ops import lib
        from ..ops.lib import ptr, stream_ptr

        lib.call("b200_a2a_heads", ptr(src), src.stride(0), self._region_ptrs(region, offset), self.sp, ld_dst, ptr(cols), T, T // self.sp,
                 cols.numel(), stream_ptr())

    # ------------------------------------------------------------------ the four exchanges
    def qkv_project(self, layer: int, n1_local: torch.Tensor, wqkv: torch.Tensor, T: int) -> torch.Tensor:
        """QKV projection of my tokens, scattered to the head owners; returns my heads for all ``T`` tokens."""
        lo, _ = self.local_tokens(T)
        self._gemm_scatter(n1_local, wqkv, False, self.qkv_table[layer], lo, self.cols_l)
        self.barrier()
        return self._view("qkv", layer * self.max_tokens * self.cols_l, T, self.cols_l)

    def attn_exchange(self, layer: int, attn_full: torch.Tensor) -> torch.Tensor:
        """Attention output [T, my heads] -> [my tokens, all heads]."""
        T = attn_full.shape[0]
        off = layer * self.t_l_max * self.spec.q_dim
        self._a2a(attn_full, "attn_recv", off, self.spec.q_dim, self.attn_cols, T)
        self.barrier()
        return self._view("attn_recv", off, T // self.sp, self.spec.q_dim)

    def d_attn_project(self, d_mid_local: torch.Tensor, wo: torch.Tensor, T: int) -> torch.Tensor:
        """d(attention output) = d_mid @ wo for my tokens, scattered to the head owners; returns [T, my heads]."""
        lo, _ = self.local_tokens(T)
        self._gemm_scatter(d_mid_local, wo, True, self.d_attn_table, lo, self.q_l)
        self.barrier()
        return self._view("d_attn", 0, T, self.q_l)

    def dqkv_exchange(self, dqkv_full: torch.Tensor) -> torch.Tensor:
        """dq/dk/dv [T, my heads] -> [my tokens, fused qkv width]."""
        T = dqkv_full.shape[0]
        self._a2a(dqkv_full, "dqkv_recv", 0, self.spec.qkv_dim, self.dqkv_cols, T)
        self.barrier()
        return self._view("dqkv_recv", 0, T // self.sp, self.spec.qkv_dim)


class HostUlyssesContext:
    """The four exchanges of ``UlyssesContext`` with plain ``torch.distributed`` all-gathers (gloo on CPU): every rank gathers
    the ranks' pieces and keeps what it owns.  Nothing here is fast; it gives the sequence-parallel branches of the model's
    hand-driven forward / backward (``ops="emulated"``) the same interface and results, so they run as CPU processes."""

    def __init__(self, spec, max_tokens: int, device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.sp = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.plan = ExchangePlan(self.sp, spec.num_heads, spec.num_kv_heads, spec.head_dim)
        if max_tokens % self.sp:
            raise ValueError("max_tokens must divide by the sequence-parallel size")
        self.spec, self.device, self.max_tokens = spec, torch.device(device), max_tokens
        d = spec.head_dim
        self.hq_l, self.hk_l = spec.num_heads // self.sp, spec.num_kv_heads // self.sp
        self.cols_l, self.q_l = self.plan.local_cols, self.hq_l * d
        self._cols = [self._local_cols(r) for r in range(self.sp)]
        self.local_cols_index = self._cols[self.rank]

    def _local_cols(self, r: int) -> torch.Tensor:
        """Full-width column index of every element of rank ``r``'s local [q | k | v] row."""
        s, d = self.spec, self.spec.head_dim
        k0, v0 = s.q_dim, s.q_dim + s.kv_dim
        blocks = [(r * self.hq_l + b) * d for b in range(self.hq_l)]
        blocks += [k0 + (r * self.hk_l + b) * d for b in range(self.hk_l)]
        blocks += [v0 + (r * self.hk_l + b) * d for b in range(self.hk_l)]
        return (torch.tensor(blocks, dtype=torch.long, device=self.device)[:, None] + torch.arange(d, device=self.device)[None, :]).reshape(-1)

    def _gather(self, t: torch.Tensor) -> list[torch.Tensor]:
        parts = [torch.empty_like(t) for _ in range(self.sp)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return parts

    def local_tokens(self, T: int) -> tuple[int, int]:
        if T % self.sp or T > self.max_tokens:
            raise ValueError(f"{T} tokens: need a multiple of {self.sp} and at most {self.max_tokens}")
        t_l = T // self.sp
        return self.rank * t_l, (self.rank + 1) * t_l

    def qkv_project(self, layer: int, n1_local: torch.Tensor, wqkv: torch.Tensor, T: int) -> torch.Tensor:
        full = torch.cat(self._gather((n1_local.float() @ wqkv.float().t()).to(n1_local.dtype)))      # [T, qkv_dim], token order
        return full[:, self.local_cols_index].contiguous()

    def attn_exchange(self, layer: int, attn_full: torch.Tensor) -> torch.Tensor:
        lo, hi = self.local_tokens(attn_full.shape[0])
        return torch.cat([p[lo:hi] for p in self._gather(attn_full)], dim=1).contiguous()          # my tokens, every rank's heads

    def d_attn_project(self, d_mid_local: torch.Tensor, wo: torch.Tensor, T: int) -> torch.Tensor:
        full = torch.cat(self._gather((d_mid_local.float() @ wo.float()).to(d_mid_local.dtype)))        # [T, q_dim]
        return full[:, self.rank * self.q_l:(self.rank + 1) * self.q_l].contiguous()

    def dqkv_exchange(self, dqkv_full: torch.Tensor) -> torch.Tensor:
        lo, hi = self.local_tokens(dqkv_full.shape[0])
        out = torch.empty(hi - lo, self.spec.qkv_dim, dtype=dqkv_full.dtype, device=dqkv_full.device)
        for r, p in enumerate(self._gather(dqkv_full)):
            out[:, self._cols[r]] = p[lo:hi]
        return out
