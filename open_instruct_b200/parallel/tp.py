"""Tensor parallelism for the rollout engine: weight sharding and the fused all-reduce + residual + RMSNorm.

Megatron-style split of a decoder layer over ``tp`` GPUs (what vLLM does for ``--vllm_tensor_parallel_size``,
``open_instruct/vllm_utils.py:1234-1270``): q/k/v and gate/up are column-parallel (each rank keeps ``heads / tp``
heads and ``intermediate / tp`` channels), o_proj and down_proj are row-parallel, so each of the two produces a
partial ``[T, hidden]`` that must be summed over ranks.  Embedding, norms and lm_head are replicated.  Because a
rank's shard is itself a valid model layout with fewer heads and a narrower MLP, the engine runs its ordinary layer
stack on ``local_spec`` and only swaps the "add residual + norm" step for ``TPContext.reduce_norm``, which sums the
partials out of the peers' symmetric buffers inside the same kernel (``ops/csrc/tp_comm.cu``).

All ranks of a TP group run the same schedule on the same requests (SPMD): the reduced activations are bitwise
identical on every rank, and so are the sampled tokens.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..models.spec import ModelSpec, ParamLayout
from ..ops import lib
from ..ops.lib import ptr, status_word, stream_ptr
from .symm import _ptr_array

_P, _I, _F, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_uint
_PP = ctypes.POINTER(ctypes.c_void_p)
lib._SIGNATURES["b200_tp_allreduce_norm"] = [_PP, _PP, _I, _I, _U, _P, _P, _P, _P, _I, _I, _F, _I, _P, _P]


def local_spec(spec: ModelSpec, tp: int) -> ModelSpec:
    if spec.num_heads % tp or spec.num_kv_heads % tp or spec.intermediate_size % tp:
        raise ValueError(f"heads {spec.num_heads}/{spec.num_kv_heads} and intermediate size {spec.intermediate_size} must divide by tp={tp}")
    return spec.replace(num_heads=spec.num_heads // tp, num_kv_heads=spec.num_kv_heads // tp, intermediate_size=spec.intermediate_size // tp)


@torch.no_grad()
def shard_flat(full_flat: torch.Tensor, spec: ModelSpec, rank: int, tp: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """This rank's shard of a full flat parameter buffer, laid out as ``ParamLayout(local_spec(spec, tp))``."""
    ls = local_spec(spec, tp)
    full, loc = ParamLayout(spec), ParamLayout(ls)
    if out is None:
        out = torch.empty(loc.total, dtype=full_flat.dtype, device=full_flat.device)
    fv, lv = full.views(full_flat), loc.views(out)
    hq, hk, f, d = ls.num_heads * ls.head_dim, ls.num_kv_heads * ls.head_dim, ls.intermediate_size, spec.head_dim
    for name, dst in lv.items():
        src = fv[name]
        leaf = name.split(".", 1)[-1]
        if leaf in ("wqkv", "bqkv"):
            q0, k0, v0 = 0, spec.q_dim, spec.q_dim + spec.kv_dim
            dst.copy_(torch.cat([src[q0 + rank * hq: q0 + (rank + 1) * hq], src[k0 + rank * hk: k0 + (rank + 1) * hk],
                                 src[v0 + rank * hk: v0 + (rank + 1) * hk]], 0))
        elif leaf == "wo":
            dst.copy_(src[:, rank * hq:(rank + 1) * hq])
        elif leaf == "w_gate_up":
            F = spec.intermediate_size
            dst.copy_(torch.cat([src[rank * f:(rank + 1) * f], src[F + rank * f: F + (rank + 1) * f]], 0))
        elif leaf == "w_down":
            dst.copy_(src[:, rank * f:(rank + 1) * f])
        else:
            dst.copy_(src)
    return out


@torch.no_grad()
def unshard_flat(shards: list[torch.Tensor], spec: ModelSpec, out: torch.Tensor | None = None) -> torch.Tensor:
    """Inverse of ``shard_flat``: the full flat buffer from the ``tp`` rank shards (replicated entries come from shard 0)."""
    tp = len(shards)
    ls = local_spec(spec, tp)
    full, loc = ParamLayout(spec), ParamLayout(ls)
    if out is None:
        out = torch.zeros(full.total, dtype=shards[0].dtype, device=shards[0].device)
    fv = full.views(out)
    lvs = [loc.views(s) for s in shards]
    hq, hk, f = ls.num_heads * ls.head_dim, ls.num_kv_heads * ls.head_dim, ls.intermediate_size
    for name, dst in fv.items():
        leaf = name.split(".", 1)[-1]
        parts = [lv[name] for lv in lvs]
        if leaf in ("wqkv", "bqkv"):
            dst.copy_(torch.cat([p[:hq] for p in parts] + [p[hq:hq + hk] for p in parts] + [p[hq + hk:] for p in parts], 0))
        elif leaf in ("wo", "w_down"):
            dst.copy_(torch.cat(parts, 1))
        elif leaf == "w_gate_up":
            dst.copy_(torch.cat([p[:f] for p in parts] + [p[f:] for p in parts], 0))
        else:
            dst.copy_(parts[0])
    return out


class _SumOverTP(torch.autograd.Function):
    """Forward: sum of the ranks' partial outputs (after a row-parallel projection).  Backward: identity - the upstream
    gradient is the same on every rank."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """Forward: identity (a replicated activation enters a column-parallel projection).  Backward: the ranks' partial input
    gradients are summed."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class TrainTP:
    """Tensor parallelism of the TRAINING engine (what olmo-core's ``tensor_parallel_degree`` gives the reference's DPO
    trainer, ``open_instruct/dpo_utils.py:129-130``, ``open_instruct/dpo.py:295-299``).  The model runs ``local_spec`` on this
    rank's shard; the two row-parallel outputs of a layer are summed over the group in the forward, the two
    column-parallel input gradients in the backward.  Replicated parameters (embedding, norms, output head) see
    identical inputs and gradients on every rank; two exceptions are summed at the optimizer step (``sync_replicated_grads``):
    the q/k norm weights, whose gradient is a sum over heads, and the untied output head, whose log-prob computation is split
    over the vocabulary (``vocab_parallel``) so that every rank produces the gradient of its own rows."""

    def __init__(self, group, vocab_parallel: bool = True):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        # the output head's vocabulary is split over the group for the log-prob computation: every rank multiplies the hidden
        # states with ITS rows of the (replicated) head and the ranks exchange [T]-sized partial results, so no rank holds
        # [T, V] logits (what the reference's ``DPOLMHead`` does on its local vocabulary shard,
        # ``open_instruct/olmo_core_train_modules.py:39-85``)
        self.vocab_parallel = vocab_parallel

    def vocab_range(self, vocab: int) -> tuple[int, int]:
        """Rows of the output head this rank multiplies with (multiples of 8 rows, the last shard takes what is left)."""
        per = -(-vocab // self.world)
        per = (per + 7) // 8 * 8
        lo = min(vocab, self.rank * per)
        return lo, min(vocab, lo + per)

    def combine_logprobs(self, label_logit, lse_local, mean_logit_local, labels, want_entropy: bool):
        """Global ``(logp, lse, entropy | None)`` from the ranks' shard partials ([T] fp32 each; not differentiable - the
        callers differentiate through the global lse themselves)."""
        m = lse_local.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
        w = torch.exp(lse_local - m)                       # this shard's share of the softmax mass, up to the common factor
        parts = torch.stack([w, label_logit, w * mean_logit_local])
        dist.all_reduce(parts, group=self.group)
        lse = m + torch.log(parts[0])
        valid = labels >= 0
        logp = torch.where(valid, parts[1] - lse, torch.zeros_like(lse))
        ent = torch.where(valid, lse - parts[2] / parts[0], torch.zeros_like(lse)) if want_entropy else None
        return logp, lse, ent

    def vocab_parallel_logprobs(self, logits_local, labels, v0: int, temperature: float, want_entropy: bool):
        """Autograd form (PyTorch path): per-token log-probs from this rank's logit columns ``[v0, v0 + V_local)``."""
        z = logits_local.float() / temperature
        lse_loc = torch.logsumexp(z, dim=-1)
        with torch.no_grad():
            m = lse_loc.detach().clone()
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
        s = _SumOverTP.apply(torch.exp(lse_loc - m), self.group)
        lse = m + torch.log(s)
        local = labels - v0
        inside = (local >= 0) & (local < z.shape[-1])
        zl_loc = torch.where(inside, z.gather(-1, local.clamp(0, z.shape[-1] - 1)[:, None]).squeeze(-1), torch.zeros_like(lse_loc))
        zl = _SumOverTP.apply(zl_loc, self.group)
        valid = labels >= 0
        logp = torch.where(valid, zl - lse, torch.zeros_like(lse))
        ent = None
        if want_entropy:
            with torch.no_grad():
                e = (torch.softmax(z, -1) * z).sum(-1) * torch.exp(lse_loc - lse)
                dist.all_reduce(e, group=self.group)
                ent = torch.where(valid, lse - e, torch.zeros_like(lse)).detach()
        return logp, ent

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:   # fused path: explicit, in place
        """Sum ``t`` over the tensor-parallel group, in place.  bf16 ``[tokens, hidden]`` activations on a GPU go through the
        one-shot kernel the rollout engine uses (every rank stores its partial in a symmetric buffer, exchanges one flag and
        adds all ranks' slots with 16-byte peer loads in rank order: the same bits on every rank, one kernel instead of a
        library ring) when ``B200_TP_FUSED_ALLREDUCE=1``; everything else through ``torch.distributed``.  The fused route is
        opt-in: it has not run on GPUs yet (on CPU it is never taken)."""
        ctx = self._fused_ctx(t)
        if ctx is None:
            dist.all_reduce(t, group=self.group)
            return t
        buf = ctx.out_buffer(t.shape[0])
        buf.copy_(t)
        ctx.reduce_norm(buf, None, 0.0, res=None, out=t)
        return t

    def _fused_ctx(self, t: torch.Tensor):
        """The symmetric exchange buffers for ``[<= max_tokens, t.shape[1]]`` tensors, created on first use (a collective:
        every rank reaches its first all-reduce at the same place), or None where the fused kernel does not apply."""
        import os

        if (not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or not t.is_contiguous() or self.world < 2 or self.world > 8
                or t.shape[1] % 128 or t.shape[1] > 8192 or os.environ.get("B200_TP_FUSED_ALLREDUCE", "0") != "1"):
            return None
        ctxs = self.__dict__.setdefault("_ctxs", {})
        D = t.shape[1]
        if D not in ctxs:
            max_tokens = int(os.environ.get("B200_TP_MAX_TOKENS", "16384"))
            ctxs[D] = TPContext(D, max_tokens, t.device, group=self.group)
        ctx = ctxs[D]
        return ctx if t.shape[0] <= ctx.max_tokens else None

    def sum_partials(self, x):    # autograd path
        return _SumOverTP.apply(x, self.group)

    def enter(self, x):
        return _CopyToTP.apply(x, self.group)

    def norm_weights(self, layout: ParamLayout) -> list[tuple[int, int, float]]:
        """Ranges of the local flat layout with their weight in the global gradient norm: 1 for entries split over the group,
        1 / tp for replicated ones (every rank holds the same gradient).  Adjacent entries of equal weight are merged."""
        out: list[list] = []
        for name, e in layout.entries.items():
            leaf = name.split(".", 1)[-1]
            w = 1.0 if leaf in ("wqkv", "wo", "w_gate_up", "w_down", "bqkv") else 1.0 / self.world
            if out and out[-1][2] == w:
                out[-1][1] = e.offset + e.numel
            else:
                out.append([e.offset, e.offset + e.numel, w])
        return [tuple(x) for x in out]

    def sync_replicated_grads(self, grads: dict, spec: ModelSpec) -> None:
        if spec.qk_norm:
            for name, g in grads.items():
                if name.endswith(("q_norm", "k_norm")):
                    dist.all_reduce(g, group=self.group)
        if self.vocab_parallel and "lm_head" in grads:
            # every rank produced the gradient of its own rows of the head only: the sum is the full gradient everywhere
            dist.all_reduce(grads["lm_head"], group=self.group)


class HostTPContext:
    """Tensor-parallel context of the rollout engine's PyTorch path: the row-parallel partial sums are added with a plain
    ``torch.distributed`` all-reduce (gloo on CPU, NCCL on a GPU).  It lets every host-side part of a tensor-parallel engine -
    the leader's command stream, the followers, weight updates that arrive as whole models and are re-laid out per rank - run
    as CPU processes."""

    def __init__(self, hidden: int, max_tokens: int, device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device, self.hidden, self.max_tokens = torch.device(device), hidden, max_tokens

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t


class TPContext:
    """Two symmetric ``[max_tokens, hidden]`` bf16 buffers for the row-parallel outputs + the fused reduction."""

    def __init__(self, hidden: int, max_tokens: int, device, group=None, peer_timeout_ms: int = 20000):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device, self.hidden, self.max_tokens = torch.device(device), hidden, max_tokens
        self.peer_timeout_ms = peer_timeout_ms
        # per parity: ``world`` slots of [max_tokens, hidden]; slot r holds rank r's partial.  A rank always writes its own
        # slot of its own buffer; with the fused push (large T) the GEMM epilogue also stores the tile into the same slot
        # of every peer's buffer, so that the reduction afterwards reads local memory only.
        self.bufs, self._ptrs = [], []
        self.slot = max_tokens * hidden
        for _ in range(2):
            b = symm_mem.empty(self.world * self.slot, dtype=torch.bfloat16, device=self.device)
            b.zero_()
            h = symm_mem.rendezvous(b, self.group)
            self.bufs.append(b)
            self._ptrs.append([int(p) for p in h.buffer_ptrs])
            self._pads = _ptr_array(h.signal_pad_ptrs)
            self._h = h
        self._next, self._epoch = 0, 0
        self._pushed = False
        if hidden % 128:
            raise ValueError("hidden size must be a multiple of 128")
        nblk = hidden // 128
        mine = 2 * self.rank * self.slot  # byte offset of my slot
        self._tab_local, self._tab_peer = [], []
        for par in range(2):
            self._tab_local.append(torch.tensor([self._ptrs[par][self.rank] + mine + 256 * j for j in range(nblk)], dtype=torch.int64, device=self.device))
            peer = (self.rank + 1) % self.world
            self._tab_peer.append(torch.tensor([self._ptrs[par][peer] + mine + 256 * j for j in range(nblk)], dtype=torch.int64, device=self.device))
        lib._SIGNATURES["b200_gemm2_bf16_scatter"] = [_P, _P, _I, _I, _I, ctypes.c_longlong, ctypes.c_longlong, _I, _I, _P, _I, ctypes.c_longlong, _P, _P, _P]
        fn2 = lib.load_ops().b200_gemm2_bf16_scatter
        fn2.argtypes, fn2.restype = lib._SIGNATURES["b200_gemm2_bf16_scatter"], ctypes.c_int
        fn = lib.load_ops().b200_tp_allreduce_norm
        fn.argtypes, fn.restype = lib._SIGNATURES["b200_tp_allreduce_norm"], ctypes.c_int
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def out_buffer(self, tokens: int) -> torch.Tensor:
        """The symmetric buffer the next row-parallel GEMM must write its ``[tokens, hidden]`` partial into."""
        if tokens > self.max_tokens:
            raise ValueError(f"{tokens} tokens exceed the tensor-parallel exchange buffer ({self.max_tokens})")
        a = self.rank * self.slot
        return self.bufs[self._next][a: a + tokens * self.hidden].view(tokens, self.hidden)

    def row_gemm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Row-parallel projection ``x @ w^T`` whose epilogue stores every output tile into this rank's slot of BOTH GPUs'
        exchange buffers (two ranks): the NVLink transfer of a tile overlaps the computation of the next ones, and the
        reduction that follows reads only local memory.  Returns this rank's partial (a view of the local slot)."""
        if self.world != 2:
            raise NotImplementedError("the fused push is written for two ranks")
        T, _ = x.shape
        out = self.out_buffer(T)
        par = self._next
        lib.call("b200_gemm2_bf16_scatter", ptr(x), ptr(w), T, w.shape[0], x.shape[1], x.stride(0), w.stride(0), 0, 0, ptr(self._tab_local[par]),
                 0, self.hidden, ptr(status_word(self.device)), stream_ptr(), ptr(self._tab_peer[par]))
        self._pushed = True
        return out

    def reduce_norm(self, partial: torch.Tensor, weight: torch.Tensor | None, eps: float, res: torch.Tensor | None = None,
                    out: torch.Tensor | None = None):
        """``h = res + sum_ranks partial``; ``y = rmsnorm(h) * weight``.  Returns ``(y, h)`` (``y`` is None without a weight);
        ``out`` (bf16 [T, D], contiguous) receives ``h`` instead of a fresh tensor."""
        T, D = partial.shape
        buf = self.bufs[self._next]
        if partial.data_ptr() != buf.data_ptr() + 2 * self.rank * self.slot:
            raise ValueError("the partial must live in the buffer handed out by out_buffer()")
        h = out if out is not None else torch.empty(T, D, dtype=torch.bfloat16, device=self.device)
        y = torch.empty_like(h) if weight is not None else None
        self._epoch += 1
        if self._pushed:  # every rank's partial already sits in my buffer: slot r at a local address
            srcs = [self._ptrs[self._next][self.rank] + 2 * r * self.slot for r in range(self.world)]
        else:             # read slot r out of rank r's buffer over NVLink
            srcs = [self._ptrs[self._next][r] + 2 * r * self.slot for r in range(self.world)]
        self._pushed = False
        lib.call("b200_tp_allreduce_norm", _ptr_array(srcs), self._pads, self.rank, self.world, self._epoch,
                 ptr(res) if res is not None else None, ptr(weight) if weight is not None else None, ptr(h), ptr(y) if y is not None else None,
                 T, D, eps, self.peer_timeout_ms, ptr(status_word(self.device)), stream_ptr())
        self._next ^= 1
        return y, h
