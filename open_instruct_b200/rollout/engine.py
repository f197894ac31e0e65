"""Rollout engine: continuous batching over a paged KV cache, in process (no HTTP hop).

Stands where the reference wraps vLLM (``open_instruct/vllm_utils.py:553-843``, ``:1188-1313``): requests
arrive as token ids with a sampling config, ``n`` samples per prompt share the prompt's KV blocks,
every generated token comes back with its log-prob under the *processed* distribution
(temperature / top-p applied - the reference asks vLLM for ``logprobs_mode="processed_logprobs"``,
``vllm_utils.py:1284``), finished requests carry finish reasons and token statistics.

Scheduling and block management are native (``ops/csrc/host/host_runtime.cpp``); the model math runs
on this package's kernels: packed varlen attention for prefill, ``b200_paged_decode`` for decode
steps, ``b200_kv_write`` to fill cache blocks, ``b200_sample`` (Philox Gumbel-max) for sampling.
``ops="ref"`` keeps everything in PyTorch (CPU-testable; same cache layout and scheduler).
"""

from __future__ import annotations

import os

import ctypes
import time
from dataclasses import dataclass, field

import torch

from ..data_types import GenerationResult, RequestInfo, SamplingConfig, TokenStatistics
from ..models import LlamaModel, ModelSpec
from ..ops import lib, ref

KV_BLOCK = 64


class _Host:
    """ctypes view of the native scheduler / block manager."""

    def __init__(self, num_blocks: int, max_running: int):
        h = lib.load_host()
        i64, i32, p = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        h.b200_engine_create.restype = p
        h.b200_engine_create.argtypes = [i32, i32, i32]
        h.b200_engine_destroy.argtypes = [p]
        h.b200_engine_add.argtypes = [p, i64, i64, i32, i32]
        h.b200_engine_finish.argtypes = [p, i64]
        h.b200_engine_advance.argtypes = [p, i64, i32]
        h.b200_engine_free_blocks.argtypes = [p]
        h.b200_engine_preemptions.argtypes = [p]
        h.b200_engine_preemptions.restype = i64
        PI64, PI32 = ctypes.POINTER(i64), ctypes.POINTER(i32)
        h.b200_engine_schedule.argtypes = [p, PI64, PI32, PI64, PI32, PI64, PI32, i32]
        h.b200_engine_blocks.argtypes = [p, i64, PI32, i32, PI32]
        h.b200_engine_counts.argtypes = [p, PI32, PI32]
        h.b200_engine_enable_prefix_cache.argtypes = [p, i32]
        h.b200_engine_reset_prefix_cache.argtypes = [p]
        h.b200_engine_prefix_cache_stats.argtypes = [p, PI64]
        h.b200_engine_set_tokens.argtypes = [p, i64, PI32, i32]
        h.b200_engine_cached_tokens.argtypes = [p, i64]
        h.b200_engine_finish_tokens.argtypes = [p, i64, PI32, i32]
        h.b200_engine_pack_decode.argtypes = [p, p, i32, i32, p, p, p, p, p, i64, PI32]
        h.b200_engine_advance_many.argtypes = [p, p, i32]
        self.h = h
        self.e = h.b200_engine_create(num_blocks, KV_BLOCK, max_running)
        self.cap = max(1024, max_running * 2)
        self._pre = (i64 * self.cap)()
        self._dec = (i64 * self.cap)()
        self._pmt = (i64 * self.cap)()
        self._blk = (i32 * 65536)()

    def add(self, sid, group, prompt_len, max_len):
        rc = self.h.b200_engine_add(self.e, sid, group, prompt_len, max_len)
        if rc:
            raise ValueError(f"cannot queue sequence {sid} (code {rc}): prompt+response does not fit the KV cache")

    def schedule(self):
        a, b, c = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        self.h.b200_engine_schedule(self.e, self._pre, ctypes.byref(a), self._dec, ctypes.byref(b), self._pmt, ctypes.byref(c), self.cap)
        return list(self._pre[: a.value]), list(self._dec[: b.value]), list(self._pmt[: c.value])

    def blocks(self, sid):
        shared = ctypes.c_int(0)
        n = self.h.b200_engine_blocks(self.e, sid, self._blk, 65536, ctypes.byref(shared))
        return list(self._blk[:n]), shared.value

    def advance(self, sid, n=1):
        return self.h.b200_engine_advance(self.e, sid, n)

    def advance_many(self, sids) -> None:
        """One new token for every sequence of the int64 numpy array ``sids``."""
        if self.h.b200_engine_advance_many(self.e, sids.ctypes.data, len(sids)):
            raise KeyError("advance of an unknown sequence")

    def pack_decode(self, sids, pos, slots, ctx, ctr, bt, round_to: int = 4) -> int:
        """Fill the numpy staging arrays of one decode step natively; returns the block-table row width (-2: ``bt`` too small)."""
        w = ctypes.c_int(0)
        rc = self.h.b200_engine_pack_decode(self.e, sids.ctypes.data, len(sids), round_to, pos.ctypes.data, slots.ctypes.data, ctx.ctypes.data,
                                            ctr.ctypes.data, bt.ctypes.data, bt.size, ctypes.byref(w))
        if rc == -2:
            return -2
        if rc:
            raise KeyError("decode step names a sequence the scheduler does not hold")
        return w.value

    def finish(self, sid, tokens=None):
        """Remove a sequence; with ``tokens`` (everything it holds) its full blocks stay findable in the prefix cache."""
        if tokens is not None:
            arr = (ctypes.c_int * len(tokens))(*tokens)
            self.h.b200_engine_finish_tokens(self.e, sid, arr, len(tokens))
        else:
            self.h.b200_engine_finish(self.e, sid)

    def enable_prefix_cache(self, on: bool) -> None:
        self.h.b200_engine_enable_prefix_cache(self.e, int(on))

    def reset_prefix_cache(self) -> None:
        self.h.b200_engine_reset_prefix_cache(self.e)

    def prefix_cache_stats(self) -> dict:
        out = (ctypes.c_int64 * 4)()
        self.h.b200_engine_prefix_cache_stats(self.e, out)
        return {"block_lookups": out[0], "block_hits": out[1], "evictions": out[2], "cached_blocks": out[3]}

    def set_tokens(self, sid, tokens) -> None:
        arr = (ctypes.c_int * len(tokens))(*tokens)
        self.h.b200_engine_set_tokens(self.e, sid, arr, len(tokens))

    def cached_tokens(self, sid) -> int:
        return max(0, self.h.b200_engine_cached_tokens(self.e, sid))

    def free_blocks(self):
        return self.h.b200_engine_free_blocks(self.e)

    def counts(self):
        w, r = ctypes.c_int(0), ctypes.c_int(0)
        self.h.b200_engine_counts(self.e, ctypes.byref(w), ctypes.byref(r))
        return w.value, r.value

    def preemptions(self):
        return int(self.h.b200_engine_preemptions(self.e))

    def __del__(self):
        try:
            self.h.b200_engine_destroy(self.e)
        except Exception:  # noqa: BLE001
            pass


@dataclass
class _Sequence:
    sid: int
    request: "_Request"
    sample_idx: int
    tokens: list[int]  # prompt + generated
    prompt_len: int
    logprobs: list[float] = field(default_factory=list)
    finish_reason: str | None = None
    seed: int = 0
    last_token: int = 0


@dataclass
class _Request:
    rid: int
    prompt: list[int]
    sampling: SamplingConfig
    meta: dict
    seqs: list[_Sequence] = field(default_factory=list)
    start_time: float = 0.0
    done: int = 0


class RolloutEngine:
    """One engine = one GPU (or CPU with ``ops='ref'``) holding a bf16 copy of the weights."""

    def __init__(self, spec: ModelSpec, device="cuda", ops: str = "auto", num_blocks: int | None = None,
                 gpu_memory_utilization: float = 0.85, max_running: int = 256, max_model_len: int = 8192, seed: int = 0,
                 flat: torch.Tensor | None = None, eos_token_ids: list[int] | None = None, tokenizer=None, tp=None,
                 enable_prefix_caching: bool = False):
        # ``enable_prefix_caching``: full KV blocks outlive their request and serve later requests that start with the same
        # tokens (multi-turn conversations re-submit their history; the reference reaches this through vLLM's
        # ``enable_prefix_caching``, ``open_instruct/vllm_utils.py:1057-1070``).  Without it only the ``n`` samples of one
        # request share their prompt blocks.
        # ``tp``: a ``parallel.tp.TPContext``; ``spec`` and ``flat`` are then this rank's shard (``local_spec`` / ``shard_flat``)
        self.tp = tp
        self.spec = spec
        self.device = torch.device(device)
        if ops == "auto":
            windowed = bool(spec.min_window and max_model_len > spec.min_window)   # the paged attention kernels have no window
            ops = "fused" if (self.device.type == "cuda" and spec.head_dim == 128 and not spec.post_norm and not spec.num_experts
                              and not windowed and not spec.has_gdn and lib.available()) else "ref"
        self.ops = ops
        if ops == "fused" and spec.min_window and max_model_len > spec.min_window:
            raise NotImplementedError(f"the paged attention kernels attend to the whole context; sequences longer than the model's sliding "
                                      f"window ({spec.min_window}) need ops='ref' (or a max_model_len within the window)")
        if ops == "fused" and spec.num_experts:
            raise NotImplementedError("mixture-of-experts layers run on the engine's PyTorch path (ops='ref')")
        if spec.has_gdn and (ops != "ref" or tp is not None or enable_prefix_caching):
            raise NotImplementedError("hybrid models (gated-DeltaNet layers) are sampled on the PyTorch path (ops='ref'), one engine per "
                                      "model copy, without prefix caching: their per-sequence recurrent state lives beside the paged KV cache")
        if tp is not None and (spec.post_norm or spec.num_experts):
            raise NotImplementedError("tensor-parallel engines are built for dense pre-norm blocks (a norm or a router over all heads / "
                                      "experts does not split by rank)")
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = LlamaModel(spec, device=self.device, dtype=dtype, ops=ops, seed=seed, flat=flat)
        if ops == "ref":
            self.model.flat.requires_grad_(False)
        self.dtype = dtype
        self.max_model_len = max_model_len
        self.tokenizer = tokenizer
        self.eos = set(eos_token_ids if eos_token_ids is not None else ([spec.eos_token_id] if spec.eos_token_id is not None else []))
        per_block = 2 * spec.num_layers * spec.num_kv_heads * KV_BLOCK * spec.head_dim * (2 if dtype == torch.bfloat16 else 4)
        if num_blocks is None:
            if self.device.type == "cuda":
                free, total = torch.cuda.mem_get_info(self.device)
                num_blocks = max(16, int((free - (1 - gpu_memory_utilization) * total) // per_block))
            else:
                num_blocks = 256
        self.num_blocks = num_blocks
        shape = (spec.num_layers, num_blocks, spec.num_kv_heads, KV_BLOCK, spec.head_dim)
        self.k_cache = torch.zeros(shape, dtype=dtype, device=self.device)
        self.v_cache = torch.zeros(shape, dtype=dtype, device=self.device)
        self.host = _Host(num_blocks, max_running)
        self.prefix_caching = bool(enable_prefix_caching)
        if self.prefix_caching:
            self.host.enable_prefix_cache(True)
        self.max_running = max_running
        self._next_sid = 0
        self._next_rid = 0
        self.seqs: dict[int, _Sequence] = {}
        self.requests: dict[int, _Request] = {}
        self.base_seed = seed
        self.model_step = 0
        # host_* are wall seconds of the host phases of decode steps (packing inputs, waiting for the device, accepting tokens)
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "steps": 0, "host_pack_s": 0.0, "device_wait_s": 0.0, "host_accept_s": 0.0,
                      "host_sched_s": 0.0, "decode_steps": 0}
        self.prefill_token_budget = 16384
        self.decode_splitk = os.environ.get("B200_DECODE_SPLITK", "1") == "1"  # split-K for o_proj / down_proj at <= 256 rows
        # up to 256 rows: every projection runs on the one-wave decode GEMM (tile width and K slices chosen per weight shape)
        self.decode_gemm = os.environ.get("B200_DECODE_GEMM", "1") == "1"
        self._acc32: dict = {}
        # captured decode steps, keyed by (batch size, padded block-table width, kv splits)
        self.use_cuda_graphs = os.environ.get("B200_DECODE_GRAPHS", "1") == "1" and tp is None
        self._graphs: dict = {}
        self._graph_seen: dict = {}
        self._graph_pool = None
        # hybrid models: (convolution tail, recurrent state) of every gated-DeltaNet layer, per running sequence
        self._gdn_state: dict[int, dict[int, tuple]] = {}
        self._gdn_runs: list = []   # (first row, end row, sequence continued or None, sequences that receive the new state) of the pass in flight
        self._stages: dict = {}  # pinned staging blobs of the decode step, by batch size
        self._last_sids = None

    # ------------------------------------------------------------------ public API
    def kv_cache_max_concurrency(self, seq_len: int) -> int:
        """How many sequences of ``seq_len`` tokens fit at once (cf. ``get_kv_cache_info``, ``vllm_utils.py:826-843``)."""
        return self.num_blocks // max(1, -(-seq_len // KV_BLOCK))

    def add_request(self, prompt: list[int], sampling: SamplingConfig, **meta) -> int:
        rid = self._next_rid
        self._next_rid += 1
        if len(prompt) + sampling.max_tokens > self.max_model_len:
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({sampling.max_tokens}) exceeds max_model_len {self.max_model_len}")
        req = _Request(rid, list(prompt), sampling, meta, start_time=time.perf_counter())
        base = sampling.seed if sampling.seed is not None else self.base_seed * 1000003 + rid
        for j in range(sampling.n):
            sid = self._next_sid
            self._next_sid += 1
            seq = _Sequence(sid, req, j, list(prompt), len(prompt), seed=base + j)
            req.seqs.append(seq)
            self.seqs[sid] = seq
            self.host.add(sid, rid, len(prompt), len(prompt) + sampling.max_tokens)
            if self.prefix_caching:
                self.host.set_tokens(sid, seq.tokens)
        self.requests[rid] = req
        return rid

    def has_unfinished(self) -> bool:
        return bool(self.requests)

    def num_active(self) -> int:
        w, r = self.host.counts()
        return w + r

    def reset_prefix_cache(self) -> bool:
        """Drop KV blocks that are kept only so that a LATER request can reuse them: after a weight update they hold K/V of
        the old policy (``open_instruct/vllm_utils.py:791-793``).  Blocks of running requests stay with them."""
        self.host.reset_prefix_cache()
        return True

    def update_weights(self, flat: torch.Tensor, model_step: int | None = None) -> None:
        """Replace the weights (same flat layout) between steps; cached KV of running sequences stays."""
        with torch.no_grad():
            n = min(flat.numel(), self.model.flat.numel())  # the two buffers may be padded for different world sizes
            self.model.flat[:n].copy_(flat[:n].to(self.model.flat.dtype), non_blocking=True)
        if self.prefix_caching:
            self.host.reset_prefix_cache()
        if model_step is not None:
            self.model_step = model_step

    @torch.no_grad()
    def step(self) -> list[GenerationResult]:
        """One scheduling + model step.  Returns the requests that completed in it."""
        t0 = time.perf_counter()
        prefill_ids, decode_ids, preempted = self.host.schedule()
        self.stats["host_sched_s"] += time.perf_counter() - t0
        finished: list[GenerationResult] = []
        if decode_ids:
            self._decode([self.seqs[s] for s in decode_ids])
        if prefill_ids:
            self._prefill([self.seqs[s] for s in prefill_ids])
        self.stats["steps"] += 1
        for sid in list(decode_ids) + list(prefill_ids):
            seq = self.seqs.get(sid)
            if seq is None or seq.finish_reason is None:
                continue
            self.host.finish(sid, seq.tokens if self.prefix_caching else None)
            self._gdn_state.pop(sid, None)
            del self.seqs[sid]
            req = seq.request
            req.done += 1
            if req.done == len(req.seqs):
                finished.append(self._finalize(req))
                del self.requests[req.rid]
        return finished

    def generate(self, prompts: list[list[int]], sampling: SamplingConfig) -> list[GenerationResult]:
        rids = [self.add_request(p, sampling) for p in prompts]
        out: dict[int, GenerationResult] = {}
        while self.has_unfinished():
            for res in self.step():
                out[res.index] = res
        return [out[r] for r in rids]

    # ------------------------------------------------------------------ bookkeeping
    def _finalize(self, req: _Request) -> GenerationResult:
        responses = [s.tokens[s.prompt_len:] for s in req.seqs]
        now = time.perf_counter()
        n = len(req.seqs)
        info = RequestInfo(num_calls=[0] * n, timeouts=[0] * n, tool_errors=[""] * n, tool_outputs=[""] * n,
                           tool_runtimes=[0.0] * n, tool_calleds=[False] * n, rollout_states=[{} for _ in range(n)])
        return GenerationResult(
            responses=responses, finish_reasons=[s.finish_reason for s in req.seqs], masks=[[1] * len(r) for r in responses],
            request_info=info, index=req.rid, prompt_id=req.meta.get("prompt_id"), epoch_number=req.meta.get("epoch_number"),
            token_statistics=TokenStatistics(len(req.prompt), sum(len(r) for r in responses), now - req.start_time, req.start_time),
            start_time=req.start_time, logprobs=[s.logprobs for s in req.seqs], model_step=self.model_step,
            is_eval=req.meta.get("is_eval", False), queries=[list(req.prompt)] * n, ground_truth=req.meta.get("ground_truth"),
            dataset=req.meta.get("dataset"), raw_query=req.meta.get("raw_query"))

    def _accept(self, seq: _Sequence, token: int, logprob: float, advance: bool = True) -> None:
        seq.tokens.append(token)
        seq.logprobs.append(logprob)
        seq.last_token = token
        if advance:  # the decode step advances all its sequences with one native call
            self.host.advance(seq.sid, 1)
        sp = seq.request.sampling
        n_gen = len(seq.tokens) - seq.prompt_len
        if token in self.eos and n_gen >= sp.min_tokens:
            seq.finish_reason = "stop"
        elif sp.stop and self.tokenizer is not None and n_gen >= sp.min_tokens:
            tail = self.tokenizer.decode(seq.tokens[max(seq.prompt_len, len(seq.tokens) - 16):])
            if any(s in tail for s in sp.stop):
                seq.finish_reason = "stop"
        if seq.finish_reason is None and n_gen >= sp.max_tokens:
            seq.finish_reason = "length"

    def _sampling_tensors(self, seqs: list[_Sequence]):
        dev = self.device
        temp = torch.tensor([s.request.sampling.temperature for s in seqs], dtype=torch.float32, device=dev)
        top_p = torch.tensor([s.request.sampling.top_p for s in seqs], dtype=torch.float32, device=dev)
        seeds = torch.tensor([s.seed for s in seqs], dtype=torch.int64, device=dev)
        ctr = torch.tensor([len(s.tokens) - s.prompt_len for s in seqs], dtype=torch.int32, device=dev)
        return temp, top_p, seeds, ctr

    def _sample(self, logits: torch.Tensor, seqs: list[_Sequence]):
        temp, top_p, seeds, ctr = self._sampling_tensors(seqs)
        # the sampler kernel only needs bf16 logits on a B200: the PyTorch path of the model (OLMo-family models on a GPU) uses it
        # too instead of the row-by-row host sampler, which is the oracle and the CPU path
        if self.ops == "fused" or (logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(-1) == 1 and lib.available()):
            from ..ops.lib import call, ptr, stream_ptr

            B, V = logits.shape
            toks = torch.empty(B, dtype=torch.int64, device=self.device)
            lps = torch.empty(B, dtype=torch.float32, device=self.device)
            call("b200_sample", ptr(logits), logits.stride(0), B, V, ptr(temp), ptr(top_p), ptr(seeds), ptr(ctr), ptr(toks), ptr(lps), stream_ptr())
            return toks.tolist(), lps.tolist()
        from .sampler import sample_ref

        return sample_ref(logits, temp, top_p, seeds, ctr)

    # ------------------------------------------------------------------ model math
    def _splitk_acc(self, which: int, T: int) -> torch.Tensor:
        """Persistent zero-initialised fp32 [256, hidden] accumulators (one per projection); the consuming norm re-zeroes them."""
        if which not in self._acc32:
            self._acc32[which] = torch.zeros(256, self.spec.hidden_size, dtype=torch.float32, device=self.device)
        return self._acc32[which][:T]

    def _slots_for(self, seq: _Sequence, start: int, end: int) -> list[int]:
        blocks, _ = self.host.blocks(seq.sid)
        return [blocks[t // KV_BLOCK] * KV_BLOCK + t % KV_BLOCK for t in range(start, end)]

    def _layer_stack(self, ids: torch.Tensor, pos: torch.Tensor, slots: torch.Tensor, attn_fn) -> torch.Tensor:
        """Embedding -> decoder layers -> final norm for a flat batch of tokens.  ``slots`` may hold
        several destination maps back to back (length a multiple of the token count)."""
        s, p = self.spec, self.model.p
        T = ids.numel()
        if self.ops == "fused":
            from ..ops import fused as f
            from ..ops.lib import call, ptr, stream_ptr

            pos32 = pos.to(torch.int32)
            rope_tab = f.rope_table(pos32, self.model.inv_freq, s.head_dim)
            impl = "2cta"
            # few rows and a 4096-wide output: the 256-wide tiles leave most SMs idle, the 64-wide kernel streams the weights
            # from four times as many CTAs (measured at M = 256: o_proj 34 -> 21 us, down_proj 81 -> 54 us)
            impl_narrow = "skinny" if T <= 256 else "2cta"
            impl_qkv = "skinny128" if T <= 256 else "2cta"  # 6144-wide: 128-wide tiles (qkv 36.8 -> 29.5 us at M = 256)
            stream, delta = f.embedding_fwd(p["embed"], ids), None
            tp = self.tp

            dec = tp is None and T <= 256 and self.decode_gemm
            fuse_rope_kv = slots.numel() == T and s.head_dim == 128 and rope_tab is not None

            def add_norm(partial, w, res):
                """(normed, new residual stream): local fused add+norm, or the cross-rank reduction fused with it."""
                if partial.dim() == 3:  # fp32 K-slice planes of the decode GEMM: summed by the norm
                    return f.rmsnorm_fwd_parts(partial, w, s.rms_norm_eps, res)
                if partial.dtype == torch.float32:  # split-K accumulator: consumed (and zeroed) by the norm
                    return f.rmsnorm_fwd_acc32_(partial, w, s.rms_norm_eps, res)
                if tp is None or res is None:
                    y, h, _ = f.rmsnorm_fwd(partial, w, s.rms_norm_eps, res=res)
                    return y, h
                return tp.reduce_norm(partial, w, s.rms_norm_eps, res=res)

            row_out = (lambda: tp.out_buffer(T)) if tp is not None else (lambda: None)
            # peer push fused into the GEMM epilogue: built and tested, but measured 2.4x slower than "plain GEMM + pulling
            # reduction" at T = 4096 (row-per-thread epilogue stores reach the peer as 16-byte writes), so it is opt-in
            push = tp is not None and tp.world == 2 and T > 256 and os.environ.get("B200_TP_PUSH", "0") == "1"

            splitk = tp is None and T <= 256 and self.decode_splitk

            def col_proj(x, w, wide_impl):
                return f.gemm_decode(x, w) if dec else f.gemm(x, w, impl=wide_impl)

            def row_proj(x, w, which=0):
                if dec:  # K slices on different CTA pairs where that fills the GPU; the following norm adds them up
                    return f.gemm_decode(x, w, plan=f.decode_gemm_plan(w.shape[0], w.shape[1], True, T))
                # few rows, long K: cut K over SMs, fp32 partial sums added into a persistent buffer that the following norm
                # consumes.  Measured (8B shapes): down_proj 54 -> 38 us at 64 rows (4 slices), 54 -> 49 us at 256 rows (2 slices);
                # o_proj 22 -> 17 us at 64 rows, no gain at 256 rows (stays on the narrow-tile kernel)
                if splitk and (which == 1 or T <= 128):
                    return f.gemm_splitk_(self._splitk_acc(which, T), x, w, 4 if T <= 128 else 2)
                return tp.row_gemm(x, w) if push else f.gemm(x, w, row_out(), impl=impl_narrow)

            for i in range(s.num_layers):
                if s.post_norm:   # OLMo-2 / OLMo-3: the sub-layers read the stream as it is and their output is normalised
                    n1 = stream
                else:
                    n1, h_in = add_norm(delta if delta is not None else stream, p[f"l{i}.attn_norm"], stream if delta is not None else None)
                qkv = col_proj(n1, p[f"l{i}.wqkv"], impl_qkv)
                self.model.qkv_bias_and_norm_(qkv, i)
                if fuse_rope_kv:  # one destination per token (decode, plain prefill): rotation and cache write in one pass
                    call("b200_rope_kv_decode", ptr(qkv), ptr(rope_tab), ptr(self.k_cache[i]), ptr(self.v_cache[i]), ptr(slots), T,
                         s.num_heads, s.num_kv_heads, s.head_dim, stream_ptr())
                else:
                    f.rope_(qkv, pos32, self.model.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim, table=rope_tab)
                    call("b200_kv_write", ptr(qkv), ptr(self.k_cache[i]), ptr(self.v_cache[i]), ptr(slots), slots.numel(), T,
                         s.num_heads, s.num_kv_heads, s.head_dim, stream_ptr())
                attn = attn_fn(i, qkv)
                o = row_proj(attn, p[f"l{i}.wo"])
                if s.post_norm:
                    stream = stream + add_norm(o, p[f"l{i}.attn_norm"], None)[0]
                    act = f.swiglu_fwd(col_proj(stream, p[f"l{i}.w_gate_up"], impl))
                    stream = stream + add_norm(row_proj(act, p[f"l{i}.w_down"], 1), p[f"l{i}.mlp_norm"], None)[0]
                    continue
                n2, h_mid = add_norm(o, p[f"l{i}.mlp_norm"], h_in)
                act = f.swiglu_fwd(col_proj(n2, p[f"l{i}.w_gate_up"], impl))
                delta = row_proj(act, p[f"l{i}.w_down"], 1)
                stream = h_mid
            nf, _ = add_norm(delta, p["final_norm"], stream) if delta is not None else add_norm(stream, p["final_norm"], None)
            return nf
        x = p["embed"][ids]
        for i in range(s.num_layers):
            if s.is_gdn(i):   # a pre-norm block whose mixer carries a recurrent state per sequence instead of cached keys and values
                from ..models.gdn import gdn_segment

                n1 = ref.rmsnorm(x, p[f"l{i}.attn_norm"], s.rms_norm_eps)
                if all(hi - lo == 1 and src is not None for lo, hi, src, _ in self._gdn_runs):
                    # a decode step: one recurrence step for all sequences at once
                    from ..models.gdn import gdn_decode_step

                    states = [self._gdn_state[src][i] for _, _, src, _ in self._gdn_runs]
                    mixed, tails, S = gdn_decode_step(n1, p, i, s, torch.stack([t for t, _ in states]), torch.stack([st for _, st in states]))
                    for b, (_, _, _, dsts) in enumerate(self._gdn_runs):
                        for sid in dsts:
                            self._gdn_state[sid][i] = (tails[b], S[b])
                    x = x + mixed
                else:
                    outs = []
                    for lo, hi, src, dsts in self._gdn_runs:
                        o, st = gdn_segment(n1[lo:hi], p, i, s, None if src is None else self._gdn_state[src][i])
                        outs.append(o)
                        for sid in dsts:
                            self._gdn_state.setdefault(sid, {})[i] = st
                    x = x + torch.cat(outs)
                x = x + self.model.ref_mlp(ref.rmsnorm(x, p[f"l{i}.mlp_norm"], s.rms_norm_eps), p, i)
                continue
            # pre-norm blocks (Llama, Qwen, Mistral) norm the sub-layer's input; post-norm blocks (OLMo-2 / OLMo-3) its output
            n1 = x if s.post_norm else ref.rmsnorm(x, p[f"l{i}.attn_norm"], s.rms_norm_eps)
            qkv = self.model.ref_qkv(n1, p, i)
            if s.use_rope:
                qkv = ref.rope(qkv, pos, self.model.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim)
            heads = qkv.view(T, s.num_heads + 2 * s.num_kv_heads, s.head_dim)
            k_new, v_new = heads[:, s.num_heads : s.num_heads + s.num_kv_heads], heads[:, s.num_heads + s.num_kv_heads :]
            for rep in range(slots.numel() // T):
                sl = slots[rep * T : (rep + 1) * T]
                ok = sl >= 0
                blk, off = sl[ok] // KV_BLOCK, sl[ok] % KV_BLOCK
                self.k_cache[i][blk, :, off] = k_new[ok]
                self.v_cache[i][blk, :, off] = v_new[ok]
            attn = attn_fn(i, qkv)
            o = ref.linear(attn, p[f"l{i}.wo"])
            if self.tp is not None:   # this rank's heads only: the projection's output is a partial sum
                o = self.tp.all_reduce_sum(o.contiguous())
            x = x + (ref.rmsnorm(o, p[f"l{i}.attn_norm"], s.rms_norm_eps) if s.post_norm else o)
            n2 = x if s.post_norm else ref.rmsnorm(x, p[f"l{i}.mlp_norm"], s.rms_norm_eps)
            d = self.model.ref_mlp(n2, p, i)  # dense SwiGLU, or the router's experts
            if self.tp is not None:
                d = self.tp.all_reduce_sum(d.contiguous())
            x = x + (ref.rmsnorm(d, p[f"l{i}.mlp_norm"], s.rms_norm_eps) if s.post_norm else d)
        return ref.rmsnorm(x, p["final_norm"], s.rms_norm_eps)

    def _logits(self, hidden: torch.Tensor) -> torch.Tensor:
        w = self.model.lm_head_weight()
        if self.ops == "fused":
            from ..ops import fused as f

            hidden = hidden.contiguous()
            if self.tp is None and self.decode_gemm and hidden.shape[0] <= 256 and w.shape[0] % 16 == 0:
                return f.gemm_decode(hidden, w)
            return f.gemm(hidden, w, impl="2cta")
        return ref.linear(hidden, w)

    def _prefill(self, seqs: list[_Sequence]) -> None:
        """Prompt pass for newly admitted sequences.  Samples of one request that start from the same
        tokens run through the model ONCE; the others reuse the result (their private tail block gets
        its own copy of the K/V rows, their first token is sampled from the same logits row)."""
        s = self.spec
        groups: dict[tuple, list[_Sequence]] = {}
        for q in seqs:
            groups.setdefault((q.request.rid, len(q.tokens), len(q.tokens) == q.prompt_len), []).append(q)
        reps, members = [], []
        for (rid, n, fresh), qs in groups.items():
            if fresh:
                reps.append(qs[0])
                members.append(qs)
            else:  # resumed after preemption: each has its own history
                for q in qs:
                    reps.append(q)
                    members.append([q])
        # run the prompts in sub-batches of at most ``prefill_token_budget`` tokens (documents are independent): bounds the
        # activation memory of a step and, with tensor parallelism, fits the exchange buffers
        budget = self.prefill_token_budget if self.tp is None else min(self.prefill_token_budget, self.tp.max_tokens)
        i = 0
        while i < len(reps):
            j, tok = i, 0
            while j < len(reps) and (j == i or tok + len(reps[j].tokens) <= budget):
                tok += len(reps[j].tokens)
                j += 1
            self._prefill_batch(reps[i:j], members[i:j])
            i = j

    def _prefill_batch(self, reps: list, members: list) -> None:
        """Prompt pass of a sub-batch.  A sequence admitted with a cached prefix (``enable_prefix_caching``) runs the layers
        over its remaining tokens only; its attention sees the cached K/V of the prefix, gathered from the paged cache into
        the packed layout the varlen kernel reads (prefix rows carry zero queries and their outputs are dropped - the
        projections, which dominate, are skipped for them)."""
        s = self.spec
        lens = [len(q.tokens) for q in reps]
        cached = [min(self.host.cached_tokens(q.sid), n - 1) if self.prefix_caching else 0 for q, n in zip(reps, lens)]
        ids = torch.tensor([t for q, c in zip(reps, cached) for t in q.tokens[c:]], dtype=torch.long)
        new_lens = [n - c for n, c in zip(lens, cached)]
        T = int(ids.numel())
        pos = torch.cat([torch.arange(c, n) for c, n in zip(cached, lens)])
        cu = torch.tensor([0] + list(torch.tensor(new_lens).cumsum(0)), dtype=torch.int32)
        n_var = max(len(m) for m in members)
        slot_rows = []
        for v in range(n_var):
            row = []
            for q, ms, n, c in zip(reps, members, lens, cached):
                if v < len(ms):
                    full = (ms[v].prompt_len // KV_BLOCK) * KV_BLOCK if (v > 0) else 0
                    sl = self._slots_for(ms[v], c, n)
                    skip = max(0, min(full, n) - c)
                    row += [-1] * skip + sl[skip:]  # shared full blocks were written by variant 0 (or came from the cache)
                else:
                    row += [-1] * (n - c)
            slot_rows.append(row)
        dev = self.device
        ids_d, pos_d, cu_d = ids.to(dev), pos.to(dev), cu.to(dev)
        if s.has_gdn:   # every prompt starts from an empty state; the samples of one request all continue from their prompt's
            b = cu.tolist()
            self._gdn_runs = [(b[j], b[j + 1], None, [m.sid for m in members[j]]) for j in range(len(reps))]
        slots = torch.tensor([x for r in slot_rows for x in r], dtype=torch.long, device=dev)
        scale = s.attn_scale
        if self.ops == "fused":
            from ..ops import fused as f

            attend = lambda qkv, cu_, i: f.attn_fwd(qkv, cu_, s.num_heads, s.num_kv_heads, s.head_dim, scale)[0]
        else:
            attend = lambda qkv, cu_, i: ref.attention_varlen(qkv, cu_, s.num_heads, s.num_kv_heads, s.head_dim, scale,
                                                              allow_sdpa=bool(s.post_norm or s.num_experts), window=s.window(i))
        if any(cached):
            # packed layout with the prefixes in place: sequence j occupies rows [o_j, o_j + n_j), its first c_j rows are cached
            offs = [0]
            for n in lens:
                offs.append(offs[-1] + n)
            new_rows = torch.tensor([offs[j] + t for j, (c, n) in enumerate(zip(cached, lens)) for t in range(c, n)], dtype=torch.long, device=dev)
            pref_rows = torch.tensor([offs[j] + t for j, c in enumerate(cached) for t in range(c)], dtype=torch.long, device=dev)
            pslots = [x for q, c in zip(reps, cached) for x in self._slots_for(q, 0, c)]
            pblk = torch.tensor([x // KV_BLOCK for x in pslots], dtype=torch.long, device=dev)
            poff = torch.tensor([x % KV_BLOCK for x in pslots], dtype=torch.long, device=dev)
            cu_ext = torch.tensor(offs, dtype=torch.int32, device=dev)
            qd, kd = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim

            def attn_fn(i, qkv):
                ext = torch.zeros(offs[-1], qkv.shape[1], dtype=qkv.dtype, device=dev)
                ext[new_rows] = qkv
                ext[pref_rows, qd:qd + kd] = self.k_cache[i][pblk, :, poff].reshape(len(pslots), kd)
                ext[pref_rows, qd + kd:] = self.v_cache[i][pblk, :, poff].reshape(len(pslots), kd)
                return attend(ext, cu_ext, i)[new_rows].contiguous()
        else:
            attn_fn = lambda i, qkv: attend(qkv, cu_d, i)
        hidden = self._layer_stack(ids_d, pos_d, slots, attn_fn)
        last = cu_d[1:].long() - 1
        logits = self._logits(hidden[last])
        self.stats["prefill_tokens"] += T
        self.stats["prefix_cached_tokens"] = self.stats.get("prefix_cached_tokens", 0) + sum(cached)
        flat_members = [m for ms in members for m in ms]
        rows = torch.tensor([ri for ri, ms in enumerate(members) for _ in ms], device=dev)
        toks, lps = self._sample(logits[rows].contiguous(), flat_members)
        for q, t, lp in zip(flat_members, toks, lps):
            self._accept(q, int(t), float(lp))

    # ---- fused decode step: everything between "inputs on the device" and "sampled tokens" is one replayable unit
    def _decode_device(self, buf: dict, B: int, max_blocks: int, splits: int):
        """Layer stack + lm_head + sampling for ``B`` sequences, reading only the device tensors in ``buf``."""
        from ..ops.lib import call, ptr, stream_ptr

        s, dev = self.spec, self.device
        scale = s.attn_scale
        part_o = torch.empty(B * s.num_heads * splits * s.head_dim, dtype=torch.float32, device=dev) if splits > 1 else None
        part_ml = torch.empty(B * s.num_heads * splits * 2, dtype=torch.float32, device=dev) if splits > 1 else None

        def attn_fn(i, qkv):
            out = torch.empty(B, s.num_heads * s.head_dim, dtype=qkv.dtype, device=dev)
            call("b200_paged_decode", ptr(qkv), ptr(self.k_cache[i]), ptr(self.v_cache[i]), ptr(buf["bt"]), max_blocks, ptr(buf["ctx"]), B,
                 s.num_heads, s.num_kv_heads, s.head_dim, scale, splits, ptr(out), ptr(part_o), ptr(part_ml), stream_ptr())
            return out

        hidden = self._layer_stack(buf["ids"], buf["pos"], buf["slots"], attn_fn)
        logits = self._logits(hidden)
        V = logits.shape[1]
        call("b200_sample", ptr(logits), logits.stride(0), B, V, ptr(buf["temp"]), ptr(buf["top_p"]), ptr(buf["seeds"]), ptr(buf["ctr"]),
             ptr(buf["toks"]), ptr(buf["lps"]), stream_ptr())

    _IN_FIELDS = (("ids", "int64"), ("pos", "int64"), ("slots", "int64"), ("seeds", "int64"), ("ctx", "int32"), ("ctr", "int32"),
                  ("temp", "float32"), ("top_p", "float32"))

    def _stage(self, B: int, width: int):
        """Pinned host staging for ``B`` sequences: ONE blob holding every per-step input (block table last, room for
        ``width`` blocks per sequence) and one for the outputs, with numpy views of the fields."""
        import numpy as np

        st = self._stages.get(B)
        if st is not None and st["width"] >= width:
            return st
        width = max(64, -(-width // 64) * 64)
        fixed = 48 * B
        blob = torch.empty(fixed + 4 * B * width, dtype=torch.uint8).pin_memory() if self.device.type == "cuda" else torch.empty(fixed + 4 * B * width, dtype=torch.uint8)
        out = torch.empty(12 * B, dtype=torch.uint8).pin_memory() if self.device.type == "cuda" else torch.empty(12 * B, dtype=torch.uint8)
        raw = blob.numpy()
        views, off = {}, 0
        for name, dt in self._IN_FIELDS:
            nbytes = np.dtype(dt).itemsize * B
            views[name] = raw[off:off + nbytes].view(dt)
            off += nbytes
        views["bt"] = raw[off:].view("int32")
        oraw = out.numpy()
        st = {"width": width, "blob": blob, "out": out, "np": views, "toks": oraw[: 8 * B].view("int64"), "lps": oraw[8 * B:].view("float32"), "static_key": None}
        self._stages[B] = st
        return st

    def _device_buffers(self, B: int, max_blocks: int) -> dict:
        """Device twin of the staging blob for one (B, block-table width): typed views into one allocation, so a step's
        inputs arrive with a single copy and its outputs leave with one."""
        import numpy as np

        dev = self.device
        blob = torch.empty(48 * B + 4 * B * max_blocks, dtype=torch.uint8, device=dev)
        out = torch.empty(12 * B, dtype=torch.uint8, device=dev)
        buf, off = {"blob": blob, "out": out}, 0
        for name, dt in self._IN_FIELDS:
            nbytes = np.dtype(dt).itemsize * B
            buf[name] = blob[off:off + nbytes].view(getattr(torch, dt))
            off += nbytes
        buf["bt"] = blob[off:].view(torch.int32).view(B, max_blocks)
        buf["toks"] = out[: 8 * B].view(torch.int64)
        buf["lps"] = out[8 * B:].view(torch.float32)
        return buf

    def _decode_fused(self, seqs: list[_Sequence]):
        """Host side of the fused decode step: the scheduler writes positions, cache slots, context lengths and the block
        table of all sequences into one pinned blob (one native call), one copy takes it to the device, then the device
        part runs - replaying a CUDA graph when this (batch size, block-table width) has been seen before, so the
        launch-bound inner loop (about 400 kernels for a 32-layer model) costs one graph launch - and one copy brings the
        sampled tokens and their log-probs back."""
        import numpy as np

        B = len(seqs)
        s = self.spec
        sids = np.fromiter((q.sid for q in seqs), dtype=np.int64, count=B)
        st = self._stage(B, 64)
        v = st["np"]
        max_blocks = self.host.pack_decode(sids, v["pos"], v["slots"], v["ctx"], v["ctr"], v["bt"])
        while max_blocks == -2:  # a longer context than the staging was sized for
            st = self._stage(B, st["width"] * 2)
            v = st["np"]
            max_blocks = self.host.pack_decode(sids, v["pos"], v["slots"], v["ctx"], v["ctr"], v["bt"])
        v["ids"][:] = np.fromiter((q.last_token for q in seqs), dtype=np.int64, count=B)
        key_static = sids.tobytes()
        if st["static_key"] != key_static:  # sampling parameters change only when the set of sequences does
            v["temp"][:] = np.fromiter((q.request.sampling.temperature for q in seqs), dtype=np.float32, count=B)
            v["top_p"][:] = np.fromiter((q.request.sampling.top_p for q in seqs), dtype=np.float32, count=B)
            v["seeds"][:] = np.fromiter((q.seed for q in seqs), dtype=np.int64, count=B)
            st["static_key"] = key_static
        self._last_sids = sids
        splits = 1 if B * s.num_kv_heads >= 148 else max(1, min(8, 148 // max(1, B * s.num_kv_heads), max_blocks // 4))
        nbytes = 48 * B + 4 * B * max_blocks
        key = (B, max_blocks, splits)
        entry = self._graphs.get(key)
        cuda = self.device.type == "cuda"

        def results(buf):
            st["out"].copy_(buf["out"], non_blocking=True)
            if cuda:
                torch.cuda.current_stream(self.device).synchronize()
            return st["toks"].tolist(), st["lps"].tolist()

        if entry is None:
            buf = self._device_buffers(B, max_blocks)
            buf["blob"].copy_(st["blob"][:nbytes], non_blocking=True)
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            if not self.use_cuda_graphs or seen < 1 or B < 4:
                self._decode_device(buf, B, max_blocks, splits)  # eager (also the warm-up of this shape)
                return results(buf)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self._decode_device(buf, B, max_blocks, splits)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, buf)
            if len(self._graphs) >= 48:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = entry
            graph.replay()  # the capture only records; this runs the step
            return results(buf)
        graph, buf = entry
        buf["blob"].copy_(st["blob"][:nbytes], non_blocking=True)
        graph.replay()
        self._t_launched = time.perf_counter()
        return results(buf)

    def _decode(self, seqs: list[_Sequence]) -> None:
        """One token for every running sequence."""
        s = self.spec
        dev = self.device
        B = len(seqs)
        if self.ops == "fused":
            t0 = time.perf_counter()
            self._t_launched = None
            toks, lps = self._decode_fused(seqs)
            t1 = time.perf_counter()
            self.stats["decode_tokens"] += B
            self.host.advance_many(self._last_sids)
            for q, t, lp in zip(seqs, toks, lps):
                self._accept(q, t, lp, advance=False)
            if self._t_launched is not None:  # graph replay: split the call into packing and waiting for the device
                self.stats["host_pack_s"] += self._t_launched - t0
                self.stats["device_wait_s"] += t1 - self._t_launched
                self.stats["host_accept_s"] += time.perf_counter() - t1
                self.stats["decode_steps"] += 1
            return
        ids = torch.tensor([q.last_token for q in seqs], dtype=torch.long, device=dev)
        if s.has_gdn:
            self._gdn_runs = [(b, b + 1, q.sid, [q.sid]) for b, q in enumerate(seqs)]
        ctx_list = [len(q.tokens) for q in seqs]  # the new token sits at position len-1
        pos = torch.tensor([n - 1 for n in ctx_list], dtype=torch.long, device=dev)
        tables = [self.host.blocks(q.sid)[0] for q in seqs]
        max_blocks = max(len(t) for t in tables)
        bt = torch.zeros(B, max_blocks, dtype=torch.int32)
        for i, t in enumerate(tables):
            bt[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
        bt = bt.to(dev)
        slots = torch.tensor([tables[i][(n - 1) // KV_BLOCK] * KV_BLOCK + (n - 1) % KV_BLOCK for i, n in enumerate(ctx_list)],
                             dtype=torch.long, device=dev)
        ctx = torch.tensor(ctx_list, dtype=torch.int32, device=dev)
        scale = s.attn_scale
        g = s.num_heads // s.num_kv_heads
        # all sequences at once: their pages gathered into one padded [B, positions] view, positions beyond a sequence's
        # context (and before a sliding-window layer's window) masked; in groups of sequences so that a group's gathered
        # keys and values stay within about 4 GB
        span = max_blocks * KV_BLOCK
        group = max(1, min(B, int(4e9 // (2 * span * s.num_kv_heads * s.head_dim * self.k_cache.element_size()))))
        ctx_col = ctx.long()[:, None]
        where = torch.arange(span, device=dev)[None, :]

        def attn_fn(i, qkv):
            q = qkv.view(B, s.num_heads + 2 * s.num_kv_heads, s.head_dim)[:, : s.num_heads].reshape(B, s.num_kv_heads, g, s.head_dim)
            w = s.window(i)
            live = where < ctx_col
            if w:   # sliding-window layers read the latest w positions only
                live = live & (where >= ctx_col - w)
            out = torch.empty(B, s.num_heads * s.head_dim, dtype=torch.float32, device=dev)
            for b0 in range(0, B, group):
                b1 = min(B, b0 + group)
                pages = bt[b0:b1].long()
                # [b, blocks, Hkv, BLOCK, D] -> [b, Hkv, blocks * BLOCK, D]
                k = self.k_cache[i][pages].permute(0, 2, 1, 3, 4).reshape(b1 - b0, s.num_kv_heads, span, s.head_dim)
                v = self.v_cache[i][pages].permute(0, 2, 1, 3, 4).reshape(b1 - b0, s.num_kv_heads, span, s.head_dim)
                qg = q[b0:b1]
                if k.numel() * 8 <= 1e9:   # small enough to hold in fp32 (this path is also the oracle of the kernel tests)
                    k, v, qg = k.float(), v.float(), qg.float()
                sc = torch.einsum("bhgd,bhtd->bhgt", qg, k).float() * scale   # half precision: products accumulate in fp32 inside the matmul
                sc = sc.masked_fill(~live[b0:b1, None, None, :], float("-inf"))
                out[b0:b1] = torch.einsum("bhgt,bhtd->bhgd", torch.softmax(sc, -1).to(v.dtype), v).float().reshape(b1 - b0, -1)
            return out.to(qkv.dtype)
        hidden = self._layer_stack(ids, pos, slots, attn_fn)
        logits = self._logits(hidden)
        self.stats["decode_tokens"] += B
        toks, lps = self._sample(logits, seqs)
        for q, t, lp in zip(seqs, toks, lps):
            self._accept(q, int(t), float(lp))
