"""Decoder-only transformer (Llama / Qwen / Mistral pre-norm blocks, OLMo-2 / OLMo-3 post-norm blocks, OLMoE mixture of experts)
over a flat parameter buffer.

Two execution paths share the same weights:

* ``ops="fused"`` - the B200 path.  Forward and backward are driven explicitly, layer by layer,
  through the sm_100a kernels in ``open_instruct_b200.ops.fused``: tcgen05 GEMMs for the
  projections (weight gradients are accumulated in fp32 straight from the GEMM epilogue into
  the flat ``main_grad`` buffer), varlen packed attention, fused residual-add RMSNorm, in-place
  RoPE, SwiGLU and the in-place log-prob gradient.  Cheap ops (RMSNorm output, SwiGLU
  activation) are recomputed in the backward instead of stored.
  Post-norm blocks (``h = x + norm(attn(x))``) run through the same kernels; mixture-of-experts layers do not.
* ``ops="ref"`` - plain PyTorch autograd over the same buffer; runs on CPU (fp32) and is the
  oracle the fused path is tested against, and the compute path of the library baseline.
* ``ops="emulated"`` - the fused path's driver with every kernel replaced by its PyTorch restatement
  (``open_instruct_b200.ops.emulated``): any device and dtype; the CPU test bed of the driver's bookkeeping.

The public entry points return per-token log-probabilities (or final hidden states) that are
differentiable with respect to the flat parameter buffer on both paths, so SFT, DPO, GRPO and
reward-model losses are written once in PyTorch on ``[T]``-sized tensors.

Packed input convention (same as the reference's padding-free collator,
``open_instruct/padding_free_collator.py:67-120``): ``input_ids`` and ``position_ids`` are 1-D over
all tokens of the micro-batch, ``cu_seqlens`` int32 ``[num_docs + 1]`` gives document boundaries.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from ..ops import ref
from .spec import ModelSpec, ParamLayout


def _fused():
    from ..ops import fused

    return fused


@dataclass
class _LayerStash:
    h_in: torch.Tensor  # residual stream entering the layer
    rstd1: torch.Tensor
    qkv: torch.Tensor  # post-RoPE
    attn: torch.Tensor
    lse: torch.Tensor
    h_mid: torch.Tensor  # residual stream after attention
    rstd2: torch.Tensor
    gate_up: torch.Tensor
    attn_tok: torch.Tensor | None = None  # sequence parallel: attention output for MY tokens, all heads
    qk: tuple | None = None                # per-head q/k RMSNorm: (q_pre, rstd_q, k_pre, rstd_k)
    n1: torch.Tensor | None = None         # kept instead of recomputed when ``keep_cheap_activations``
    n2: torch.Tensor | None = None
    act: torch.Tensor | None = None
    o: torch.Tensor | None = None          # post-norm blocks: the attention sub-layer's output before its norm
    d: torch.Tensor | None = None          # post-norm blocks: the feed-forward sub-layer's output before its norm
    moe: "_MoEStash | None" = None         # mixture of experts: routing and the experts' intermediate results


@dataclass
class _MoEStash:
    tok: torch.Tensor       # [T * k] token of every (token, expert) assignment, grouped by expert
    slot: torch.Tensor      # [T * k] which of the token's k choices the assignment is
    counts: list            # assignments per expert (the groups' lengths)
    gu: torch.Tensor        # [T * k, 2F] gate | up of every assignment (overwritten by its gradient in the backward)
    y: torch.Tensor         # [T * k, D] expert outputs before the routing weight
    lg: torch.Tensor        # [T, E] fp32 router logits, leaf of the small autograd graph that yields ...
    probs: torch.Tensor     # ... their softmax and
    top_w: torch.Tensor     # ... the k routing weights of every token


def load_balancing_loss(router_logits: list, num_experts: int, top_k: int):
    """Switch-Transformer auxiliary loss over the router logits of all layers of one forward (what transformers returns as
    ``aux_loss`` for OLMoE and the reference adds to the SFT loss, ``open_instruct/finetune.py:817-819``): ``num_experts *
    sum_e f_e * P_e`` with ``f_e`` the share of (token, rank) assignments that went to expert e, per top-k rank, and ``P_e`` the
    mean router probability of e."""
    if not router_logits:
        return None
    logits = torch.cat(list(router_logits), dim=0).float()
    probs = torch.softmax(logits, dim=-1)
    _, sel = probs.topk(top_k, dim=-1)
    mask = torch.nn.functional.one_hot(sel, num_experts).float()       # [N, k, E]
    tokens_per_expert = mask.mean(dim=0)                                  # [k, E]
    prob_per_expert = probs.mean(dim=0)                                   # [E]
    return (tokens_per_expert * prob_per_expert[None, :]).sum() * num_experts


class LlamaModel:
    """Weights + forward/backward engine.  Not an ``nn.Module``: state is one flat tensor."""

    def __init__(self, spec: ModelSpec, device="cpu", dtype=torch.float32, ops: str = "ref", seed: int = 0,
                 init: str = "normal", with_lm_head: bool = True, flat: torch.Tensor | None = None,
                 gradient_checkpointing: bool = False, sharded: bool = False):
        if ops not in ("ref", "fused", "emulated"):
            raise ValueError("ops must be 'ref', 'fused' or 'emulated'")
        # "emulated": the fused path's hand-driven forward / backward with every kernel replaced by its PyTorch restatement
        # (``ops.emulated``), on any device and dtype - the CPU test bed of the driver; everything else sees ops == "fused"
        self.emulated = ops == "emulated"
        if self.emulated:
            ops = "fused"
        if ops == "fused" and (spec.has_gdn or not spec.use_rope):
            raise NotImplementedError("hybrid models (gated DeltaNet layers) and attention without RoPE run with ops='ref'")
        self.spec = spec
        self.ops = ops
        self.device = torch.device(device)
        self.dtype = dtype
        self.layout = ParamLayout(spec, with_lm_head=with_lm_head)
        self.with_lm_head = with_lm_head
        self.gradient_checkpointing = gradient_checkpointing
        if self.emulated:
            from ..ops import emulated

            self.kernels = emulated
        elif ops == "fused":
            self.kernels = _fused()
            if dtype != torch.bfloat16 or self.device.type != "cuda":
                raise ValueError("the fused path runs bf16 on CUDA")
            if spec.head_dim != 128:
                raise NotImplementedError("fused attention is built for head_dim 128")
            if spec.num_experts and (spec.post_norm or sharded):
                raise NotImplementedError("mixture-of-experts layers on the fused path: pre-norm blocks with resident parameters only")
            from ..ops import lib

            if not lib.available():
                raise RuntimeError("ops='fused' needs a B200 (sm_100) device and libb200ops.so")
        self.zero3 = None  # parallel.zero3.Zero3State when the parameters are sharded over the ranks (fused path)
        if sharded:
            # no resident flat buffer: ``Zero3State.attach`` points ``p`` / ``g`` at its gather workspaces
            if ops != "fused":
                raise NotImplementedError("parameter sharding runs on the fused path")
            self.flat, self.p = None, {}
        elif flat is None:
            flat = torch.empty(self.layout.total, dtype=dtype, device=self.device)
            self.flat = flat
            self.init_weights(seed, init)
        else:
            if flat.numel() < self.layout.total:
                raise ValueError("flat buffer is smaller than the layout")
            self.flat = flat
        if not sharded:
            self.p = self.layout.views(self.flat)
        self._last_qk = None
        self._rope_tab = None
        self._max_doc = 0   # longest document of the batch in flight when the model has sliding-window layers
        # keep the RMSNorm outputs and the SwiGLU activation for the backward pass instead of recomputing them
        # (5.8 GB per 4096-token micro-batch at 8B; about 2.5 % of the step): on by default, off under checkpointing
        self.keep_cheap_activations = os.environ.get("B200_RECOMPUTE_CHEAP", "0") != "1"
        # mixture of experts: the weight with which the trainer adds ``aux_loss`` to its loss.  On the fused path ``aux_loss`` is a
        # detached scalar and the backward pass adds this multiple of its gradient to the routers itself.
        self.aux_loss_coef = 0.0
        self.tp = None  # parallel.tp.TrainTP when the layers are split over a tensor-parallel group (spec is then the LOCAL spec)
        self.sp = None  # parallel.ulysses.UlyssesContext when the sequence is split over ranks (fused path)
        # called with (lo, hi) once the flat gradient range [lo, hi) is final for this optimizer step; the learner sets it
        # for the LAST micro-batch's backward only, so that the gradient exchange can start under the backward pass
        self.grad_ready_hook = None
        self.main_grad: torch.Tensor | None = None  # fp32 flat gradient (fused path)
        self.g: dict[str, torch.Tensor] = {}
        self.inv_freq = ref.rope_inv_freq(spec.head_dim, spec.rope_theta, spec.rope_scaling, device=self.device)
        if ops == "ref":
            self.flat.requires_grad_(True)
        # autograd anchor for the fused path: the custom Functions take it as an input so that
        # loss.backward() reaches their manual backward
        self._anchor = torch.zeros(1, device=self.device, requires_grad=True) if ops == "fused" else None

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def init_weights(self, seed: int = 0, init: str = "normal", std: float = 0.02) -> None:
        """Random init: N(0, 0.02) matrices, unit norm weights (HF ``_init_weights`` convention)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        views = self.layout.views(self.flat)
        self.flat.zero_()
        for name, v in views.items():
            e = self.layout.entries[name]
            if name.endswith("norm"):
                v.fill_(1.0)
            elif name.endswith("bqkv"):
                v.zero_()
            elif name.endswith("gdn_A_log"):     # decay rates A ~ U(0, 16), stored as log A
                v.copy_(torch.log(torch.rand(v.shape, generator=g) * 16.0 + 1e-3).to(v.dtype))
            elif name.endswith("gdn_dt_bias"):   # softplus^-1 of a step size drawn log-uniformly from [1e-3, 1e-1]
                dt = torch.exp(torch.rand(v.shape, generator=g) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
                v.copy_((dt + torch.log(-torch.expm1(-dt))).to(v.dtype))
            elif name.endswith("gdn_conv"):      # depthwise taps: U(-1/sqrt(taps), 1/sqrt(taps))
                bound = v.shape[1] ** -0.5
                v.copy_(((torch.rand(v.shape, generator=g) * 2 - 1) * bound).to(v.dtype))
            elif init == "normal":
                if v.device.type == "cuda":
                    # generate on device in chunks: 8B parameters on the host would take minutes
                    gg = torch.Generator(device=v.device).manual_seed(seed * 1000003 + e.offset % 1000003)
                    flatv = v.view(-1)
                    step = 1 << 26
                    for s in range(0, flatv.numel(), step):
                        n = min(step, flatv.numel() - s)
                        flatv[s:s + n].copy_(torch.randn(n, device=v.device, generator=gg, dtype=torch.float32) * std)
                else:
                    v.copy_((torch.randn(v.shape, generator=g, dtype=torch.float32) * std).to(v.dtype))
        # tied output head shares the embedding; nothing else to do

    def vocab_parallel_head(self) -> bool:
        """True when the log-prob head is computed vocabulary-parallel over a tensor-parallel group (untied head only: a tied
        embedding also receives the lookup's gradient, which is the same on every rank and must not be summed)."""
        return (self.tp is not None and getattr(self.tp, "vocab_parallel", False) and self.tp.world > 1
                and not self.spec.tie_word_embeddings and "lm_head" in self.layout.entries)

    def lm_head_weight(self) -> torch.Tensor:
        return self.p["embed"] if self.spec.tie_word_embeddings or "lm_head" not in self.p else self.p["lm_head"]

    def ensure_main_grad(self) -> torch.Tensor:
        if self.zero3 is not None:
            return None  # gradients live in the sharded state's workspaces
        if self.main_grad is None:
            self.main_grad = torch.zeros(self.flat.numel(), dtype=torch.float32, device=self.device)
            self.g = self.layout.views(self.main_grad)
        return self.main_grad

    def bind_main_grad(self, buf: torch.Tensor) -> None:
        """Use an externally owned fp32 gradient buffer (e.g. a symmetric-memory bucket)."""
        if buf.numel() < self.layout.total or buf.dtype != torch.float32:
            raise ValueError("main_grad must be fp32 and at least the layout's size")
        self.main_grad = buf
        self.g = self.layout.views(buf)

    def rebind(self, flat: torch.Tensor) -> None:
        """Point the model at another flat buffer of the same layout (no copy)."""
        self.flat = flat
        self.p = self.layout.views(flat)
        if self.ops == "ref":
            self.flat.requires_grad_(True)

    def logit_workspace(self, rows: int, vocab: int) -> torch.Tensor:
        """One reused ``[rows, vocab]`` buffer (bf16 on the kernel path) for the chunked lm_head (allocated on first use)."""
        ws = getattr(self, "_logit_ws", None)
        if ws is None or ws.shape[0] < rows or ws.shape[1] != vocab:
            ws = self._logit_ws = torch.empty(rows, vocab, dtype=self.dtype, device=self.device)
        return ws

    def layer_grad_range(self, i: int) -> tuple[int, int]:
        """Flat-buffer range of layer ``i``'s matrices (wqkv, wo, w_gate_up, w_down are adjacent in the layout)."""
        e = self.layout.entries
        lo = e[f"l{i}.wqkv"].offset
        if i + 1 < self.spec.num_layers:
            return lo, e[f"l{i + 1}.wqkv"].offset
        return lo, (e["lm_head"].offset if "lm_head" in e else self.layout.decay_end)

    def grad_flat(self) -> torch.Tensor | None:
        """Flat gradient: fp32 ``main_grad`` (fused) or autograd's ``flat.grad`` (ref)."""
        return self.main_grad if self.ops == "fused" else self.flat.grad

    def zero_grad(self) -> None:
        if self.ops == "fused":
            if self.main_grad is not None:
                self.main_grad.zero_()
        else:
            self.flat.grad = None

    # ------------------------------------------------------------------ public API
    def token_logprobs(self, input_ids, position_ids, cu_seqlens, labels, temperature: float = 1.0,
                       want_entropy: bool = False):
        """log p(labels[t] | prefix) for every packed position (0 where ``labels < 0``).

        ``labels`` is already shifted: ``labels[t]`` is the token that follows position ``t``.
        Returns ``(logp [T] fp32, entropy [T] fp32 | None)``; ``logp`` is differentiable.
        """
        if self.ops == "ref":
            h = self._ref_hidden(input_ids, position_ids, cu_seqlens)
            if self.vocab_parallel_head():
                v0, v1 = self.tp.vocab_range(self.spec.vocab_size)
                logits = ref.linear(self.tp.enter(h), self.lm_head_weight_ref()[v0:v1])  # my vocabulary rows; dh is summed over the group
                return self.tp.vocab_parallel_logprobs(logits, labels, v0, temperature, want_entropy)
            logits = ref.linear(h, self.lm_head_weight_ref())
            return ref.token_logprobs(logits, labels, temperature, with_entropy=want_entropy)
        keep = torch.is_grad_enabled()
        logp, ent = _FusedLogprobFn.apply(self, input_ids, position_ids, cu_seqlens, labels, temperature, want_entropy,
                                          keep, self._anchor if keep else None)
        return logp, (ent if want_entropy else None)

    def hidden_states(self, input_ids, position_ids, cu_seqlens) -> torch.Tensor:
        """Final-norm hidden states [T, D] (differentiable); used by the reward-model head."""
        if self.ops == "ref":
            return self._ref_hidden(input_ids, position_ids, cu_seqlens)
        keep = torch.is_grad_enabled()
        return _FusedHiddenFn.apply(self, input_ids, position_ids, cu_seqlens, keep, self._anchor if keep else None)

    @torch.no_grad()
    def logits(self, input_ids, position_ids, cu_seqlens) -> torch.Tensor:
        """Full logits [T, V] (inference / tests only; training never materialises fp32 logits)."""
        if self.ops == "ref":
            return ref.linear(self._ref_hidden(input_ids, position_ids, cu_seqlens), self.lm_head_weight_ref())
        h, _ = self._fused_forward_hidden(input_ids, position_ids, cu_seqlens, keep=False)
        if self.zero3 is not None:
            self.zero3.head()
        return self.kernels.gemm(h, self.lm_head_weight())

    # ------------------------------------------------------------------ ref path
    def _ref_params(self) -> dict:
        """Parameter tensors of the autograd path: views of the flat leaf, or differentiable overrides
        installed by an adapter (``param_override``)."""
        return self.param_override if getattr(self, "param_override", None) is not None else self.layout.views(self.flat)

    def lm_head_weight_ref(self) -> torch.Tensor:
        v = self._ref_params()
        return v["embed"] if self.spec.tie_word_embeddings or "lm_head" not in v else v["lm_head"]

    def _ref_hidden(self, input_ids, position_ids, cu_seqlens) -> torch.Tensor:
        s = self.spec
        v = self._ref_params()  # autograd views of the single leaf
        x = v["embed"][input_ids]
        self._router_logits = [] if s.num_experts else None
        for i in range(s.num_layers):
            x = self._ref_layer(x, v, i, position_ids, cu_seqlens)
        # mixture of experts: the load-balancing loss of THIS forward (a differentiable scalar), for the trainer to add
        self.aux_loss = load_balancing_loss(self._router_logits, s.num_experts, s.num_experts_per_tok) if s.num_experts else None
        return ref.rmsnorm(x, v["final_norm"], s.rms_norm_eps)

    def ref_mlp(self, n2, v, i):
        """The layer's feed-forward on normed input ``n2``: one SwiGLU MLP, or (mixture of experts) the router's top-k experts,
        each token's expert outputs weighted by the router's softmax probabilities."""
        s = self.spec
        if not s.num_experts:
            return ref.linear(ref.swiglu(ref.linear(n2, v[f"l{i}.w_gate_up"])), v[f"l{i}.w_down"])
        E, F, D, k = s.num_experts, s.intermediate_size, s.hidden_size, s.num_experts_per_tok
        logits = ref.linear(n2, v[f"l{i}.router"])                      # [T, E]
        if getattr(self, "_router_logits", None) is not None:
            self._router_logits.append(logits)
        probs = torch.softmax(logits.float(), dim=-1)
        top_w, top_e = probs.topk(k, dim=-1)
        if s.norm_topk_prob:
            top_w = top_w / top_w.sum(-1, keepdim=True)
        top_w = top_w.to(n2.dtype)
        w_gu = v[f"l{i}.w_gate_up"].view(E, 2 * F, D)
        w_dn = v[f"l{i}.w_down"].view(E, D, F)
        out = torch.zeros_like(n2)
        for e in range(E):
            tok, slot = torch.where(top_e == e)
            if tok.numel() == 0:
                continue
            y = ref.linear(ref.swiglu(ref.linear(n2[tok], w_gu[e])), w_dn[e])
            out = out.index_add(0, tok, y * top_w[tok, slot, None])
        return out

    def ref_qkv(self, n1, v, i):
        """QKV projection of the PyTorch path with the family's extras: Qwen2-style bias, Qwen3 / OLMo-2 per-head RMSNorm of
        q and k (before RoPE)."""
        s = self.spec
        qkv = ref.linear(n1, v[f"l{i}.wqkv"])
        if s.attention_bias:
            qkv = qkv + v[f"l{i}.bqkv"]
        if s.qk_norm and s.qk_norm_full:  # OLMo-2: one norm over all heads of q, one over all heads of k
            q = ref.rmsnorm(qkv[:, : s.q_dim], v[f"l{i}.q_norm"], s.rms_norm_eps)
            k = ref.rmsnorm(qkv[:, s.q_dim : s.q_dim + s.kv_dim], v[f"l{i}.k_norm"], s.rms_norm_eps)
            qkv = torch.cat([q, k, qkv[:, s.q_dim + s.kv_dim :]], dim=1)
        elif s.qk_norm:
            T = qkv.shape[0]
            heads = qkv.view(T, s.num_heads + 2 * s.num_kv_heads, s.head_dim)
            q = ref.rmsnorm(heads[:, : s.num_heads], v[f"l{i}.q_norm"], s.rms_norm_eps)
            k = ref.rmsnorm(heads[:, s.num_heads : s.num_heads + s.num_kv_heads], v[f"l{i}.k_norm"], s.rms_norm_eps)
            qkv = torch.cat([q, k, heads[:, s.num_heads + s.num_kv_heads :]], dim=1).reshape(T, -1)
        return qkv

    def _ref_layer(self, x, v, i, position_ids, cu_seqlens):
        s = self.spec
        tp = self.tp
        rope = (lambda qkv: ref.rope(qkv, position_ids, self.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim)) if s.use_rope else (lambda qkv: qkv)
        if s.is_gdn(i):  # hybrid models: a pre-norm block whose sequence mixer is a gated DeltaNet
            if tp is not None:
                raise NotImplementedError("tensor parallelism is not built for gated-DeltaNet layers")
            from .gdn import gdn_mixer

            x = x + gdn_mixer(ref.rmsnorm(x, v[f"l{i}.attn_norm"], s.rms_norm_eps), v, i, s, cu_seqlens)
            return x + self.ref_mlp(ref.rmsnorm(x, v[f"l{i}.mlp_norm"], s.rms_norm_eps), v, i)
        if s.post_norm:  # OLMo-2 / OLMo-3: the sub-layer reads the stream as it is, its OUTPUT is normed before the residual add
            if tp is not None:
                raise NotImplementedError("tensor parallelism is not built for post-norm blocks")
            qkv = rope(self.ref_qkv(x, v, i))
            attn = ref.attention_varlen(qkv, cu_seqlens, s.num_heads, s.num_kv_heads, s.head_dim, s.attn_scale, allow_sdpa=True, window=s.window(i))
            x = x + ref.rmsnorm(ref.linear(attn, v[f"l{i}.wo"]), v[f"l{i}.attn_norm"], s.rms_norm_eps)
            return x + ref.rmsnorm(self.ref_mlp(x, v, i), v[f"l{i}.mlp_norm"], s.rms_norm_eps)
        n1 = ref.rmsnorm(x, v[f"l{i}.attn_norm"], s.rms_norm_eps)
        if tp is not None:
            n1 = tp.enter(n1)
        qkv = rope(self.ref_qkv(n1, v, i))
        attn = ref.attention_varlen(qkv, cu_seqlens, s.num_heads, s.num_kv_heads, s.head_dim, s.attn_scale, allow_sdpa=bool(s.num_experts), window=s.window(i))
        o = ref.linear(attn, v[f"l{i}.wo"])
        x = x + (tp.sum_partials(o) if tp is not None else o)
        n2 = ref.rmsnorm(x, v[f"l{i}.mlp_norm"], s.rms_norm_eps)
        if tp is not None:
            n2 = tp.enter(n2)
        if s.num_experts and tp is not None:
            raise NotImplementedError("tensor parallelism is not built for mixture-of-experts layers")
        d = self.ref_mlp(n2, v, i)
        return x + (tp.sum_partials(d) if tp is not None else d)

    # ------------------------------------------------------------------ fused path
    def _fused_forward_hidden(self, input_ids, position_ids, cu_seqlens, keep: bool):
        """Runs the stack; returns final-norm hidden states.  ``keep`` stores what backward needs."""
        f = self.kernels
        s, p = self.spec, self.p
        # sliding-window layers: while every document fits in the window the attention kernel is exact; for longer documents those
        # layers go through the windowed library attention (``attn_fwd_window``), the only part of the step that is not a kernel of
        # this package
        self._max_doc = int((cu_seqlens[1:] - cu_seqlens[:-1]).max()) if (s.min_window and cu_seqlens.numel() > 1) else 0
        if s.min_window and self._max_doc > s.min_window and self.sp is not None:
            raise NotImplementedError(f"documents longer than the model's sliding window ({s.min_window}) together with sequence parallelism")
        pos = position_ids.to(torch.int32)
        cu = cu_seqlens.to(torch.int32)
        scale = s.attn_scale
        stash: list[_LayerStash] = []
        self._rope_tab = f.rope_table(pos, self.inv_freq, s.head_dim)  # cos/sin once per packed batch, for every layer and the backward
        if self.sp is not None:
            # sequence parallel: this rank embeds and projects its contiguous chunk of the packed tokens
            lo, hi = self.sp.local_tokens(input_ids.numel())
            input_ids = input_ids[lo:hi]
        z = self.zero3
        if z is not None:
            z.fwd_begin()
        stream = f.embedding_fwd(p["embed"], input_ids)
        self._routing = [] if s.num_experts else None   # (logits, chosen experts) of every layer, for the load-balancing loss
        delta = None  # pending residual contribution, added inside the next RMSNorm
        for i in range(s.num_layers):
            if z is not None:
                z.layer_fwd(i)  # layer i's parameters are in their workspace; the next layer's gather is under way
            if s.post_norm:
                st = self._post_norm_layer(i, stream, pos, cu)
                stream = st.h_mid + st.n2   # n2 holds norm(d) until here
                st.n2 = None
                if keep:
                    stash.append(_LayerStash(st.h_in, None, None, None, None, None, None, None) if self.gradient_checkpointing else st)
                continue
            n1, h_in, rstd1 = f.rmsnorm_fwd(delta if delta is not None else stream, p[f"l{i}.attn_norm"], s.rms_norm_eps,
                                            res=stream if delta is not None else None)
            qkv, attn, lse, attn_tok = self._attention_block(i, n1, pos, cu)
            o = f.gemm(attn_tok if attn_tok is not None else attn, p[f"l{i}.wo"])
            if self.tp is not None:
                self.tp.all_reduce_(o)      # row-parallel projection: sum of the ranks' partials
            n2, h_mid, rstd2 = f.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], s.rms_norm_eps, res=h_in)
            del o
            moe = None
            if s.num_experts:
                delta, moe = self._moe_forward(i, n2)
                gate_up, act = moe.gu, None
            else:
                gate_up = f.gemm(n2, p[f"l{i}.w_gate_up"])
                act = f.swiglu_fwd(gate_up)
                delta = f.gemm(act, p[f"l{i}.w_down"])
            if self.tp is not None:
                self.tp.all_reduce_(delta)
            keep_cheap = keep and self.keep_cheap_activations and not self.gradient_checkpointing
            if not keep_cheap:
                n1 = n2 = act = None
            stream = h_mid
            if keep:
                if self.gradient_checkpointing:
                    stash.append(_LayerStash(h_in, None, None, None, None, None, None, None))
                else:
                    stash.append(_LayerStash(h_in, rstd1, qkv, attn, lse, h_mid, rstd2, gate_up, attn_tok, self._last_qk, n1, n2, act, moe=moe))
            del n1, n2, act, moe
        if delta is None:   # post-norm blocks leave no pending contribution: the stream is complete
            nf, h_last, rstd_f = f.rmsnorm_fwd(stream, p["final_norm"], s.rms_norm_eps)
        else:
            nf, h_last, rstd_f = f.rmsnorm_fwd(delta, p["final_norm"], s.rms_norm_eps, res=stream)
        state = None
        if keep:
            state = {"stash": stash, "final": (h_last, rstd_f), "ids": input_ids, "pos": pos, "cu": cu, "rope_tab": self._rope_tab,
                     "max_doc": self._max_doc}
        if s.num_experts:
            # the load-balancing loss of this forward (a plain number here: the backward adds ``aux_loss_coef`` times its gradient,
            # which reaches the routers through the mean probability of every expert, E / N * sum_k f[k, e] per softmax entry)
            logits = torch.cat([lg for lg, _ in self._routing])
            sel = torch.cat([te for _, te in self._routing])
            self.aux_loss = load_balancing_loss([logits], s.num_experts, s.num_experts_per_tok).detach()
            if keep:
                share = torch.nn.functional.one_hot(sel, s.num_experts).float().mean(0).sum(0)   # sum over the k ranks of f[k, e]
                state["aux_dprobs"] = share * (s.num_experts / logits.shape[0])
            self._routing = None
        return nf, state

    def _post_norm_layer(self, i: int, x, pos, cu) -> _LayerStash:
        """Forward of an OLMo-2 / OLMo-3 block: ``h = x + norm(attn(x))``, ``out = h + norm(mlp(h))`` - the sub-layers read the
        stream as it is and their OUTPUT is normalised.  Returns the stash of the layer with ``n2`` holding ``norm(mlp(h))``
        (the caller adds it to ``h_mid`` to form the layer's output)."""
        f = self.kernels
        s, p = self.spec, self.p
        if self.tp is not None:
            raise NotImplementedError("tensor parallelism is not built for post-norm blocks")
        qkv, attn, lse, attn_tok = self._attention_block(i, x, pos, cu)
        o = f.gemm(attn_tok if attn_tok is not None else attn, p[f"l{i}.wo"])
        a_n, _, rstd1 = f.rmsnorm_fwd(o, p[f"l{i}.attn_norm"], s.rms_norm_eps)
        h_mid = x + a_n
        del a_n
        gate_up = f.gemm(h_mid, p[f"l{i}.w_gate_up"])
        act = f.swiglu_fwd(gate_up)
        d = f.gemm(act, p[f"l{i}.w_down"])
        m_n, _, rstd2 = f.rmsnorm_fwd(d, p[f"l{i}.mlp_norm"], s.rms_norm_eps)
        keep_act = self.keep_cheap_activations and not self.gradient_checkpointing
        return _LayerStash(x, rstd1, qkv, attn, lse, h_mid, rstd2, gate_up, attn_tok, self._last_qk, None, m_n, act if keep_act else None, o, d)

    def _post_norm_layer_bwd(self, i: int, st: _LayerStash, d_out, pos, cu, wgrad_mode):
        """Backward of ``_post_norm_layer``: gradient of the layer's output in, gradient of its input out."""
        f = self.kernels
        s, p, g, sp = self.spec, self.p, self.g, self.sp
        scale = s.attn_scale
        # ---- out = h_mid + norm(d),  d = down(swiglu(gate_up(h_mid)))
        d_d = f.rmsnorm_bwd(st.d, p[f"l{i}.mlp_norm"], st.rstd2, d_out, None, g[f"l{i}.mlp_norm"])
        st.d = None
        act = st.act if st.act is not None else f.swiglu_fwd(st.gate_up)
        st.act = None
        f.gemm(d_d, act, g[f"l{i}.w_down"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
        d_act = f.gemm(d_d, p[f"l{i}.w_down"], b_mn=True)
        del act, d_d
        dgu = f.swiglu_bwd_(st.gate_up, d_act)
        del d_act
        f.gemm(dgu, st.h_mid, g[f"l{i}.w_gate_up"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
        d_mid = f.gemm(dgu, p[f"l{i}.w_gate_up"], b_mn=True)
        del dgu
        d_mid.add_(d_out)
        del d_out
        # ---- h_mid = x + norm(o),  o = wo(attn(rope(wqkv(x))))
        d_o = f.rmsnorm_bwd(st.o, p[f"l{i}.attn_norm"], st.rstd1, d_mid, None, g[f"l{i}.attn_norm"])
        st.o = None
        f.gemm(d_o, st.attn_tok if sp is not None else st.attn, g[f"l{i}.wo"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
        if sp is None:
            d_attn = f.gemm(d_o, p[f"l{i}.wo"], b_mn=True)
            dqkv = self._attn_bwd(i, st, d_attn, cu, scale)
            del d_attn
            f.rope_(dqkv, pos, self.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim, backward=True, table=self._rope_tab)
            self._qkv_bias_and_norm_bwd_(dqkv, i, st.qk)
        else:
            d_attn = sp.d_attn_project(d_o, p[f"l{i}.wo"], pos.numel())
            dqkv_heads = f.attn_bwd(st.qkv, st.attn, d_attn, st.lse, cu, sp.hq_l, sp.hk_l, s.head_dim, scale)
            f.rope_(dqkv_heads, pos, self.inv_freq, sp.hq_l, sp.hk_l, s.head_dim, backward=True, table=self._rope_tab)
            self._qkv_bias_and_norm_bwd_(dqkv_heads, i, st.qk, sp.hq_l, sp.hk_l, bias=False)
            dqkv = sp.dqkv_exchange(dqkv_heads)
            if s.attention_bias:
                g[f"l{i}.bqkv"].add_(dqkv.float().sum(0))
        del d_o
        f.gemm(dqkv, st.h_in, g[f"l{i}.wqkv"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
        d_x = f.gemm(dqkv, p[f"l{i}.wqkv"], b_mn=True)
        d_x.add_(d_mid)
        return d_x

    def _moe_forward(self, i: int, n2):
        """Mixture-of-experts feed-forward of layer ``i`` on normed input ``n2`` [T, D]: the router's k best experts per token,
        each a SwiGLU MLP, outputs weighted by the router's softmax probabilities.  The (token, expert) assignments are sorted by
        expert, so that an expert's tokens are consecutive rows and its two projections are one GEMM each over that row range
        (the stacked expert weights are row slices of one flat-buffer entry).  Returns ``(delta [T, D], stash)``."""
        f = self.kernels
        s, p = self.spec, self.p
        if self.tp is not None or self.sp is not None:
            raise NotImplementedError("tensor and sequence parallelism are not built for mixture-of-experts layers")
        E, F, D, k = s.num_experts, s.intermediate_size, s.hidden_size, s.num_experts_per_tok
        T = n2.shape[0]
        logits = n2 @ p[f"l{i}.router"].t()   # [T, E]: small, and E need not suit the GEMM kernel's tile and stride rules
        with torch.enable_grad():   # [T, E]-sized: softmax, top-k and renormalisation are left to autograd
            lg = logits.detach().float().requires_grad_(True)
            probs = torch.softmax(lg, dim=-1)
            top_w, top_e = probs.topk(k, dim=-1)
            if s.norm_topk_prob:
                top_w = top_w / top_w.sum(-1, keepdim=True)
        if self._routing is not None:
            self._routing.append((lg.detach(), top_e))
        flat_e = top_e.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=E).tolist()   # the one host synchronisation of the layer
        tok, slot = order // k, order % k
        x = n2[tok]
        w_gu, w_dn = p[f"l{i}.w_gate_up"], p[f"l{i}.w_down"]
        gu = torch.empty(T * k, 2 * F, dtype=n2.dtype, device=n2.device)
        r = 0
        for e, n in enumerate(counts):
            if n:
                f.gemm(x[r:r + n], w_gu[e * 2 * F:(e + 1) * 2 * F], gu[r:r + n])
            r += n
        act = f.swiglu_fwd(gu)
        y = torch.empty(T * k, D, dtype=n2.dtype, device=n2.device)
        r = 0
        for e, n in enumerate(counts):
            if n:
                f.gemm(act[r:r + n], w_dn[e * D:(e + 1) * D], y[r:r + n])
            r += n
        tw = top_w.detach().to(n2.dtype)[tok, slot]
        delta = torch.zeros(T, D, dtype=torch.float32, device=n2.device).index_add_(0, tok, (y * tw[:, None]).float()).to(n2.dtype)
        return delta, _MoEStash(tok, slot, counts, gu, y, lg, probs, top_w)

    def _moe_backward(self, i: int, m: _MoEStash, d_delta, n2, aux_dprobs, wgrad_mode):
        """Backward of ``_moe_forward``: gradient of its output in, gradient of ``n2`` out; expert and router weight gradients
        are accumulated into the flat gradient buffer."""
        f = self.kernels
        s, p, g = self.spec, self.p, self.g
        E, F, D, k = s.num_experts, s.intermediate_size, s.hidden_size, s.num_experts_per_tok
        T = n2.shape[0]
        tw = m.top_w.detach().to(n2.dtype)[m.tok, m.slot]
        dwy = d_delta[m.tok]
        d_tw = torch.zeros(T, k, dtype=torch.float32, device=n2.device)
        d_tw[m.tok, m.slot] = (dwy.float() * m.y.float()).sum(-1)
        dy = dwy * tw[:, None]
        del dwy
        act = f.swiglu_fwd(m.gu)
        w_gu, w_dn = p[f"l{i}.w_gate_up"], p[f"l{i}.w_down"]
        g_gu, g_dn = g[f"l{i}.w_gate_up"], g[f"l{i}.w_down"]
        d_act = torch.empty_like(act)
        r = 0
        for e, n in enumerate(m.counts):
            if n:
                f.gemm(dy[r:r + n], act[r:r + n], g_dn[e * D:(e + 1) * D], a_mn=True, b_mn=True, out_mode=wgrad_mode)
                f.gemm(dy[r:r + n], w_dn[e * D:(e + 1) * D], d_act[r:r + n], b_mn=True)
            r += n
        del act, dy
        dgu = f.swiglu_bwd_(m.gu, d_act)
        del d_act
        x = n2[m.tok]
        dx = torch.empty_like(x)
        r = 0
        for e, n in enumerate(m.counts):
            if n:
                f.gemm(dgu[r:r + n], x[r:r + n], g_gu[e * 2 * F:(e + 1) * 2 * F], a_mn=True, b_mn=True, out_mode=wgrad_mode)
                f.gemm(dgu[r:r + n], w_gu[e * 2 * F:(e + 1) * 2 * F], dx[r:r + n], b_mn=True)
            r += n
        d_n2 = torch.zeros(T, D, dtype=torch.float32, device=n2.device).index_add_(0, m.tok, dx.float())
        # routing weights (and the load-balancing loss, when the trainer adds it) back to the router logits, then to the router
        with torch.enable_grad():   # the backward pass runs with gradient recording off
            objective = (m.top_w * d_tw).sum()
            if self.aux_loss_coef and aux_dprobs is not None:
                objective = objective + self.aux_loss_coef * (m.probs * aux_dprobs).sum()
            (d_lg,) = torch.autograd.grad(objective, m.lg)
        d_logits = d_lg.to(n2.dtype)
        g[f"l{i}.router"].add_((d_logits.t() @ n2).float())
        d_n2 += (d_logits @ p[f"l{i}.router"]).float()
        return d_n2.to(n2.dtype)

    def _attn_bwd(self, i: int, st: _LayerStash, d_attn, cu, scale):
        """Gradient with respect to the post-RoPE qkv of layer ``i`` (one rank holds all heads)."""
        f, s = self.kernels, self.spec
        if st.lse is None:   # the forward of this layer went through the windowed library attention
            return f.attn_bwd_window(st.qkv, d_attn, cu, s.num_heads, s.num_kv_heads, s.head_dim, scale, s.window(i), self._max_doc)
        return f.attn_bwd(st.qkv, st.attn, d_attn, st.lse, cu, s.num_heads, s.num_kv_heads, s.head_dim, scale)

    def _attention_block(self, i: int, n1, pos, cu):
        """QKV projection, RoPE and attention of layer ``i``.  Returns ``(qkv, attn, lse, attn_tok)``; with sequence
        parallelism ``qkv``/``attn`` cover all tokens for this rank's heads and ``attn_tok`` this rank's tokens for all
        heads (else ``attn_tok`` is None)."""
        f = self.kernels
        s, p, sp = self.spec, self.p, self.sp
        scale = s.attn_scale
        if sp is None:
            qkv = f.gemm(n1, p[f"l{i}.wqkv"])
            self._last_qk = self.qkv_bias_and_norm_(qkv, i)
            f.rope_(qkv, pos, self.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim, table=self._rope_tab)
            w = s.window(i)
            if w and self._max_doc > w:   # lse None marks the layer for the windowed backward
                return qkv, f.attn_fwd_window(qkv, cu, s.num_heads, s.num_kv_heads, s.head_dim, scale, w, self._max_doc), None, None
            attn, lse = f.attn_fwd(qkv, cu, s.num_heads, s.num_kv_heads, s.head_dim, scale)
            return qkv, attn, lse, None
        qkv = sp.qkv_project(i, n1, p[f"l{i}.wqkv"], pos.numel())
        # after the exchange a row is [q | k | v] of THIS rank's heads: same structure, fewer heads
        self._last_qk = self.qkv_bias_and_norm_(qkv, i, sp.hq_l, sp.hk_l, cols=sp.local_cols_index)
        f.rope_(qkv, pos, self.inv_freq, sp.hq_l, sp.hk_l, s.head_dim, table=self._rope_tab)
        attn, lse = f.attn_fwd(qkv, cu, sp.hq_l, sp.hk_l, s.head_dim, scale)
        return qkv, attn, lse, sp.attn_exchange(i, attn)

    def qkv_bias_and_norm_(self, qkv: torch.Tensor, i: int, hq: int | None = None, hk: int | None = None, cols: torch.Tensor | None = None):
        """Qwen2-style q/k/v bias and Qwen3 / OLMo-2 style per-head RMSNorm of q and k, in place on the fused projection
        output (before RoPE).  Returns what the backward needs (``None`` when the model has neither).  ``hq`` / ``hk``:
        query / key heads in a row of ``qkv`` (sequence parallelism: this rank's heads only, ``cols`` then indexes their
        columns in the full fused width for the bias)."""
        f = self.kernels
        s, p = self.spec, self.p
        hq = s.num_heads if hq is None else hq
        hk = s.num_kv_heads if hk is None else hk
        if s.attention_bias:
            qkv.add_(p[f"l{i}.bqkv"] if cols is None else p[f"l{i}.bqkv"][cols])
        if not s.qk_norm:
            return None
        T = qkv.shape[0]
        out = []
        if s.qk_norm_full and (hq != s.num_heads or hk != s.num_kv_heads):
            # sequence parallelism: this rank holds some heads of every token, the norm runs over all heads.  Each rank sums the
            # squares of its heads, one [T]-sized all-reduce over the group completes the statistic, and the rank scales its own
            # columns with its slice of the weight
            import torch.distributed as dist

            sp = self.sp
            for lo, heads, name, width in ((0, hq, "q_norm", s.q_dim), (hq * s.head_dim, hk, "k_norm", s.kv_dim)):
                n = heads * s.head_dim
                pre = qkv[:, lo:lo + n].contiguous()
                ss = pre.float().pow(2).sum(-1)
                dist.all_reduce(ss, group=sp.group)
                rstd = torch.rsqrt(ss / width + s.rms_norm_eps)
                w = p[f"l{i}.{name}"][sp.rank * n:(sp.rank + 1) * n]
                qkv[:, lo:lo + n].copy_(w * (pre.float() * rstd[:, None]).to(qkv.dtype))
                out += [pre, rstd]
            return tuple(out)
        rows = (lambda heads: T) if s.qk_norm_full else (lambda heads: T * heads)   # one norm per row, or one per head
        for lo, heads, name in ((0, hq, "q_norm"), (hq * s.head_dim, hk, "k_norm")):
            pre = qkv[:, lo:lo + heads * s.head_dim].contiguous().view(rows(heads), -1)
            y, _, rstd = f.rmsnorm_fwd(pre, p[f"l{i}.{name}"], s.rms_norm_eps)
            qkv[:, lo:lo + heads * s.head_dim].copy_(y.view(T, heads * s.head_dim))
            out += [pre, rstd]
        return tuple(out)

    def _qkv_bias_and_norm_bwd_(self, dqkv: torch.Tensor, i: int, qk, hq: int | None = None, hk: int | None = None, bias: bool = True) -> None:
        """Backward of ``qkv_bias_and_norm_`` in place on ``dqkv`` (after the RoPE backward); accumulates the norm and
        bias gradients.  ``bias=False``: the caller adds the bias gradient itself (sequence parallelism does it after the
        exchange, on full-width rows)."""
        f = self.kernels
        s, g, p = self.spec, self.g, self.p
        hq = s.num_heads if hq is None else hq
        hk = s.num_kv_heads if hk is None else hk
        T = dqkv.shape[0]
        if qk is not None and s.qk_norm_full and (hq != s.num_heads or hk != s.num_kv_heads):
            import torch.distributed as dist

            sp = self.sp
            for (lo, heads, name, width), pre, rstd in (((0, hq, "q_norm", s.q_dim), qk[0], qk[1]), ((hq * s.head_dim, hk, "k_norm", s.kv_dim), qk[2], qk[3])):
                n = heads * s.head_dim
                w = p[f"l{i}.{name}"][sp.rank * n:(sp.rank + 1) * n].float()
                dy = dqkv[:, lo:lo + n].float()
                xhat = pre.float() * rstd[:, None]
                g[f"l{i}.{name}"][sp.rank * n:(sp.rank + 1) * n].add_((dy * xhat).sum(0))
                dxhat = dy * w
                dot = (dxhat * xhat).sum(-1)
                dist.all_reduce(dot, group=sp.group)   # the mean in the norm's derivative runs over all heads too
                dqkv[:, lo:lo + n].copy_((rstd[:, None] * (dxhat - xhat * (dot / width)[:, None])).to(dqkv.dtype))
            qk = None
        if qk is not None:
            for (lo, heads, name), pre, rstd in (((0, hq, "q_norm"), qk[0], qk[1]), ((hq * s.head_dim, hk, "k_norm"), qk[2], qk[3])):
                dy = dqkv[:, lo:lo + heads * s.head_dim].contiguous().view(pre.shape)
                dx = f.rmsnorm_bwd(pre, p[f"l{i}.{name}"], rstd, dy, None, g[f"l{i}.{name}"])
                dqkv[:, lo:lo + heads * s.head_dim].copy_(dx.view(T, heads * s.head_dim))
        if s.attention_bias and bias:
            g[f"l{i}.bqkv"].add_(dqkv.float().sum(0))

    def _recompute_layer(self, i: int, st: _LayerStash, pos, cu) -> _LayerStash:
        """Gradient checkpointing: rebuild a layer's activations from its input stream."""
        f = self.kernels
        s, p = self.spec, self.p
        if s.post_norm:
            st = self._post_norm_layer(i, st.h_in, pos, cu)
            st.n2 = None
            return st
        n1, _, rstd1 = f.rmsnorm_fwd(st.h_in, p[f"l{i}.attn_norm"], s.rms_norm_eps)
        qkv, attn, lse, attn_tok = self._attention_block(i, n1, pos, cu)
        o = f.gemm(attn_tok if attn_tok is not None else attn, p[f"l{i}.wo"])
        if self.tp is not None:
            self.tp.all_reduce_(o)
        n2, h_mid, rstd2 = f.rmsnorm_fwd(o, p[f"l{i}.mlp_norm"], s.rms_norm_eps, res=st.h_in)
        if s.num_experts:
            moe = self._moe_forward(i, n2)[1]
            return _LayerStash(st.h_in, rstd1, qkv, attn, lse, h_mid, rstd2, moe.gu, attn_tok, self._last_qk, moe=moe)
        gate_up = f.gemm(n2, p[f"l{i}.w_gate_up"])
        return _LayerStash(st.h_in, rstd1, qkv, attn, lse, h_mid, rstd2, gate_up, attn_tok, self._last_qk)

    def _fused_backward_hidden(self, state: dict, d_nf: torch.Tensor) -> None:
        """Backward from d(final-norm hidden) to the embedding; accumulates into ``main_grad``."""
        f = self.kernels
        s, p = self.spec, self.p
        self.ensure_main_grad()
        g = self.g
        h_last, rstd_f = state["final"]
        stash, pos, cu = state["stash"], state["pos"], state["cu"]
        self._rope_tab = state["rope_tab"]
        self._max_doc = state["max_doc"]   # another forward pass may have run since this one
        # final norm: h_last = stream + delta ; both get the same gradient
        d_stream = f.rmsnorm_bwd(h_last, p["final_norm"], rstd_f, d_nf, None, g["final_norm"])
        del d_nf
        scale = s.attn_scale
        z = self.zero3
        # sharded parameters: a layer's gradient workspace is written once per micro-batch and reduced right away, so the
        # weight-gradient GEMMs overwrite it (no zeroing pass, no read in the epilogue); otherwise they accumulate
        wgrad_mode = f.OUT_F32 if z is not None else f.OUT_F32_ACC
        for i in reversed(range(s.num_layers)):
            if z is not None:
                z.layer_bwd(i)
            st = stash[i]
            if st.qkv is None:
                st = self._recompute_layer(i, st, pos, cu)
            stash[i] = None
            if s.post_norm:
                d_stream = self._post_norm_layer_bwd(i, st, d_stream, pos, cu, wgrad_mode)
                if z is not None:
                    z.layer_bwd_done(i)
                elif self.grad_ready_hook is not None:
                    self.grad_ready_hook(*self.layer_grad_range(i))
                continue
            # ---- MLP: out = h_mid + down(swiglu(gate_up(norm(h_mid))))
            if s.num_experts:
                n2 = st.n2 if st.n2 is not None else f.rmsnorm_fwd(st.h_mid, p[f"l{i}.mlp_norm"], s.rms_norm_eps)[0]
                st.n2 = None
                d_n2 = self._moe_backward(i, st.moe, d_stream, n2, state.get("aux_dprobs"), wgrad_mode)
                st.moe = None
                del n2
            else:
                act = st.act if st.act is not None else f.swiglu_fwd(st.gate_up)
                st.act = None
                f.gemm(d_stream, act, g[f"l{i}.w_down"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
                d_act = f.gemm(d_stream, p[f"l{i}.w_down"], b_mn=True)
                del act
                dgu = f.swiglu_bwd_(st.gate_up, d_act)
                del d_act
                n2 = st.n2 if st.n2 is not None else f.rmsnorm_fwd(st.h_mid, p[f"l{i}.mlp_norm"], s.rms_norm_eps)[0]
                st.n2 = None
                f.gemm(dgu, n2, g[f"l{i}.w_gate_up"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
                del n2
                d_n2 = f.gemm(dgu, p[f"l{i}.w_gate_up"], b_mn=True)
                if self.tp is not None:
                    self.tp.all_reduce_(d_n2)   # column-parallel projection: the input gradient is a sum over the ranks
                del dgu
            d_mid = f.rmsnorm_bwd(st.h_mid, p[f"l{i}.mlp_norm"], st.rstd2, d_n2, d_stream, g[f"l{i}.mlp_norm"])
            del d_n2, d_stream
            # ---- attention: h_mid = h_in + wo(attn(rope(wqkv(norm(h_in)))))
            sp = self.sp
            f.gemm(d_mid, st.attn_tok if sp is not None else st.attn, g[f"l{i}.wo"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
            if sp is None:
                d_attn = f.gemm(d_mid, p[f"l{i}.wo"], b_mn=True)
                dqkv = self._attn_bwd(i, st, d_attn, cu, scale)
                del d_attn
                f.rope_(dqkv, pos, self.inv_freq, s.num_heads, s.num_kv_heads, s.head_dim, backward=True, table=self._rope_tab)
                self._qkv_bias_and_norm_bwd_(dqkv, i, st.qk)
            else:
                d_attn = sp.d_attn_project(d_mid, p[f"l{i}.wo"], pos.numel())
                dqkv_heads = f.attn_bwd(st.qkv, st.attn, d_attn, st.lse, cu, sp.hq_l, sp.hk_l, s.head_dim, scale)
                f.rope_(dqkv_heads, pos, self.inv_freq, sp.hq_l, sp.hk_l, s.head_dim, backward=True, table=self._rope_tab)
                self._qkv_bias_and_norm_bwd_(dqkv_heads, i, st.qk, sp.hq_l, sp.hk_l, bias=False)
                dqkv = sp.dqkv_exchange(dqkv_heads)
                if s.attention_bias:  # my tokens, every head: this rank's share of the bias gradient
                    g[f"l{i}.bqkv"].add_(dqkv.float().sum(0))
            n1 = st.n1 if st.n1 is not None else f.rmsnorm_fwd(st.h_in, p[f"l{i}.attn_norm"], s.rms_norm_eps)[0]
            st.n1 = None
            f.gemm(dqkv, n1, g[f"l{i}.wqkv"], a_mn=True, b_mn=True, out_mode=wgrad_mode)
            del n1
            d_n1 = f.gemm(dqkv, p[f"l{i}.wqkv"], b_mn=True)
            if self.tp is not None:
                self.tp.all_reduce_(d_n1)
            del dqkv
            d_stream = f.rmsnorm_bwd(st.h_in, p[f"l{i}.attn_norm"], st.rstd1, d_n1, d_mid, g[f"l{i}.attn_norm"])
            del d_n1, d_mid
            if z is not None:
                z.layer_bwd_done(i)  # this layer's weight gradients go to their owners while the next layer runs
            elif self.grad_ready_hook is not None:
                self.grad_ready_hook(*self.layer_grad_range(i))
        f.embedding_bwd(g["embed"], state["ids"], d_stream)
        state.clear()


class _FusedHiddenFn(torch.autograd.Function):
    """Autograd bridge: hidden states out, manual backward in.  ``flat`` only anchors the graph."""

    @staticmethod
    def forward(ctx, model: LlamaModel, input_ids, position_ids, cu_seqlens, keep, anchor):
        ctx.model = model
        nf, ctx.state = model._fused_forward_hidden(input_ids, position_ids, cu_seqlens, keep=keep)
        return nf

    @staticmethod
    def backward(ctx, d_nf):
        ctx.model._fused_backward_hidden(ctx.state, d_nf.contiguous())
        return None, None, None, None, None, None


# Rows of the lm_head GEMM's output that exist at one time.  A micro-batch of at most this many tokens keeps its bf16
# logits for the backward pass (no recomputation); a longer one is processed in chunks of this many tokens through one
# reused [chunk, V] workspace and recomputes each chunk's logits in the backward, so the head's memory does not grow
# with the number of tokens (a 35,840-token GRPO pack at V = 128,256 would otherwise hold 9 GB of logits).
LOGIT_CHUNK_TOKENS = int(os.environ.get("B200_LOGIT_CHUNK", "8192"))


class _FusedLogprobFn(torch.autograd.Function):
    """lm_head GEMM + streaming log-softmax (log-prob of the label, log-sum-exp, entropy) over token chunks; the backward
    rewrites each chunk's bf16 logits in place into their gradient and feeds the head's dgrad / wgrad GEMMs from it.
    Stands where the reference uses liger's fused-linear-cross-entropy (``open_instruct/finetune.py:571-587``) and its
    ``[T, V]``-free ``log_softmax_and_gather`` helper (``open_instruct/model_utils.py:587-600``)."""

    @staticmethod
    def forward(ctx, model: LlamaModel, input_ids, position_ids, cu_seqlens, labels, temperature, want_entropy, keep,
                anchor):
        f = model.kernels
        needs_grad = keep
        nf, ctx.state = model._fused_forward_hidden(input_ids, position_ids, cu_seqlens, keep=needs_grad)
        if model.sp is not None:  # log-probs of this rank's chunk of the tokens
            lo, hi = model.sp.local_tokens(labels.numel())
            labels = labels[lo:hi].contiguous()
        if model.zero3 is not None:
            model.zero3.head()
        w = model.lm_head_weight()
        T, C = nf.shape[0], max(128, LOGIT_CHUNK_TOKENS)
        ctx.model, ctx.temperature, ctx.chunk = model, temperature, C
        ctx.vp = None
        if model.vocab_parallel_head():
            # tensor-parallel group: every rank multiplies with its rows of the head; [T]-sized partials are exchanged
            v0, v1 = model.tp.vocab_range(w.shape[0])
            ctx.vp = (v0, v1)
            w = w[v0:v1]
            zl, lse_loc, ez = (torch.empty(T, dtype=torch.float32, device=nf.device) for _ in range(3))
            logits = None
            keep_logits = needs_grad and T <= C
            ws = None if keep_logits else model.logit_workspace(min(C, T), w.shape[0])
            for t0 in range(0, T, C):
                t1 = min(T, t0 + C)
                lg = f.gemm(nf[t0:t1], w) if keep_logits else f.gemm(nf[t0:t1], w, ws[: t1 - t0])
                zl[t0:t1], lse_loc[t0:t1], ez[t0:t1] = f.logprob_fwd_vp(lg, labels[t0:t1], v0, temperature)
                if keep_logits:
                    logits = lg
            logp, lse, ent = model.tp.combine_logprobs(zl, lse_loc, ez, labels, want_entropy)
        elif T <= C:
            logits = f.gemm(nf, w)
            logp, lse, ent = f.logprob_fwd(logits, labels, temperature, want_entropy)
        else:
            logits = None
            ws = model.logit_workspace(C, w.shape[0])
            logp = torch.empty(T, dtype=torch.float32, device=nf.device)
            lse = torch.empty_like(logp)
            ent = torch.empty_like(logp) if want_entropy else None
            for t0 in range(0, T, C):
                t1 = min(T, t0 + C)
                lg = f.gemm(nf[t0:t1], w, ws[: t1 - t0])
                lp_c, lse_c, ent_c = f.logprob_fwd(lg, labels[t0:t1], temperature, want_entropy)
                logp[t0:t1], lse[t0:t1] = lp_c, lse_c
                if want_entropy:
                    ent[t0:t1] = ent_c
        if needs_grad:
            ctx.save_for_backward(nf, logits if logits is not None else lse.new_zeros(0), lse, labels)
        if ent is None:
            ent = torch.zeros(0, device=logp.device)
        ctx.mark_non_differentiable(ent)
        return logp, ent

    @staticmethod
    def backward(ctx, d_logp, _d_ent):
        model = ctx.model
        f = model.kernels
        nf, logits, lse, labels = ctx.saved_tensors
        model.ensure_main_grad()
        head = "embed" if (model.spec.tie_word_embeddings or "lm_head" not in model.p) else "lm_head"
        w = model.lm_head_weight()
        d_logp = d_logp.contiguous().float()
        T, C = nf.shape[0], ctx.chunk
        if ctx.vp is not None:
            v0, v1 = ctx.vp
            w = w[v0:v1]
            g_head = model.g[head][v0:v1]
            d_nf = torch.empty_like(nf)
            ws = None if logits.numel() else model.logit_workspace(min(C, T), w.shape[0])
            for t0 in range(0, T, C):
                t1 = min(T, t0 + C)
                lg = logits if logits.numel() else f.gemm(nf[t0:t1], w, ws[: t1 - t0])
                f.logprob_bwd_vp_(lg, labels[t0:t1], lse[t0:t1], d_logp[t0:t1], v0, ctx.temperature)
                f.gemm(lg, nf[t0:t1], g_head, a_mn=True, b_mn=True, out_mode=f.OUT_F32_ACC)
                f.gemm(lg, w, d_nf[t0:t1], b_mn=True)
            del logits
            model.tp.all_reduce_(d_nf)  # every rank contributed its vocabulary shard's part of d(hidden)
        elif logits.numel():
            d_logits = f.logprob_bwd_(logits, labels, lse, d_logp, ctx.temperature)
            f.gemm(d_logits, nf, model.g[head], a_mn=True, b_mn=True, out_mode=f.OUT_F32_ACC)
            d_nf = f.gemm(d_logits, w, b_mn=True)
            del d_logits, logits
        else:
            ws = model.logit_workspace(C, w.shape[0])
            d_nf = torch.empty_like(nf)
            for t0 in range(0, T, C):
                t1 = min(T, t0 + C)
                lg = f.gemm(nf[t0:t1], w, ws[: t1 - t0])  # recomputed: the forward kept no logits
                f.logprob_bwd_(lg, labels[t0:t1], lse[t0:t1], d_logp[t0:t1], ctx.temperature)
                f.gemm(lg, nf[t0:t1], model.g[head], a_mn=True, b_mn=True, out_mode=f.OUT_F32_ACC)
                f.gemm(lg, w, d_nf[t0:t1], b_mn=True)
        if head == "lm_head" and model.grad_ready_hook is not None and model.zero3 is None:
            e = model.layout.entries["lm_head"]
            model.grad_ready_hook(e.offset, model.layout.decay_end)
        model._fused_backward_hidden(ctx.state, d_nf)
        return None, None, None, None, None, None, None, None, None
