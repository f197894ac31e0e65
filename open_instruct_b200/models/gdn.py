"""Gated DeltaNet sequence mixer (the linear-attention layers of OLMo-Hybrid) on the PyTorch path.

The reference trains OLMo-Hybrid through olmo-core's ``GatedDeltaNetConfig`` blocks, three of them per full-attention block
(``open_instruct/olmo_core_hybrid.py:83-140``), and converts checkpoints between the Hugging Face ``olmo_hybrid`` names and
olmo-core's (``:29-75``).  Here the layer is part of ``LlamaModel``'s PyTorch path and the flat layout carries the Hugging Face
names directly (``ParamLayout.hf_names``: ``linear_attn.{q,k,v,g,a,b,o}_proj``, ``{q,k,v}_conv1d``, ``o_norm``, ``A_log``,
``dt_bias``).

Per head the layer keeps a state ``S`` of shape [key_dim, value_dim] and for every token t

    S  <- exp(g_t) * S                              (decay, g_t <= 0)
    d  =  beta_t * (v_t - S^T k_t)                  (what the state does not yet return for this key)
    S  <- S + k_t d^T
    o_t = S^T q_t

with q and k passed through a causal depthwise convolution + SiLU, L2-normalised, q scaled by key_dim^-1/2;
``g = -exp(A_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)`` (times 2 when negative eigenvalues are allowed).  The output
is RMS-normalised per head, gated by ``silu(gate)`` and projected back.

``gated_delta_rule`` evaluates the recurrence chunk by chunk: inside a chunk of C tokens the d_t obey a unit lower-triangular
system (d_i depends on the earlier d_j through k_i . k_j), solved with one triangular solve for all heads; the chunk's outputs and
the state handed to the next chunk are then matrix products.  ``gated_delta_rule_sequential`` is the token-by-token form the
chunked one is tested against.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def gated_delta_rule_sequential(q, k, v, g, beta, state=None):
    """Token-by-token evaluation.  q, k [L, H, dk] (already normalised and scaled), v [L, H, dv], g, beta [L, H]; returns
    (o [L, H, dv], final state [H, dk, dv])."""
    L, H, dk = q.shape
    S = q.new_zeros(H, dk, v.shape[-1]) if state is None else state
    out = []
    for t in range(L):
        S = S * g[t].exp()[:, None, None]
        d = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * d[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def gated_delta_rule(q, k, v, g, beta, state=None, chunk: int = 64):
    """Chunked evaluation of the same recurrence (same arguments and results as the sequential form)."""
    L, H, dk = q.shape
    dv = v.shape[-1]
    S = q.new_zeros(H, dk, dv) if state is None else state
    outs = []
    for c0 in range(0, L, chunk):
        c1 = min(L, c0 + chunk)
        C = c1 - c0
        Q, K, V = (x[c0:c1].transpose(0, 1) for x in (q, k, v))          # [H, C, d]
        G = g[c0:c1].transpose(0, 1).cumsum(-1)                          # log decay from the chunk's start up to and including i
        B = beta[c0:c1].transpose(0, 1)
        low = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()  # j <= i
        ratio = (G[:, :, None] - G[:, None, :]).masked_fill(~low, float("-inf")).exp()   # exp(G_i - G_j), 0 above the diagonal
        kk = torch.einsum("hik,hjk->hij", K, K)
        A = (B[:, :, None] * ratio * kk).tril(-1)                         # strictly lower: the earlier d_j seen through k_i . k_j
        decay = G.exp()                                                   # [H, C]
        rhs = B[:, :, None] * (V - decay[:, :, None] * torch.einsum("hkv,hik->hiv", S, K))
        D = torch.linalg.solve_triangular(A + torch.eye(C, dtype=A.dtype, device=A.device), rhs, upper=False, unitriangular=True)
        qk = torch.einsum("hik,hjk->hij", Q, K) * ratio
        outs.append((decay[:, :, None] * torch.einsum("hkv,hik->hiv", S, Q) + torch.einsum("hij,hjv->hiv", qk, D)).transpose(0, 1))
        tail = (G[:, -1:] - G).exp()                                      # decay from token j to the end of the chunk
        S = decay[:, -1, None, None] * S + torch.einsum("hjk,hjv->hkv", K * tail[:, :, None], D)
    return torch.cat(outs), S


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_segment(x: torch.Tensor, v: dict, i: int, spec, state=None, chunk: int = 64, sequential: bool = False):
    """The mixer over ONE run of consecutive tokens ``x`` [L, D] of a single sequence.  ``state`` continues an earlier run of
    the same sequence: ``(conv_tail, S)`` = the last ``taps - 1`` rows that entered the convolution and the recurrent
    state; None starts a document.  Returns ``(output [L, D], new state)``."""
    s = spec
    K, V, Hk, Hv, dk, dv = s.gdn_k_total, s.gdn_v_total, s.gdn_key_heads, s.gdn_value_heads, s.gdn_key_dim, s.gdn_value_dim
    L = x.shape[0]
    proj = x @ v[f"l{i}.gdn_in"].t()
    qkv, gate, a, b = proj.split([2 * K + V, V, Hv, Hv], dim=1)
    w = v[f"l{i}.gdn_conv"]
    taps = w.shape[1]
    tail = qkv.new_zeros(taps - 1, 2 * K + V) if state is None else state[0].to(qkv.dtype)
    seq = torch.cat([tail, qkv])                                          # [taps - 1 + L, C]
    conv = F.silu(F.conv1d(seq.t()[None], w[:, None, :], groups=w.shape[0])[0].t())
    q, k, val = conv.split([K, K, V], dim=1)
    q = _l2norm(q.float().view(L, Hk, dk)) * dk ** -0.5
    k = _l2norm(k.float().view(L, Hk, dk))
    val = val.float().view(L, Hv, dv)
    if Hv > Hk:
        q, k = q.repeat_interleave(Hv // Hk, dim=1), k.repeat_interleave(Hv // Hk, dim=1)
    beta = torch.sigmoid(b.float()) * (2.0 if s.gdn_neg_eigval else 1.0)
    g = -v[f"l{i}.gdn_A_log"].float().exp() * F.softplus(a.float() + v[f"l{i}.gdn_dt_bias"].float())
    S0 = None if state is None else state[1]
    if sequential or L == 1:
        o, S = gated_delta_rule_sequential(q, k, val, g, beta, S0)
    else:
        o, S = gated_delta_rule(q, k, val, g, beta, S0, chunk=chunk)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5)           # the output norm's epsilon is fixed, not rms_norm_eps
    o = (v[f"l{i}.gdn_o_norm"] * o.to(x.dtype)).float() * F.silu(gate.float().view(L, Hv, dv))
    return o.to(x.dtype).reshape(L, V) @ v[f"l{i}.gdn_out"].t(), (seq[-(taps - 1):].detach(), S.detach())


def gdn_decode_step(x: torch.Tensor, v: dict, i: int, spec, tails: torch.Tensor, S: torch.Tensor):
    """One token for each of B sequences at once: ``x`` [B, D], ``tails`` [B, taps - 1, C] (what last entered each sequence's
    convolution), ``S`` [B, Hv, dk, dv].  Returns ``(output [B, D], new tails, new S)``; the same arithmetic as
    ``gdn_segment`` on a run of length one."""
    s = spec
    K, V, Hk, Hv, dk, dv = s.gdn_k_total, s.gdn_v_total, s.gdn_key_heads, s.gdn_value_heads, s.gdn_key_dim, s.gdn_value_dim
    B = x.shape[0]
    proj = x @ v[f"l{i}.gdn_in"].t()
    qkv, gate, a, b = proj.split([2 * K + V, V, Hv, Hv], dim=1)
    w = v[f"l{i}.gdn_conv"]                                               # [C, taps]
    seq = torch.cat([tails.to(qkv.dtype), qkv[:, None, :]], dim=1)        # [B, taps, C]
    conv = F.silu(torch.einsum("btc,ct->bc", seq, w))
    q, k, val = conv.split([K, K, V], dim=1)
    q = _l2norm(q.float().view(B, Hk, dk)) * dk ** -0.5
    k = _l2norm(k.float().view(B, Hk, dk))
    val = val.float().view(B, Hv, dv)
    if Hv > Hk:
        q, k = q.repeat_interleave(Hv // Hk, dim=1), k.repeat_interleave(Hv // Hk, dim=1)
    beta = torch.sigmoid(b.float()) * (2.0 if s.gdn_neg_eigval else 1.0)
    g = -v[f"l{i}.gdn_A_log"].float().exp() * F.softplus(a.float() + v[f"l{i}.gdn_dt_bias"].float())
    S = S * g.exp()[:, :, None, None]
    d = beta[:, :, None] * (val - torch.einsum("bhkv,bhk->bhv", S, k))
    S = S + k[:, :, :, None] * d[:, :, None, :]
    o = torch.einsum("bhkv,bhk->bhv", S, q)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5)
    o = (v[f"l{i}.gdn_o_norm"] * o.to(x.dtype)).float() * F.silu(gate.float().view(B, Hv, dv))
    return o.to(x.dtype).reshape(B, V) @ v[f"l{i}.gdn_out"].t(), seq[:, 1:].detach(), S.detach()


def gdn_mixer(x: torch.Tensor, v: dict, i: int, spec, cu_seqlens: torch.Tensor, chunk: int = 64, sequential: bool = False) -> torch.Tensor:
    """The gated-DeltaNet sub-layer of layer ``i`` on normed input ``x`` [T, D] of packed documents (``v``: the parameter
    views): every document starts from an empty state and nothing crosses a document boundary."""
    bounds = cu_seqlens.tolist()
    outs = [gdn_segment(x[lo:hi], v, i, spec, None, chunk, sequential)[0] for lo, hi in zip(bounds[:-1], bounds[1:]) if hi > lo]
    return torch.cat(outs) if outs else x.new_zeros(0, spec.hidden_size)
