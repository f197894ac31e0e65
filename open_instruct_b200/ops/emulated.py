"""The kernel wrappers of ``ops.fused`` restated in PyTorch, call for call.

``LlamaModel(ops="emulated")`` runs the SAME hand-driven forward / backward as ``ops="fused"`` (layer stash, activation
recomputation, chunked output head, in-place gradient rewrites) with these functions in place of the sm_100a kernels, on any
device and dtype.  That is how the driver's bookkeeping - which tensor is saved, which gradient is added where - is tested on a
CPU against autograd over the plain PyTorch path; the kernels themselves are tested one by one on the GPU against the same
PyTorch operations.  Nothing here is a training path: every function allocates and none is fast.

Each function keeps the contract of its namesake: argument order, in-place behaviour, what is returned and in which dtype
(statistics and log-probabilities fp32; activations in the dtype of the input).
"""

from __future__ import annotations

import torch

from . import ref

OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_F32_RED = 0, 1, 2, 3


def gemm(a, b, out=None, *, a_mn: bool = False, b_mn: bool = False, out_mode: int = OUT_BF16, max_ctas: int = 0, impl=None):
    """``C[M, N] (op)= A_op[M, K] @ B_op[N, K]^T``; ``a_mn`` / ``b_mn`` say that the operand is stored transposed.  Mode 0
    stores in the operands' dtype (bf16 on the GPU), mode 1 stores fp32, modes 2 / 3 add into the fp32 ``out``."""
    A = (a.t() if a_mn else a).float()
    B = (b if b_mn else b.t()).float()
    c = A @ B
    if out_mode == OUT_BF16:
        c = c.to(a.dtype)
        if out is None:
            return c
        out.copy_(c)
        return out
    if out is None:
        if out_mode != OUT_F32:
            raise ValueError("accumulate mode needs an output tensor")
        return c
    if out.dtype != torch.float32:
        raise TypeError("fp32 output modes need an fp32 out")
    if out_mode == OUT_F32:
        out.copy_(c)
    else:
        out.add_(c)
    return out


def rmsnorm_fwd(x, w, eps: float, res=None):
    """(y, h, rstd): ``h = x (+ res)`` in the input dtype, ``rstd`` fp32 [T], ``y = w * (h * rstd)``."""
    h = x if res is None else (x.float() + res.float()).to(x.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
    y = w * (hf * rstd[:, None]).to(x.dtype)
    return y.to(x.dtype), h, rstd


def rmsnorm_bwd(h, w, rstd, dy, dres, dw_out):
    """``dx = dRMSNorm/dh (+ dres)``; the weight gradient is ADDED into ``dw_out`` (fp32 [D]) when given."""
    hf, dyf, wf = h.float(), dy.float(), w.float()
    xhat = hf * rstd[:, None]
    if dw_out is not None:
        dw_out.add_((dyf * xhat).sum(0))
    dxhat = dyf * wf
    dx = rstd[:, None] * (dxhat - xhat * (dxhat * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx.to(h.dtype)


def rope_table(pos, inv_freq, head_dim: int):
    ang = pos.float()[:, None] * inv_freq[None, :].to(pos.device)
    return torch.stack([ang.cos(), ang.sin()], dim=-1)  # [T, head_dim / 2, 2]


def rope_(qkv, pos, inv_freq, n_q: int, n_kv: int, head_dim: int, backward: bool = False, table=None):
    """In-place rotation of the q and k heads (half-split convention); ``backward`` rotates by the negative angle, which
    is the transpose of the rotation and so its gradient."""
    T = qkv.shape[0]
    tab = table if table is not None else rope_table(pos, inv_freq, head_dim)
    cos, sin = tab[..., 0][:, None, :], tab[..., 1][:, None, :]
    if backward:
        sin = -sin
    x = qkv.view(T, n_q + 2 * n_kv, head_dim)
    rot = x[:, : n_q + n_kv].float()
    half = head_dim // 2
    x1, x2 = rot[..., :half], rot[..., half:]
    x[:, : n_q + n_kv].copy_(torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(qkv.dtype))
    return qkv


def swiglu_fwd(gate_up):
    return ref.swiglu(gate_up.float()).to(gate_up.dtype)


def swiglu_bwd_(gate_up, dact):
    """Overwrites ``gate_up`` with d(gate | up)."""
    F = gate_up.shape[1] // 2
    g, u, d = gate_up[:, :F].float(), gate_up[:, F:].float(), dact.float()
    sig = torch.sigmoid(g)
    dg = d * u * sig * (1 + g * (1 - sig))
    du = d * g * sig
    gate_up.copy_(torch.cat([dg, du], dim=1).to(gate_up.dtype))
    return gate_up


def embedding_fwd(table, ids):
    return table[ids.reshape(-1)].clone()


def embedding_bwd(grad_table, ids, dout) -> None:
    grad_table.index_add_(0, ids.reshape(-1), dout.to(grad_table.dtype))


def logprob_fwd(logits, labels, temperature: float = 1.0, want_entropy: bool = False):
    """(logp, lse, entropy | None), fp32; ``lse`` is the log-sum-exp of ``logits / temperature``."""
    lp, ent = ref.token_logprobs(logits, labels, temperature, with_entropy=want_entropy)
    return lp, torch.logsumexp(logits.float() / temperature, dim=-1), ent


def logprob_bwd_(logits, labels, lse, g, temperature: float = 1.0):
    """Rewrites ``logits`` in place with dL/dlogits given ``g = dL/dlogp``; rows with a negative label give zeros."""
    return logprob_bwd_vp_(logits, labels, lse, g, 0, temperature)


def logprob_fwd_vp(logits, labels, label_offset: int, temperature: float = 1.0):
    """Partials of this rank's logit columns ``[label_offset, label_offset + V_local)``: (the label's logit / temperature if
    the label is one of mine else 0, log-sum-exp over my columns, mean of my scaled logits under MY columns' softmax); zeros
    for rows without a label."""
    z = logits.float() / temperature
    V = z.shape[1]
    loc = labels - label_offset
    mine = (labels >= 0) & (loc >= 0) & (loc < V)
    zl = torch.where(mine, z.gather(1, loc.clamp(0, V - 1)[:, None]).squeeze(1), torch.zeros_like(z[:, 0]))
    valid = labels >= 0
    lse = torch.where(valid, torch.logsumexp(z, dim=-1), torch.zeros_like(zl))
    ez = torch.where(valid, (torch.softmax(z, dim=-1) * z).sum(-1), torch.zeros_like(zl))
    return zl, lse, ez


def logprob_bwd_vp_(logits, labels, lse_global, g, label_offset: int, temperature: float = 1.0):
    z = logits.float() / temperature
    V = z.shape[1]
    p = torch.exp(z - lse_global[:, None])
    loc = labels - label_offset
    mine = (labels >= 0) & (loc >= 0) & (loc < V)
    onehot = torch.zeros_like(p)
    onehot[mine, loc[mine]] = 1.0
    d = (onehot - p) * (g.float() / temperature)[:, None]
    d = torch.where((labels >= 0)[:, None], d, torch.zeros_like(d))
    logits.copy_(d.to(logits.dtype))
    return logits


def attn_max_tiles(total_tokens: int, num_docs: int) -> int:
    return (total_tokens + 127) // 128 + num_docs


def attn_fwd(qkv, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float):
    """(out [T, n_q * head_dim], lse [n_q, T] fp32).  The emulated backward recomputes the scores, so ``lse`` only has the
    kernel's shape."""
    out = ref.attention_varlen(qkv.float(), cu_seqlens, n_q, n_kv, head_dim, scale).to(qkv.dtype)
    return out, torch.zeros(n_q, qkv.shape[0], dtype=torch.float32, device=qkv.device)


def attn_bwd(qkv, out, d_out, lse, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float):
    """Gradient with respect to the post-RoPE fused qkv, by autograd over the explicit-softmax attention."""
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        y = ref.attention_varlen(x, cu_seqlens, n_q, n_kv, head_dim, scale)
        (dx,) = torch.autograd.grad(y, x, d_out.float())
    return dx.to(qkv.dtype)


def attn_fwd_window(qkv, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float, window: int, max_len: int):
    return ref.attention_varlen(qkv.float(), cu_seqlens, n_q, n_kv, head_dim, scale, window=window).to(qkv.dtype)


def attn_bwd_window(qkv, d_out, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float, window: int, max_len: int):
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        y = ref.attention_varlen(x, cu_seqlens, n_q, n_kv, head_dim, scale, window=window)
        (dx,) = torch.autograd.grad(y, x, d_out.float())
    return dx.to(qkv.dtype)
