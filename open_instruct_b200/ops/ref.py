"""Plain-PyTorch statements of every op (the oracles).

These run on CPU or GPU in any float dtype, are differentiable through autograd, and define
the numerics the sm_100a kernels are tested against.  They are also the compute path of
``--ops ref`` (CPU plumbing runs, the NCCL+library baseline).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x @ w^T with w stored [out, in] (HF layout)."""
    return x @ w.t()


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """HF LlamaRMSNorm: fp32 statistics, normalised value cast back before the weight multiply."""
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(dt)


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None = None, device=None) -> torch.Tensor:
    """Inverse frequencies [head_dim/2]; supports the llama3 frequency-dependent scaling rule."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64, device=device) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        smooth = (old / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(is_mid, mid, scaled)
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "linear":
        inv = inv / scaling["factor"]
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "yarn":
        # YaRN: dimensions that turn often within the original context keep their frequency (extrapolation), slow ones are
        # divided by ``factor`` (interpolation), with a linear ramp between the dimensions that make ``beta_fast`` and
        # ``beta_slow`` turns over the original context.  The accompanying attention factor is ``rope_attention_factor``.
        factor, old = scaling["factor"], scaling["original_max_position_embeddings"]
        fast, slow = scaling.get("beta_fast") or 32, scaling.get("beta_slow") or 1
        dim_of = lambda turns: head_dim * math.log(old / (turns * 2 * math.pi)) / (2 * math.log(theta))
        low, high = dim_of(fast), dim_of(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float64, device=device) - low) / (high - low)).clamp(0, 1)
        inv = (inv / factor) * ramp + inv * (1 - ramp)
    elif scaling and scaling.get("rope_type", scaling.get("type")) not in (None, "default"):
        raise NotImplementedError(f"RoPE scaling rule {scaling.get('rope_type', scaling.get('type'))!r} is not built (built: llama3, linear, yarn)")
    return inv.float()


def rope_attention_factor(scaling: dict | None) -> float:
    """The factor YaRN multiplies cos and sin with (``attention_factor``, else ``0.1 * ln(factor) + 1``, with the ``mscale``
    pair when both are given); 1 for every other rule.  q and k both carry it, so attention logits carry its square."""
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "yarn":
        return 1.0
    if scaling.get("attention_factor") is not None:
        return float(scaling["attention_factor"])
    ms = lambda f, m=1.0: 1.0 if f <= 1 else 0.1 * m * math.log(f) + 1.0
    if scaling.get("mscale") and scaling.get("mscale_all_dim"):
        return ms(scaling["factor"], scaling["mscale"]) / ms(scaling["factor"], scaling["mscale_all_dim"])
    return ms(scaling["factor"])


def rope(qkv: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, n_q: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """Rotate the q and k heads of fused qkv [T, (n_q + 2 n_kv) * head_dim] (half-split convention)."""
    T = qkv.shape[0]
    x = qkv.view(T, n_q + 2 * n_kv, head_dim)
    ang = pos.float()[:, None] * inv_freq[None, :].to(pos.device)  # [T, hd/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    rot = x[:, : n_q + n_kv].float()
    h = head_dim // 2
    x1, x2 = rot[..., :h], rot[..., h:]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(qkv.dtype)
    return torch.cat([out, x[:, n_q + n_kv :]], dim=1).reshape(T, -1)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    return F.silu(gate_up[..., :f]) * gate_up[..., f:]


_FORCE_SDPA = False  # tests flip this to run the fused-attention branch on CPU


def _use_sdpa(qkv: torch.Tensor, allow: bool) -> bool:
    return _FORCE_SDPA or (allow and qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16))


def attention_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                     scale: float | None = None, allow_sdpa: bool = False, window: int | None = None) -> torch.Tensor:
    """Causal attention per document over packed tokens: explicit softmax in fp32 (the oracle of the kernel tests; it
    materialises a [heads, L, L] score matrix per document).  With ``allow_sdpa`` and half-precision inputs on a GPU -
    models whose only path this is in production (OLMo-2 / OLMo-3 / OLMoE blocks) - PyTorch's fused scaled-dot-product
    attention per document instead, which does not.  ``window``: a token attends to the latest ``window`` tokens of its
    document only, itself included (sliding-window layers)."""
    T = qkv.shape[0]
    x = qkv.view(T, n_q + 2 * n_kv, head_dim)
    q, k, v = x[:, :n_q], x[:, n_q : n_q + n_kv], x[:, n_q + n_kv :]
    g = n_q // n_kv
    scale = scale if scale is not None else head_dim**-0.5
    bounds = cu_seqlens.tolist()
    if _use_sdpa(qkv, allow_sdpa):
        outs = []
        for s, e in zip(bounds[:-1], bounds[1:]):
            if e > s:
                band = None
                if window and e - s > window:
                    idx = torch.arange(e - s, device=qkv.device)
                    band = (idx[:, None] >= idx[None, :]) & (idx[:, None] - idx[None, :] < window)
                o = torch.nn.functional.scaled_dot_product_attention(q[s:e].transpose(0, 1)[None], k[s:e].transpose(0, 1)[None],
                                                                     v[s:e].transpose(0, 1)[None], attn_mask=band, is_causal=band is None,
                                                                     scale=scale, enable_gqa=g > 1)
                outs.append(o[0].transpose(0, 1))
        return torch.cat(outs, dim=0).reshape(T, n_q * head_dim)
    out = torch.empty(T, n_q, head_dim, dtype=qkv.dtype, device=qkv.device)
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e <= s:
            continue
        qd = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        kd = k[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vd = v[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        sc = (qd @ kd.transpose(1, 2)) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=qkv.device).tril()
        if window and L > window:
            mask &= ~torch.ones(L, L, dtype=torch.bool, device=qkv.device).tril(-window)
        sc = sc.masked_fill(~mask, float("-inf"))
        p = sc.softmax(-1)
        out[s:e] = (p @ vd).transpose(0, 1).to(qkv.dtype)
    return out.reshape(T, n_q * head_dim)


def token_logprobs(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0, with_entropy: bool = False):
    """log p(label) per row in fp32; rows with label < 0 give 0.  Returns (logp, entropy|None)."""
    z = logits.float() / temperature
    lse = torch.logsumexp(z, dim=-1)
    safe = labels.clamp(min=0)
    lp = z.gather(-1, safe[:, None]).squeeze(-1) - lse
    valid = labels >= 0
    lp = torch.where(valid, lp, torch.zeros_like(lp))
    ent = None
    if with_entropy:
        p = torch.softmax(z, -1)
        ent = lse - (p * z).sum(-1)
        ent = torch.where(valid, ent, torch.zeros_like(ent))
    return lp, ent


def adamw_step(master, m, v, grad, lr, beta1, beta2, eps, wd, step, gscale=1.0):
    """One decoupled-weight-decay Adam step on fp32 tensors, in place."""
    g = grad * gscale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    master.mul_(1 - lr * wd)
    denom = (v / bc2).sqrt_().add_(eps)
    master.addcdiv_(m / bc1, denom, value=-lr)
    return master
