"""Compact storage of top-k teacher distributions for logit distillation.

A row is the ``k`` largest log-probabilities of one position, sorted descending, plus their vocabulary ids.  Layout of
the compressed row (same ingredients as ``open_instruct/distillkit/compression/monotonic_logprobs.py:114-219``, own format):

    [exact_k values in `exact_dtype`] [polynomial coefficients of the tail in fp32] [per bin: fp16 scale, bit-packed residuals]

The tail ``logp[exact_k:k]`` is smooth and monotone, so a low-degree least-squares polynomial in the normalised rank
captures most of it; what is left is quantised to a few bits per element with one scale per bin.  Token ids are
bit-packed at ``ceil(log2(vocab))`` bits (``pack_bits`` / ``unpack_bits``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class ResidualBin:
    num_elements: int
    element_bits: int  # 1..8


@dataclass
class QuantizationConfig:
    k: int = 64
    exact_k: int = 8
    exact_dtype: torch.dtype = torch.float16
    polynomial_degree: int = 3       # 0 = no polynomial, residual is the raw tail
    residual_bins: list[ResidualBin] = field(default_factory=lambda: [ResidualBin(24, 4), ResidualBin(32, 2)])
    vocab_size: int = 128256

    def __post_init__(self):
        if sum(b.num_elements for b in self.residual_bins) > self.k - self.exact_k:
            raise ValueError("residual bins cover more elements than the approximated tail")

    @property
    def id_bits(self) -> int:
        return max(1, math.ceil(math.log2(self.vocab_size)))

    def logprob_bytes(self) -> int:
        n = self.exact_k * torch.finfo(self.exact_dtype).bits // 8
        n += 4 * (self.polynomial_degree + 1 if self.polynomial_degree > 0 else 0)
        for b in self.residual_bins:
            n += 2 + (b.num_elements * b.element_bits + 7) // 8
        return n


def pack_bits(values: torch.Tensor, bits: int) -> torch.Tensor:
    """``[..., n]`` non-negative ints < 2**bits -> ``[..., ceil(n * bits / 8)]`` uint8 (little-endian bit order)."""
    n = values.shape[-1]
    v = values.to(torch.int64)
    shifts = torch.arange(bits, device=v.device)
    bitsv = ((v.unsqueeze(-1) >> shifts) & 1).reshape(*v.shape[:-1], n * bits)
    pad = (-bitsv.shape[-1]) % 8
    if pad:
        bitsv = torch.nn.functional.pad(bitsv, (0, pad))
    by = bitsv.reshape(*v.shape[:-1], -1, 8)
    return (by << torch.arange(8, device=v.device)).sum(-1).to(torch.uint8)


def unpack_bits(packed: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    b = ((packed.to(torch.int64).unsqueeze(-1) >> torch.arange(8, device=packed.device)) & 1).reshape(*packed.shape[:-1], -1)
    b = b[..., : n * bits].reshape(*packed.shape[:-1], n, bits)
    return (b << torch.arange(bits, device=packed.device)).sum(-1)


def _basis(n: int, degree: int, device) -> torch.Tensor:
    t = torch.linspace(0.0, 1.0, n, device=device, dtype=torch.float32) if n > 1 else torch.zeros(1, device=device)
    return torch.stack([t**d for d in range(degree + 1)], dim=-1)  # [n, degree + 1]


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8).reshape(*t.shape[:-1], -1)


def compress_logprobs(logprobs: torch.Tensor, cfg: QuantizationConfig) -> torch.Tensor:
    """``[..., k]`` sorted-descending log-probs -> ``[..., cfg.logprob_bytes()]`` uint8."""
    if logprobs.shape[-1] != cfg.k:
        raise ValueError(f"expected {cfg.k} values per row")
    lp = logprobs.float()
    chunks = []
    if cfg.exact_k:
        chunks.append(_as_bytes(lp[..., : cfg.exact_k].to(cfg.exact_dtype)))
    tail = lp[..., cfg.exact_k:]
    if cfg.polynomial_degree > 0 and tail.shape[-1] > 0:
        X = _basis(tail.shape[-1], cfg.polynomial_degree, lp.device)
        coef = (torch.linalg.pinv(X) @ tail.unsqueeze(-1)).squeeze(-1)  # least squares, one solve for all rows
        chunks.append(_as_bytes(coef.float()))
        tail = tail - coef.float() @ X.t()
    cur = 0
    for b in cfg.residual_bins:
        vals = tail[..., cur:cur + b.num_elements]
        levels = (1 << b.element_bits) - 1
        half = levels / 2.0
        scale = (vals.abs().amax(-1, keepdim=True) / max(half, 0.5)).clamp(min=1e-8).to(torch.float16)
        q = torch.round(vals / scale.float() + half).clamp(0, levels).to(torch.int64)
        chunks.append(_as_bytes(scale))
        chunks.append(pack_bits(q, b.element_bits))
        cur += b.num_elements
    return torch.cat(chunks, dim=-1)


def decompress_logprobs(data: torch.Tensor, cfg: QuantizationConfig) -> torch.Tensor:
    lead = data.shape[:-1]
    pos = 0
    out = []
    if cfg.exact_k:
        nb = cfg.exact_k * torch.finfo(cfg.exact_dtype).bits // 8
        out.append(data[..., :nb].contiguous().view(cfg.exact_dtype).reshape(*lead, cfg.exact_k).float())
        pos = nb
    n_tail = cfg.k - cfg.exact_k
    fit = torch.zeros(*lead, n_tail, device=data.device)
    if cfg.polynomial_degree > 0 and n_tail > 0:
        nb = 4 * (cfg.polynomial_degree + 1)
        coef = data[..., pos:pos + nb].contiguous().view(torch.float32).reshape(*lead, cfg.polynomial_degree + 1)
        fit = coef @ _basis(n_tail, cfg.polynomial_degree, data.device).t()
        pos += nb
    res = torch.zeros_like(fit)
    cur = 0
    for b in cfg.residual_bins:
        scale = data[..., pos:pos + 2].contiguous().view(torch.float16).reshape(*lead, 1).float()
        pos += 2
        nb = (b.num_elements * b.element_bits + 7) // 8
        q = unpack_bits(data[..., pos:pos + nb], b.element_bits, b.num_elements)
        pos += nb
        half = ((1 << b.element_bits) - 1) / 2.0
        res[..., cur:cur + b.num_elements] = (q.float() - half) * scale
        cur += b.num_elements
    out.append(fit + res)
    return torch.cat(out, dim=-1)
