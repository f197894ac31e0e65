"""PyTorch statement of the sampling kernel (``ops/csrc/decode.cu:sample_kernel``): temperature,
nucleus filtering, Gumbel-max with Philox4x32-10 uniforms keyed by (seed, step counter, token id),
log-prob of the chosen token under the processed distribution.  Runs on CPU; the oracle for the
kernel and the sampler of the ``ops="ref"`` engine."""

from __future__ import annotations

import numpy as np
import torch

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox_uniform(seed: int, ctr: int, idx: np.ndarray) -> np.ndarray:
    """Uniforms in (0, 1) for token indices ``idx`` (uint32 array) of one row."""
    c0 = idx.astype(np.uint64)
    c1 = np.full_like(c0, ctr & 0xFFFFFFFF)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_M0) * c0
        p1 = np.uint64(_M1) * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)) & mask
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)) & mask
        c1, c3 = p1 & mask, p0 & mask
        c0, c2 = n0, n2
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return ((c0 >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0


def sample_ref(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor):
    """Returns (tokens, logprobs) as Python lists."""
    toks, lps = [], []
    V = logits.shape[1]
    idx = np.arange(V, dtype=np.uint32)
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        z = logits[r].float().cpu().double()
        if t <= 0:
            lp = torch.log_softmax(z, -1)
            tok = int(torch.argmax(z))
            toks.append(tok)
            lps.append(float(lp[tok]))
            continue
        z = z / t
        z = z - z.max()
        e = torch.exp(z)
        keep = torch.ones(V, dtype=torch.bool)
        tp = float(top_p[r])
        if tp < 1.0:
            srt, order = torch.sort(e, descending=True)
            csum = torch.cumsum(srt, 0)
            k = int(torch.searchsorted(csum, torch.tensor(tp * float(e.sum()), dtype=csum.dtype)).item()) + 1
            thr = srt[min(k, V) - 1]
            keep = e >= thr
        u = torch.from_numpy(philox_uniform(int(seeds[r]), int(counters[r]), idx))
        score = torch.where(keep, z - torch.log(-torch.log(u)), torch.full_like(z, float("-inf")))
        tok = int(torch.argmax(score))
        toks.append(tok)
        lps.append(float(z[tok] - torch.log(e[keep].sum())))
    return toks, lps
