"""Tensor-level wrappers over the sm_100a kernels (no autograd; the model drives fwd and bwd).

Every function launches on the current CUDA stream and returns immediately.  Inputs must be
contiguous bf16 / fp32 CUDA tensors as documented; shapes are checked here so that a bad
call fails in Python instead of on the device.
"""

from __future__ import annotations

import functools

import torch

from . import lib
from .lib import call, ptr, status_word, stream_ptr

import os

OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_F32_RED = 0, 1, 2, 3  # RED: accumulate with red.global.add (CTA-pair kernel only)
# "2cta": tcgen05 cta_group::2 kernel on CTA pairs (256x256 tiles); "1cta": one CTA per 128x256 tile
GEMM_IMPL = os.environ.get("B200_GEMM_IMPL", "2cta")
# fp32 accumulation of the CTA-pair GEMM through 16-byte `red.global.add` instead of load + add + store
WGRAD_RED = os.environ.get("B200_WGRAD_RED", "0") == "1"


def _check(t: torch.Tensor, dtype, name: str):
    if t.dtype != dtype or not t.is_cuda:
        raise TypeError(f"{name}: expected CUDA {dtype}, got {t.dtype} on {t.device}")
    if t.data_ptr() % 16:
        raise ValueError(f"{name}: pointer must be 16-byte aligned")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, a_mn: bool = False,
         b_mn: bool = False, out_mode: int = OUT_BF16, max_ctas: int = 0, impl: str | None = None) -> torch.Tensor:
    """C[M,N] (op)= A_op[M,K] @ B_op[N,K]^T on the tcgen05 kernel.

    ``a_mn=False``: ``a`` is [M,K]; ``a_mn=True``: ``a`` is [K,M] (used transposed, no copy).
    ``b_mn=False``: ``b`` is [N,K]; ``b_mn=True``: ``b`` is [K,N].
    ``out_mode``: bf16 store, fp32 store, or fp32 accumulate into ``out``.
    Rows may be strided (last dim contiguous, stride multiple of 8 elements).
    """
    _check(a, torch.bfloat16, "a")
    _check(b, torch.bfloat16, "b")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm operands need a contiguous last dimension")
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm reduction mismatch: {K} vs {Kb}")
    lda, ldb = a.stride(0), b.stride(0)
    if lda % 8 or ldb % 8:
        raise ValueError("gemm row strides must be multiples of 8 elements (TMA 16-byte rule)")
    odt = torch.bfloat16 if out_mode == OUT_BF16 else torch.float32
    if out is None:
        if out_mode in (OUT_F32_ACC, OUT_F32_RED):
            raise ValueError("accumulate mode needs an output tensor")
        out = torch.empty(M, N, dtype=odt, device=a.device)
    else:
        _check(out, odt, "out")
        if tuple(out.shape) != (M, N) or out.stride(-1) != 1:
            raise ValueError(f"gemm out shape {tuple(out.shape)} != {(M, N)}")
    ldc = out.stride(0)
    if ldc % 8 and N >= 8:
        raise ValueError("gemm output row stride must be a multiple of 8 elements")
    impl = impl or GEMM_IMPL
    if out_mode == OUT_F32_RED and impl != "2cta":
        raise ValueError("OUT_F32_RED is a mode of the CTA-pair kernel")
    if impl in ("skinny", "skinny128"):
        # 128 x 64 tiles: for small M, where the GEMM is a stream over the weights and needs many CTAs pulling on HBM
        if a_mn or b_mn or out_mode != OUT_BF16:
            raise ValueError("the skinny GEMM covers the forward layout with bf16 output only")
        call("b200_gemm_bf16_skinny", ptr(a), ptr(b), ptr(out), M, N, K, lda, ldb, ldc, ptr(status_word(a.device)), stream_ptr(),
             64 if impl == "skinny" else 128)
        return out
    call("b200_gemm2_bf16" if impl == "2cta" else "b200_gemm_bf16", ptr(a), ptr(b), ptr(out), M, N, K, lda, ldb, ldc,
         int(a_mn), int(b_mn), 3 if (out_mode == OUT_F32_ACC and WGRAD_RED and impl == "2cta") else out_mode,
         ptr(status_word(a.device)), stream_ptr(), max_ctas)
    return out


def gemm_splitk_(acc32: torch.Tensor, a: torch.Tensor, b: torch.Tensor, splits: int) -> torch.Tensor:
    """``acc32 += a @ b^T`` (fp32 [M, N], atomically) with the K range cut into ``splits`` slices on different SMs: for small M and
    long K, where one tile per output block would leave most of the GPU idle.  ``acc32`` must hold zeros (or a seed)."""
    _check(a, torch.bfloat16, "a")
    _check(b, torch.bfloat16, "b")
    _check(acc32, torch.float32, "acc32")
    M, K = a.shape
    N = b.shape[0]
    if tuple(acc32.shape) != (M, N) or b.shape[1] != K or a.stride(0) % 8 or b.stride(0) % 8 or acc32.stride(0) % 4:
        raise ValueError("split-K GEMM: shape or stride mismatch")
    call("b200_gemm_bf16_splitk", ptr(a), ptr(b), ptr(acc32), M, N, K, a.stride(0), b.stride(0), acc32.stride(0), splits,
         ptr(status_word(a.device)), stream_ptr())
    return acc32


# ---------------------------------------------------------------------------------- decode-sized GEMM (M <= 256)
DECODE_TILES = ((64, 1), (96, 1), (128, 1), (256, 1), (192, 2), (224, 2), (256, 2))  # (columns per MMA, MMAs side by side)
DECODE_SPLIT_TILES = ((128, 1), (256, 1), (256, 2))                                   # shapes that can write fp32 K-slice planes
_PAIRS = 74            # CTA pairs of one B200 (148 SMs)
_SM_BYTES_PER_US = 80e3   # what one busy SM was measured to take in from L2 (about 80 GB/s)
_HBM_BYTES_PER_US = 6.0e6
_PLANE_BYTES_PER_US = 4.0e6  # fp32 K-slice planes: written by the GEMM, read by the norm, mostly out of L2


def decode_splits(K: int, splits: int) -> int:
    """K slices really used for a request of ``splits`` (no slice may be empty; 64-wide K blocks)."""
    nkb = -(-K // 64)
    splits = max(1, min(splits, nkb))
    per = -(-nkb // splits)
    while splits > 1 and per * (splits - 1) >= nkb:
        splits -= 1
        per = -(-nkb // splits)
    return splits


@functools.lru_cache(maxsize=None)
def decode_gemm_plan(N: int, K: int, allow_split: bool, rows: int = 256) -> tuple[int, int, int]:
    """(columns per MMA, MMAs per tile, K slices) for ``C[rows <= 256, N] = A @ W[N, K]^T``: the combination whose modelled
    time is lowest.  The model is the one the kernel was shaped by: a launch is one or more waves of 74 CTA pairs, a CTA takes
    in its 128 rows of A plus half of the tile's weights at a fixed rate, the weights cannot arrive faster than HBM delivers
    them, and K-slice planes cost a write and a read."""
    best, best_t = (256, 1, 1), float("inf")
    a_rows = min(128, max(1, rows))  # rows of A a CTA really loads (rows past M are filled, not fetched)
    for bns, nsub in DECODE_TILES:
        bnt = bns * nsub
        tiles = -(-N // bnt)
        options = (1, 2, 3, 4, 6, 8) if allow_split and (bns, nsub) in DECODE_SPLIT_TILES else (1,)
        for want in options:
            S = decode_splits(K, want)
            per = -(-(-(-K // 64)) // S)
            if S != want or (S > 1 and per < 8):  # a slice shorter than the load pipeline only adds planes
                continue
            waves = -(-(tiles * S) // _PAIRS)
            t = waves * (a_rows + bnt // 2) * per * 128 / _SM_BYTES_PER_US
            t = max(t, N * K * 2 / _HBM_BYTES_PER_US)
            if S > 1:
                t += S * rows * N * 4 * 2 / _PLANE_BYTES_PER_US + 0.5 * (S - 1)
            if t < best_t - 1e-9:
                best, best_t = (bns, nsub, S), t
    return best


def gemm_decode(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, plan: tuple[int, int, int] | None = None) -> torch.Tensor:
    """``a[M <= 256, K] @ w[N, K]^T`` on the decode GEMM (one wave of CTA pairs over the weights).  With a plan of one K
    slice the result is bf16 [M, N]; with S > 1 slices it is fp32 [S, M, N], plane s holding the product over slice s (sum
    them, e.g. with ``rmsnorm_fwd_parts``)."""
    _check(a, torch.bfloat16, "a")
    _check(w, torch.bfloat16, "w")
    M, K = a.shape
    N = w.shape[0]
    if M > 256 or N % 16 or w.shape[1] != K or a.stride(-1) != 1 or w.stride(-1) != 1 or a.stride(0) % 8 or w.stride(0) % 8:
        raise ValueError("decode GEMM: at most 256 rows, N a multiple of 16, K-major operands with 16-byte aligned rows")
    bns, nsub, S = plan or decode_gemm_plan(N, K, False, M)
    if S > 1:
        if decode_splits(K, S) != S:
            raise ValueError(f"{S} K slices leave one empty at K = {K}")
        if out is None:
            out = torch.empty(S, M, N, dtype=torch.float32, device=a.device)
        elif out.dtype != torch.float32 or tuple(out.shape) != (S, M, N) or not out.is_contiguous():
            raise ValueError("decode GEMM: K-slice planes must be a contiguous fp32 [S, M, N]")
        call("b200_gemm_decode", ptr(a), ptr(w), ptr(out), M, N, K, a.stride(0), w.stride(0), N, M * N, bns, nsub, S,
             ptr(status_word(a.device)), stream_ptr())
        return out
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or out.stride(-1) != 1 or out.stride(0) % 8:
        raise ValueError("decode GEMM: out must be bf16 [M, N] with a 16-byte aligned row stride")
    call("b200_gemm_decode", ptr(a), ptr(w), ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0), 0, bns, nsub, 1,
         ptr(status_word(a.device)), stream_ptr())
    return out


def rmsnorm_fwd_parts(parts: torch.Tensor, w: torch.Tensor, eps: float, res: torch.Tensor | None):
    """RMSNorm of ``bf16(sum over planes of parts) (+ res)`` for fp32 ``parts`` [S, T, D] (the K-slice planes of
    ``gemm_decode``).  Returns ``(y, h)`` like ``rmsnorm_fwd_acc32_``; nothing is zeroed."""
    _check(parts, torch.float32, "parts")
    S, T, D = parts.shape
    if not parts.is_contiguous():
        raise ValueError("K-slice planes must be contiguous")
    y = torch.empty(T, D, dtype=torch.bfloat16, device=parts.device)
    h = torch.empty_like(y)
    call("b200_rmsnorm_fwd_parts", ptr(parts), S, T * D, ptr(res), ptr(w), ptr(h), ptr(y), T, D, eps, stream_ptr())
    return y, h


def rmsnorm_fwd_acc32_(acc32: torch.Tensor, w: torch.Tensor, eps: float, res: torch.Tensor | None):
    """RMSNorm of ``bf16(acc32) (+ res)``; ``acc32`` (fp32 [T, D]) is zeroed on the way so that the next split-K GEMM can add
    into it again.  Returns ``(y, h)``."""
    T, D = acc32.shape
    y = torch.empty(T, D, dtype=torch.bfloat16, device=acc32.device)
    h = torch.empty_like(y)
    call("b200_rmsnorm_fwd_acc32", ptr(acc32), ptr(res), ptr(w), ptr(h), ptr(y), None, T, D, eps, stream_ptr())
    return y, h


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, res: torch.Tensor | None = None):
    """Returns (y, h, rstd): h = x (+ res) is the residual stream that was normalised."""
    T, D = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    h = torch.empty_like(x) if res is not None else x
    call("b200_rmsnorm_fwd", ptr(x), ptr(res), ptr(w), ptr(h), ptr(y), ptr(rstd), T, D, eps, stream_ptr())
    return y, h, rstd


def rmsnorm_bwd(h: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, dy: torch.Tensor,
                dres: torch.Tensor | None, dw_out: torch.Tensor | None) -> torch.Tensor:
    """dx = d/dh RMSNorm (+ dres); ``dw_out`` (fp32 [D]) is accumulated into when given."""
    T, D = h.shape
    dx = torch.empty_like(h)
    ctas = lib.load_ops().b200_rmsnorm_bwd_ctas(T)
    partial = torch.empty(ctas, D, dtype=torch.float32, device=h.device)
    call("b200_rmsnorm_bwd", ptr(h), ptr(w), ptr(rstd), ptr(dy), ptr(dres), ptr(dx), ptr(partial), ptr(dw_out), T, D,
         stream_ptr())
    return dx


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor, head_dim: int) -> torch.Tensor:
    """(cos, sin) of every (token, frequency) pair, fp32 [T, head_dim / 2, 2]: computed once per packed batch and shared by all
    layers and by the backward rotation."""
    if pos.dtype != torch.int32:
        raise TypeError("rope positions must be int32")
    tab = torch.empty(pos.numel(), head_dim // 2, 2, dtype=torch.float32, device=pos.device)
    call("b200_rope_table", ptr(pos), ptr(inv_freq), ptr(tab), pos.numel(), head_dim, stream_ptr())
    return tab


def rope_(qkv: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
          backward: bool = False, table: torch.Tensor | None = None) -> torch.Tensor:
    """In-place rotary embedding of the q and k heads of fused qkv; ``pos`` int32 [T].  With ``table`` (from ``rope_table``)
    the rotation reads precomputed cos/sin instead of evaluating them per head."""
    if table is not None and head_dim % 16 == 0:
        call("b200_rope_apply", ptr(qkv), ptr(table), qkv.shape[0], n_q, n_kv, head_dim, int(backward), stream_ptr())
        return qkv
    if pos.dtype != torch.int32:
        raise TypeError("rope positions must be int32")
    call("b200_rope", ptr(qkv), ptr(pos), ptr(inv_freq), qkv.shape[0], n_q, n_kv, head_dim, int(backward), stream_ptr())
    return qkv


def swiglu_fwd(gate_up: torch.Tensor) -> torch.Tensor:
    T, F2 = gate_up.shape
    act = torch.empty(T, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    call("b200_swiglu_fwd", ptr(gate_up), ptr(act), T, F2 // 2, stream_ptr())
    return act


def swiglu_bwd_(gate_up: torch.Tensor, dact: torch.Tensor) -> torch.Tensor:
    """Overwrites ``gate_up`` with d(gate|up)."""
    T, F2 = gate_up.shape
    call("b200_swiglu_bwd", ptr(gate_up), ptr(dact), ptr(gate_up), T, F2 // 2, stream_ptr())
    return gate_up


def embedding_fwd(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    V, D = table.shape
    T = ids.numel()
    out = torch.empty(T, D, dtype=table.dtype, device=table.device)
    call("b200_embedding_fwd", ptr(table), ptr(ids), ptr(out), T, D, V, stream_ptr())
    return out


def embedding_bwd(grad_table: torch.Tensor, ids: torch.Tensor, dout: torch.Tensor) -> None:
    V, D = grad_table.shape
    call("b200_embedding_bwd", ptr(grad_table), ptr(ids), ptr(dout), ids.numel(), D, V, stream_ptr())


_sumsq_scratch: dict[int, torch.Tensor] = {}


def sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= sum(g^2) for an fp32 tensor, deterministic two-stage reduction."""
    dev = g.device.index
    sc = _sumsq_scratch.get(dev)
    if sc is None:
        sc = torch.empty(lib.load_ops().b200_sumsq_scratch_floats(), dtype=torch.float32, device=g.device)
        _sumsq_scratch[dev] = sc
    call("b200_sumsq", ptr(g), g.numel(), ptr(sc), ptr(out), int(accumulate), stream_ptr())
    return out


def adamw(master, m, v, grad, param_bf16, *, lr, beta1, beta2, eps, wd, step, gscale=None, zero_grad=True) -> None:
    """Partitioned AdamW on fp32 shards; refreshes the bf16 working copy; zeroes the grad shard."""
    call("b200_adamw", ptr(master), ptr(m), ptr(v), ptr(grad), ptr(param_bf16), master.numel(), ptr(gscale), lr, beta1,
         beta2, eps, wd, step, int(zero_grad), stream_ptr())


def logprob_fwd(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0, want_entropy: bool = False):
    """(logp, lse, entropy|None) in fp32 from bf16 logits [T, V]; labels int64, <0 ignored."""
    T, V = logits.shape
    lp = torch.empty(T, dtype=torch.float32, device=logits.device)
    lse = torch.empty(T, dtype=torch.float32, device=logits.device)
    ent = torch.empty(T, dtype=torch.float32, device=logits.device) if want_entropy else None
    call("b200_logprob_fwd", ptr(logits), ptr(labels), ptr(lp), ptr(lse), ptr(ent), T, V, logits.stride(0), temperature,
         stream_ptr())
    return lp, lse, ent


def logprob_fwd_vp(logits: torch.Tensor, labels: torch.Tensor, label_offset: int, temperature: float = 1.0):
    """Vocabulary-parallel partials from this rank's logit columns ``[label_offset, label_offset + V_local)``:
    ``(label_logit, lse_local, mean_logit_local)`` fp32 [T]; rows whose (global) label is negative give zeros."""
    T, V = logits.shape
    zl, lse, ez = (torch.empty(T, dtype=torch.float32, device=logits.device) for _ in range(3))
    call("b200_logprob_fwd_vp", ptr(logits), ptr(labels), ptr(zl), ptr(lse), ptr(ez), T, V, logits.stride(0), temperature, label_offset,
         stream_ptr())
    return zl, lse, ez


def logprob_bwd_vp_(logits: torch.Tensor, labels: torch.Tensor, lse_global: torch.Tensor, g: torch.Tensor, label_offset: int,
                    temperature: float = 1.0) -> torch.Tensor:
    """In-place ``dL/dlogits`` of this rank's logit columns given the GLOBAL log-sum-exp and global labels."""
    T, V = logits.shape
    call("b200_logprob_bwd_vp", ptr(logits), ptr(labels), ptr(lse_global), ptr(g), T, V, logits.stride(0), temperature, label_offset,
         stream_ptr())
    return logits


def logprob_bwd_(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, g: torch.Tensor,
                 temperature: float = 1.0) -> torch.Tensor:
    """Rewrites ``logits`` in place with dL/dlogits given g = dL/dlogp (fp32 [T])."""
    T, V = logits.shape
    call("b200_logprob_bwd", ptr(logits), ptr(labels), ptr(lse), ptr(g), T, V, logits.stride(0), temperature,
         stream_ptr())
    return logits


def attn_max_tiles(total_tokens: int, num_docs: int) -> int:
    return (total_tokens + 127) // 128 + num_docs


def attn_fwd(qkv: torch.Tensor, cu_seqlens: torch.Tensor, n_q: int, n_kv: int, head_dim: int, scale: float):
    """Varlen causal attention forward.  Returns (out [T, n_q*hd] bf16, lse [n_q, T] fp32)."""
    T = qkv.shape[0]
    B = cu_seqlens.numel() - 1
    out = torch.empty(T, n_q * head_dim, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(n_q, T, dtype=torch.float32, device=qkv.device)
    call("b200_attn_fwd", ptr(qkv), ptr(cu_seqlens), ptr(out), ptr(lse), ptr(status_word(qkv.device)), T, B, n_q, n_kv,
         head_dim, attn_max_tiles(T, B), scale, stream_ptr())
    return out, lse


def attn_bwd(qkv, out, d_out, lse, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float) -> torch.Tensor:
    """Returns dqkv [T, (n_q + 2 n_kv) * hd] bf16 (gradient w.r.t. the post-RoPE fused qkv)."""
    T = qkv.shape[0]
    B = cu_seqlens.numel() - 1
    dqkv = torch.empty_like(qkv)
    scratch = torch.empty(n_q * T + T * n_q * head_dim, dtype=torch.float32, device=qkv.device)
    call("b200_attn_bwd", ptr(qkv), ptr(out), ptr(d_out), ptr(lse), ptr(cu_seqlens), ptr(dqkv), ptr(scratch),
         ptr(status_word(qkv.device)), T, B, n_q, n_kv, head_dim, attn_max_tiles(T, B), scale, stream_ptr())
    return dqkv


def _window_attention(qkv, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float, window: int, max_len: int):
    from flash_attn import flash_attn_varlen_func

    T = qkv.shape[0]
    x = qkv.view(T, n_q + 2 * n_kv, head_dim)
    out = flash_attn_varlen_func(x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:], cu_seqlens, cu_seqlens, max_len, max_len, 0.0,
                                 softmax_scale=scale, causal=True, window_size=(window - 1, 0))
    return out.reshape(T, n_q * head_dim)


def attn_fwd_window(qkv: torch.Tensor, cu_seqlens: torch.Tensor, n_q: int, n_kv: int, head_dim: int, scale: float, window: int, max_len: int):
    """Varlen causal attention in which a token sees the latest ``window`` tokens of its document only (itself included).  The
    attention kernels of this package have no window, so layers whose documents outgrow it call the FlashAttention library
    (``window_size=(window - 1, 0)``); a library call like a cuBLAS GEMM, used by sliding-window layers only."""
    with torch.no_grad():
        return _window_attention(qkv, cu_seqlens, n_q, n_kv, head_dim, scale, window, max_len)


def attn_bwd_window(qkv, d_out, cu_seqlens, n_q: int, n_kv: int, head_dim: int, scale: float, window: int, max_len: int) -> torch.Tensor:
    """dqkv of ``attn_fwd_window``: the library recomputes its forward and differentiates it."""
    with torch.enable_grad():
        x = qkv.detach().requires_grad_(True)
        y = _window_attention(x, cu_seqlens, n_q, n_kv, head_dim, scale, window, max_len)
        (dx,) = torch.autograd.grad(y, x, d_out.reshape(y.shape))
    return dx
