"""Numerics of every sm_100a kernel against the plain-PyTorch fp32 statement of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status():
    from open_instruct_b200.ops import lib

    yield
    lib.check_status()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("impl", ["1cta", "2cta"])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 512, 128), (384, 320, 192), (1000, 136, 72), (1000, 192, 72), (4096, 1024, 4096), (2048, 6144, 4096)])
def test_gemm_layouts(a_mn, b_mn, shape, impl):
    from open_instruct_b200.ops import fused

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = fused.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn, impl=impl)
    assert _rel(out, ref) < 5e-3
    out32 = fused.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn, out_mode=fused.OUT_F32, impl=impl)
    assert _rel(out32, ref) < 1e-4
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    fused.gemm(a_in, b_in, acc, a_mn=a_mn, b_mn=b_mn, out_mode=fused.OUT_F32_ACC, impl=impl)
    assert _rel(acc, ref + 1) < 1e-4
    if impl == "2cta":  # the same accumulation through red.global.add
        acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
        fused.gemm(a_in, b_in, acc, a_mn=a_mn, b_mn=b_mn, out_mode=fused.OUT_F32_RED, impl=impl)
        assert _rel(acc, ref + 1) < 1e-4


@pytest.mark.parametrize("shape", [(1, 512, 128), (37, 200, 72), (256, 4096, 4096), (300, 6144, 1024), (512, 4096, 14336)])
@pytest.mark.parametrize("impl", ["skinny", "skinny128"])
def test_gemm_skinny(shape, impl):
    from open_instruct_b200.ops import fused

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    out = fused.gemm(a, b, impl=impl)
    assert _rel(out, a.float() @ b.float().t()) < 5e-3


def test_gemm_strided_views():
    from open_instruct_b200.ops import fused

    x = torch.randn(512, 1024, device="cuda").bfloat16()
    w = torch.randn(256, 512, device="cuda").bfloat16()
    a = x[:, 256:768]  # row stride 1024
    out = fused.gemm(a, w)
    assert _rel(out, a.float() @ w.float().t()) < 5e-3


@pytest.mark.parametrize("T,D", [(7, 64), (300, 4096), (1024, 8192), (5, 2048), (700, 2048), (1500, 4096), (333, 5120)])
def test_rmsnorm(T, D):
    from open_instruct_b200.ops import fused, ref

    x = torch.randn(T, D, device="cuda").bfloat16()
    r = torch.randn(T, D, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    y, h, rstd = fused.rmsnorm_fwd(x, w, 1e-5, res=r)
    h_ref = (x + r)
    assert torch.equal(h, h_ref)
    y_ref = ref.rmsnorm(h_ref, w, 1e-5)
    assert _rel(y, y_ref) < 4e-3
    y2, h2, _ = fused.rmsnorm_fwd(x, w, 1e-5)
    assert h2 is x and _rel(y2, ref.rmsnorm(x, w, 1e-5)) < 4e-3
    # backward against autograd on the fp32 statement
    hf = h_ref.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    yf = wf * (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5))
    dy = torch.randn(T, D, device="cuda").bfloat16()
    dres = torch.randn(T, D, device="cuda").bfloat16()
    yf.backward(dy.float())
    dw = torch.zeros(D, device="cuda")
    dx = fused.rmsnorm_bwd(h, w, rstd, dy, dres, dw)
    assert _rel(dx, hf.grad + dres.float()) < 6e-3
    assert _rel(dw, wf.grad) < 5e-3


def test_rope_roundtrip_and_ref():
    from open_instruct_b200.ops import fused, ref

    T, Hq, Hkv, Dh = 333, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * Dh, device="cuda").bfloat16()
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    inv = ref.rope_inv_freq(Dh, 5e5, device="cuda")
    expect = ref.rope(qkv, pos, inv, Hq, Hkv, Dh)
    got = fused.rope_(qkv.clone(), pos, inv, Hq, Hkv, Dh)
    assert _rel(got, expect) < 4e-3
    back = fused.rope_(got.clone(), pos, inv, Hq, Hkv, Dh, backward=True)
    assert _rel(back, qkv) < 8e-3
    assert torch.equal(got[:, (Hq + Hkv) * Dh:], qkv[:, (Hq + Hkv) * Dh:])
    # same rotation from the precomputed cos/sin table (what the model uses)
    tab = fused.rope_table(pos, inv, Dh)
    got_t = fused.rope_(qkv.clone(), pos, inv, Hq, Hkv, Dh, table=tab)
    assert _rel(got_t, expect) < 4e-3 and (got_t.float() - got.float()).abs().max().item() < 0.04
    back_t = fused.rope_(got_t.clone(), pos, inv, Hq, Hkv, Dh, backward=True, table=tab)
    assert _rel(back_t, qkv) < 8e-3
    assert torch.equal(got_t[:, (Hq + Hkv) * Dh:], qkv[:, (Hq + Hkv) * Dh:])


def test_swiglu():
    from open_instruct_b200.ops import fused, ref

    T, Fd = 257, 1024
    gu = torch.randn(T, 2 * Fd, device="cuda").bfloat16()
    act = fused.swiglu_fwd(gu)
    assert _rel(act, ref.swiglu(gu.float())) < 4e-3
    guf = gu.float().requires_grad_(True)
    d = torch.randn(T, Fd, device="cuda").bfloat16()
    ref.swiglu(guf).backward(d.float())
    dgu = fused.swiglu_bwd_(gu.clone(), d)
    assert _rel(dgu, guf.grad) < 5e-3


def test_embedding():
    from open_instruct_b200.ops import fused

    V, D, T = 1000, 256, 777
    table = torch.randn(V, D, device="cuda").bfloat16()
    ids = torch.randint(0, V, (T,), device="cuda")
    out = fused.embedding_fwd(table, ids)
    assert torch.equal(out, table[ids])
    dout = torch.randn(T, D, device="cuda").bfloat16()
    g = torch.zeros(V, D, device="cuda")
    fused.embedding_bwd(g, ids, dout)
    expect = torch.zeros(V, D, device="cuda").index_add_(0, ids, dout.float())
    assert _rel(g, expect) < 1e-5


def test_sumsq_and_adamw():
    from open_instruct_b200.ops import fused, ref

    n = 1_000_003
    g = torch.randn(n, device="cuda")
    out = torch.zeros(1, device="cuda")
    fused.sumsq(g, out)
    assert abs(out.item() - g.double().pow(2).sum().item()) / n < 1e-4
    fused.sumsq(g, out, accumulate=True)
    assert abs(out.item() - 2 * g.double().pow(2).sum().item()) / n < 2e-4
    master = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    gs = torch.tensor([0.5], device="cuda")
    for step in (1, 2, 3):
        grad = torch.randn(n, device="cuda")
        ref.adamw_step(rm, rmm, rv, grad, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, gscale=0.5)
        fused.adamw(master, m, v, grad, p16, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01, step=step, gscale=gs)
        assert float(grad.abs().max()) == 0.0
    assert _rel(master, rm) < 1e-5 and _rel(m, rmm) < 1e-5 and _rel(v, rv) < 1e-4
    assert torch.equal(p16, master.bfloat16())


@pytest.mark.parametrize("T,V,temp", [(64, 512, 1.0), (300, 128256, 1.0), (37, 32003, 0.7)])
def test_logprob(T, V, temp):
    from open_instruct_b200.ops import fused, ref

    Vp = (V + 7) // 8 * 8
    buf = (3 * torch.randn(T, Vp, device="cuda")).bfloat16()
    logits = buf[:, :V]
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::5] = -100
    lp, lse, ent = fused.logprob_fwd(logits, labels, temp, want_entropy=True)
    rlp, rent = ref.token_logprobs(logits, labels, temp, with_entropy=True)
    assert (lp - rlp).abs().max().item() < 2e-3
    assert (ent - rent).abs().max().item() < 2e-3
    lf = logits.float().requires_grad_(True)
    g = torch.randn(T, device="cuda")
    (ref.token_logprobs(lf, labels, temp)[0] * g).sum().backward()
    d = fused.logprob_bwd_(logits.clone() if V == Vp else buf.clone()[:, :V], labels, lse, g, temp)
    assert _rel(d, lf.grad) < 1e-2


def _attn_case(lens, Hq, Hkv):
    from open_instruct_b200.ops import fused, ref

    Dh = 128
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * Dh, device="cuda").bfloat16()
    scale = Dh ** -0.5
    out, lse = fused.attn_fwd(qkv, cu, Hq, Hkv, Dh, scale)
    qf = qkv.float().requires_grad_(True)
    ref_out = ref.attention_varlen(qf, cu, Hq, Hkv, Dh, scale)
    assert _rel(out, ref_out) < 1e-2, "forward"
    d_out = torch.randn(T, Hq * Dh, device="cuda").bfloat16()
    ref_out.backward(d_out.float())
    dqkv = fused.attn_bwd(qkv, out, d_out, lse, cu, Hq, Hkv, Dh, scale)
    w = Hq * Dh
    assert _rel(dqkv[:, :w], qf.grad[:, :w]) < 2e-2, "dq"
    assert _rel(dqkv[:, w:w + Hkv * Dh], qf.grad[:, w:w + Hkv * Dh]) < 2e-2, "dk"
    assert _rel(dqkv[:, w + Hkv * Dh:], qf.grad[:, w + Hkv * Dh:]) < 2e-2, "dv"


@pytest.mark.parametrize("lens", [[128], [256], [100], [1, 130, 255, 384], [513, 77]])
def test_attention_varlen(lens):
    _attn_case(lens, 4, 2)


def test_attention_gqa_llama_heads():
    _attn_case([700, 324], 32, 8)


@pytest.mark.parametrize("shape", [(256, 512, 128), (300, 1024, 192), (4096, 6144, 512)])
def test_gemm_scatter_epilogue_local(shape):
    """Column-scatter epilogue (shared-memory transpose, two destination tables) with every destination on this GPU:
    128-column block j goes to buffer j % 2 at column block j // 2, rows shifted by 5; a second table mirrors it."""
    import ctypes

    from open_instruct_b200.ops import fused, lib
    from open_instruct_b200.ops.lib import ptr, status_word, stream_ptr

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    ref = fused.gemm(a, b)
    nb, off = N // 128, 5
    half = (nb + 1) // 2 * 128
    bufs = [torch.zeros(M + off, half, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    mk = lambda pair: torch.tensor([pair[j % 2].data_ptr() + 2 * (j // 2) * 128 for j in range(nb)], dtype=torch.int64, device="cuda")
    t1, t2 = mk(bufs[:2]), mk(bufs[2:])
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib._SIGNATURES["b200_gemm2_bf16_scatter"] = [P, P, I, I, I, L, L, I, I, P, I, L, P, P, P]
    fn = lib.load_ops().b200_gemm2_bf16_scatter
    fn.argtypes, fn.restype = lib._SIGNATURES["b200_gemm2_bf16_scatter"], ctypes.c_int
    lib.call("b200_gemm2_bf16_scatter", ptr(a), ptr(b), M, N, K, a.stride(0), b.stride(0), 0, 0, ptr(t1), off, half, ptr(status_word(a.device)),
             stream_ptr(), ptr(t2))
    torch.cuda.synchronize()
    for pair in (bufs[:2], bufs[2:]):
        for j in range(nb):
            got = pair[j % 2][off:, (j // 2) * 128:(j // 2 + 1) * 128]
            assert torch.equal(got, ref[:, j * 128:(j + 1) * 128]), (shape, j)
        assert all(buf[:off].abs().sum() == 0 for buf in pair)


@pytest.mark.parametrize("shape,splits", [((256, 4096, 14336), 8), ((64, 512, 4096), 4), ((37, 200, 1000), 3), ((256, 4096, 4096), 1)])
def test_gemm_splitk_and_consuming_norm(shape, splits):
    from open_instruct_b200.ops import fused

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + K)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    acc = torch.zeros(M, N, device="cuda")
    fused.gemm_splitk_(acc, a, b, splits)
    ref = a.float() @ b.float().t()
    assert _rel(acc, ref) < 1e-3
    if N % 8 == 0:
        res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
        w = (torch.rand(N, device="cuda", generator=g) + 0.5).bfloat16()
        y, h = fused.rmsnorm_fwd_acc32_(acc, w, 1e-5, res)
        y2, h2, _ = fused.rmsnorm_fwd(ref.bfloat16(), w, 1e-5, res=res)
        assert acc.abs().max().item() == 0.0  # consumed: ready for the next accumulation
        assert (h.float() - h2.float()).abs().max().item() < 0.07 and _rel(y, y2) < 2e-2


@pytest.mark.parametrize("tile", [(64, 1), (96, 1), (128, 1), (256, 1), (192, 2), (224, 2), (256, 2)])
@pytest.mark.parametrize("M", [1, 100, 256])
def test_decode_gemm_matches_reference(tile, M):
    """One-wave decode GEMM, every tile shape, against fp32 PyTorch: N not a multiple of the tile width (edge tiles), K not a
    multiple of the 64-wide block (zero-filled tail), rows below and at the 256-row limit."""
    from open_instruct_b200.ops import fused as f
    from open_instruct_b200.ops import lib

    torch.manual_seed(M + tile[0])
    N, K = 1072, 1000  # 1072 = 16 * 67: no tile width divides it; K = 1000: 15 full K blocks and a 40-wide tail
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    want = a.float() @ w.float().t()
    got = f.gemm_decode(a, w, plan=(tile[0], tile[1], 1))
    lib.check_status()
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (M, N)
    assert ((got.float() - want).norm() / want.norm()).item() < 5e-3


@pytest.mark.parametrize("tile,splits", [((128, 1), 2), ((256, 1), 4), ((256, 2), 3), ((256, 1), 5)])
def test_decode_gemm_k_slices_and_plane_summing_norm(tile, splits):
    """K-slice planes: every plane holds its slice's product, their sum is the product, and the plane-summing RMSNorm equals
    the unfused statement (sum -> bf16 -> + residual -> norm)."""
    from open_instruct_b200.ops import fused as f
    from open_instruct_b200.ops import lib, ref

    torch.manual_seed(splits)
    M, N, K = 200, 512, 1000
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    S = f.decode_splits(K, splits)
    assert S == (splits if splits != 5 else 4)  # 16 K blocks in 5 slices of 4 would leave the fifth empty: 4 are used
    parts = f.gemm_decode(a, w, plan=(tile[0], tile[1], S))
    lib.check_status()
    assert parts.dtype == torch.float32 and tuple(parts.shape) == (S, M, N)
    per = -(-(-(-K // 64)) // S) * 64
    for sidx in range(S):
        k0, k1 = sidx * per, min(K, (sidx + 1) * per)
        want = a[:, k0:k1].float() @ w[:, k0:k1].float().t()
        assert (parts[sidx] - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())
    total = a.float() @ w.float().t()
    assert ((parts.sum(0) - total).norm() / total.norm()).item() < 1e-3
    res = torch.randn(M, N, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(N, device="cuda")).bfloat16()
    y, h = f.rmsnorm_fwd_parts(parts, g, 1e-5, res)
    h_want = (parts.sum(0).bfloat16().float() + res.float()).bfloat16()
    assert torch.equal(h, h_want)
    y_want = ref.rmsnorm(h_want.float(), g.float(), 1e-5)
    assert ((y.float() - y_want).norm() / y_want.norm()).item() < 5e-3
    y2, h2 = f.rmsnorm_fwd_parts(parts, g, 1e-5, None)
    assert ((y2.float() - ref.rmsnorm(parts.sum(0).bfloat16().float(), g.float(), 1e-5)).norm() / y2.float().norm()).item() < 5e-3
