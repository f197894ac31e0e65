"""Per-kernel timing at Llama-3.1-8B layer shapes (CUDA events, L2 flushed between iterations).

    python -m open_instruct_b200.utils.kernel_bench [--tokens 4096] [--only gemm,attn,...] [--json out.json]

Reports achieved TFLOP/s or GB/s per kernel and the fraction of the measured peaks found in
``MEASURED_PEAKS.json`` at the repository root (copy bandwidth and cuBLAS bf16 GEMM throughput).
With ``--cublas`` the same GEMM shapes are also timed through ``torch.matmul`` for comparison.  With ``--library`` every
kernel family is also timed through the library the reference's trainer reaches for the same op on the same inputs
(``torch.matmul`` = cuBLAS, ``flash_attn_varlen_func`` = FlashAttention-2, liger fused-linear-cross-entropy, ATen
``_fused_adamw_``), each row named ``lib_*``; a library that does not import is reported and skipped.
"""

from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush_buf = None


def _flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_op(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--only", default="")
    ap.add_argument("--cublas", action="store_true")
    ap.add_argument("--json", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--impl", default=None, help="GEMM kernel: 1cta | 2cta (default: library default)")
    ap.add_argument("--shapes", default="", help="GEMM: comma-separated subset of qkv,o,gate_up,down,lm_head")
    ap.add_argument("--decode_m", default="64,256,512", help="decode_gemm: row counts")
    ap.add_argument("--decode_impls", default="1cta,2cta,skinny,skinny128,decode", help="decode_gemm: kernels to time")
    ap.add_argument("--doc_len", type=int, default=0, help="attention: document length (0 = one document of --tokens)")
    ap.add_argument("--pack", default="", help="attention: 'loguniform' = documents with log-uniform lengths in [128, 4096] as in the SFT bench")
    ap.add_argument("--library", action="store_true", help="also time the library kernel for each family (implies --cublas)")
    args = ap.parse_args()
    args.cublas = args.cublas or args.library
    from open_instruct_b200.ops import fused, lib

    hbm, tf, src = _peaks()
    T, D, F, V, Hq, Hkv, Dh = args.tokens, 4096, 14336, 128256, 32, 8, 128
    only = set(filter(None, args.only.split(",")))
    rows = []

    def rec(name, ms, flops=None, bytes_=None):
        r = {"kernel": name, "ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["frac_of_peak"] = round(flops / ms / 1e9 / tf, 3)
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_of_peak"] = round(bytes_ / ms / 1e6 / hbm, 3)
        rows.append(r)
        print(r, flush=True)

    bf = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    if not only or "gemm" in only:
        shapes = {"qkv": (T, (Hq + 2 * Hkv) * Dh, D), "o": (T, D, Hq * Dh), "gate_up": (T, 2 * F, D), "down": (T, D, F),
                  "lm_head": (T, V, D)}
        pick = set(filter(None, args.shapes.split(",")))
        for name, (M, N, K) in shapes.items():
            if pick and name not in pick:
                continue
            x, w, dy = bf(M, K), bf(N, K), bf(M, N)
            fl = 2.0 * M * N * K
            rec(f"gemm_fwd_{name}", time_op(lambda: fused.gemm(x, w, impl=args.impl), args.iters), fl)
            rec(f"gemm_dgrad_{name}", time_op(lambda: fused.gemm(dy, w, b_mn=True, impl=args.impl), args.iters), fl)
            g = torch.zeros(N, K, device="cuda")
            rec(f"gemm_wgrad_{name}", time_op(lambda: fused.gemm(dy, x, g, a_mn=True, b_mn=True, out_mode=fused.OUT_F32_ACC, impl=args.impl), args.iters), fl)
            if args.impl in (None, "2cta"):
                rec(f"gemm_wgrad_red_{name}", time_op(lambda: fused.gemm(dy, x, g, a_mn=True, b_mn=True, out_mode=fused.OUT_F32_RED, impl=args.impl), args.iters), fl)
            if args.cublas:
                rec(f"cublas_fwd_{name}", time_op(lambda: torch.matmul(x, w.t()), args.iters), fl)
                rec(f"cublas_dgrad_{name}", time_op(lambda: torch.matmul(dy, w), args.iters), fl)
                rec(f"cublas_wgrad_{name}", time_op(lambda: torch.matmul(dy.t(), x), args.iters), fl)
            del x, w, dy, g
    if "gemm_layouts" in only:
        # which part of the weight-gradient GEMM costs what: every operand layout x epilogue on one shape (M x N output, K tokens)
        for name, (M, N) in {"gate_up_wgrad": (2 * F, D), "qkv_wgrad": ((Hq + 2 * Hkv) * Dh, D)}.items():
            K = T
            fl = 2.0 * M * N * K
            a_k, a_m = bf(M, K), bf(K, M)
            b_k, b_n = bf(N, K), bf(K, N)
            out16, out32 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16), torch.zeros(M, N, device="cuda")
            for a_mn in (False, True):
                for b_mn in (False, True):
                    for mode, mname, out in ((fused.OUT_BF16, "bf16", out16), (fused.OUT_F32, "f32", out32), (fused.OUT_F32_ACC, "f32acc", out32)):
                        a, b = (a_m if a_mn else a_k), (b_n if b_mn else b_k)
                        rec(f"{name}_a{'MN' if a_mn else 'K'}_b{'MN' if b_mn else 'K'}_{mname}",
                            time_op(lambda: fused.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, out_mode=mode, impl=args.impl), args.iters), fl)
            del a_k, a_m, b_k, b_n, out16, out32
    if "membw" in only:
        # what the memory system delivers to plain streaming kernels (library probes, for the rooflines of the decode path):
        # a copy moves half its bytes in each direction, a reduction only reads
        n = 1 << 30
        src, dst = torch.empty(n, device="cuda", dtype=torch.bfloat16), torch.empty(n, device="cuda", dtype=torch.bfloat16)
        rec("membw_copy_2GiB_read_plus_write", time_op(lambda: dst.copy_(src), args.iters), bytes_=4 * n)
        rec("membw_read_only_sum_2GiB", time_op(lambda: src.view(torch.int32).sum(), args.iters), bytes_=2 * n)
        rec("membw_read_only_max_2GiB", time_op(lambda: src.max(), args.iters), bytes_=2 * n)
        rec("membw_write_only_fill_2GiB", time_op(lambda: dst.zero_(), args.iters), bytes_=2 * n)
        small = src[: 235 * (1 << 19)]
        rec("membw_read_only_sum_235MiB", time_op(lambda: small.view(torch.int32).sum(), args.iters), bytes_=2 * small.numel())
        del src, dst
    if "decode_gemm" in only:
        # decode-sized GEMMs: a stream over the weights; the roofline is HBM bandwidth
        pick = set(filter(None, args.shapes.split(",")))
        for M in (int(m) for m in args.decode_m.split(",")):
            for name, (N, K) in {"qkv": ((Hq + 2 * Hkv) * Dh, D), "o": (D, Hq * Dh), "gate_up": (2 * F, D), "down": (D, F)}.items():
                if pick and name not in pick:
                    continue
                x, w = bf(M, K), bf(N, K)
                by = (N * K + M * K + M * N) * 2
                if "decode" in args.decode_impls.split(",") and M <= 256:
                    plan = fused.decode_gemm_plan(N, K, name in ("o", "down"), M)
                    rec(f"decode_gemm_{name}_M{M}_onewave_{plan[0]}x{plan[1]}_k{plan[2]}", time_op(lambda: fused.gemm_decode(x, w, plan=plan), args.iters), bytes_=by)
                    if plan[2] > 1:  # with the plane-summing norm that consumes the K slices
                        g_, r_ = bf(N), bf(M, N)
                        rec(f"decode_gemm_{name}_M{M}_onewave_plus_norm", time_op(lambda: fused.rmsnorm_fwd_parts(fused.gemm_decode(x, w, plan=plan), g_, 1e-5, r_), args.iters), bytes_=by)
                        rec(f"decode_gemm_{name}_M{M}_onewave_1slice_plus_norm", time_op(lambda: fused.rmsnorm_fwd(fused.gemm_decode(x, w, plan=fused.decode_gemm_plan(N, K, False, M)), g_, 1e-5, res=r_), args.iters), bytes_=by)
                for impl in filter(lambda i: i and i != "decode", args.decode_impls.split(",")):
                    rec(f"decode_gemm_{name}_M{M}_{impl}", time_op(lambda: fused.gemm(x, w, impl=impl), args.iters), bytes_=by)
                if args.cublas:
                    rec(f"lib_cublas_decode_gemm_{name}_M{M}", time_op(lambda: torch.matmul(x, w.t()), args.iters), bytes_=by)
                if name in ("o", "down") and "splitk" in args.decode_impls + ",splitk" * (args.decode_impls == "1cta,2cta,skinny,skinny128,decode"):
                    acc = torch.zeros(M, N, device="cuda")
                    for sk in (2, 4, 8):
                        rec(f"decode_gemm_{name}_M{M}_splitk{sk}", time_op(lambda: fused.gemm_splitk_(acc, x, w, sk), args.iters), bytes_=by)
    if "decode_attn" in only:
        # paged decode attention at the rollout benchmark's shape: 256 sequences (32 prompts x 8 samples that share their
        # 4 prompt pages), contexts 256 + U[1, 256], 8 KV heads x 4 query heads; the roofline is HBM bandwidth over the
        # DISTINCT pages read
        from ..ops.lib import call, ptr, stream_ptr

        Bq, Hq, Hkv, Dh, BLK = 256, 32, 8, 128, 64
        g = torch.Generator().manual_seed(0)
        ctxs = (256 + torch.randint(1, 257, (Bq,), generator=g)).tolist()
        max_blocks = 8
        nblocks = 32 * 4 + Bq * 4
        kc = torch.randn(nblocks, Hkv, BLK, Dh, device="cuda").bfloat16()
        vc = torch.randn(nblocks, Hkv, BLK, Dh, device="cuda").bfloat16()
        bt = torch.zeros(Bq, max_blocks, dtype=torch.int32)
        for b in range(Bq):
            bt[b, :4] = torch.arange(4) + (b // 8) * 4
            bt[b, 4:] = 128 + b * 4 + torch.arange(4)
        pages = sum(-(-c // BLK) - 4 for c in ctxs) + 32 * 4
        by = pages * Hkv * BLK * Dh * 2 * 2
        bt, ctx = bt.cuda(), torch.tensor(ctxs, dtype=torch.int32, device="cuda")
        qkv = torch.randn(Bq, (Hq + 2 * Hkv) * Dh, device="cuda").bfloat16()
        out = torch.empty(Bq, Hq * Dh, device="cuda", dtype=torch.bfloat16)
        outs = {}
        for variant, name in ((1, "block_sync"), (2, "stream_kpt8"), (0, "stream_kpt4")):
            call("b200_paged_decode_variant", variant)
            fn = lambda: call("b200_paged_decode", ptr(qkv), ptr(kc), ptr(vc), ptr(bt), max_blocks, ptr(ctx), Bq, Hq, Hkv, Dh, Dh ** -0.5, 1,
                              ptr(out), None, None, stream_ptr())
            rec(f"decode_attn_{name}_B{Bq}", time_op(fn, args.iters), bytes_=by)
            outs[name] = out.float().clone()
        call("b200_paged_decode_variant", 0)
        for name in ("stream_kpt8", "stream_kpt4"):
            err = ((outs[name] - outs["block_sync"]).norm() / outs["block_sync"].norm()).item()
            print({"check": f"decode_attn_{name}_vs_block_sync", "rel_err": err}, flush=True)
    if not only or "attn" in only:
        L = args.doc_len or T
        lens = [L] * (T // L) + ([T % L] if T % L else [])
        if args.pack == "loguniform":
            from open_instruct_b200.data.synthetic import sft_pack

            gen, lens = torch.Generator().manual_seed(0), []
            while sum(lens) < T:
                cu_h = sft_pack(4096, 1000, gen)["cu_seq_lens_q"].tolist()
                lens += [b - a for a, b in zip(cu_h[:-1], cu_h[1:])]
            lens, L = lens[: max(1, len(lens))], "loguniform"
            T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
        qkv = bf(T, (Hq + 2 * Hkv) * Dh)
        scale = Dh ** -0.5
        out, lse = fused.attn_fwd(qkv, cu, Hq, Hkv, Dh, scale)
        d_out = bf(T, Hq * Dh)
        fl = sum(4.0 * l * l * Dh * Hq / 2 for l in lens)  # causal: half of the full score matrix
        rec(f"attn_fwd_L{L}", time_op(lambda: fused.attn_fwd(qkv, cu, Hq, Hkv, Dh, scale), args.iters), fl)
        rec(f"attn_bwd_L{L}", time_op(lambda: fused.attn_bwd(qkv, out, d_out, lse, cu, Hq, Hkv, Dh, scale), args.iters), 2.5 * fl)
        if args.library:
            try:
                from flash_attn import flash_attn_varlen_func

                q = qkv[:, : Hq * Dh].reshape(T, Hq, Dh).contiguous().requires_grad_(True)
                k = qkv[:, Hq * Dh:(Hq + Hkv) * Dh].reshape(T, Hkv, Dh).contiguous().requires_grad_(True)
                v = qkv[:, (Hq + Hkv) * Dh:].reshape(T, Hkv, Dh).contiguous().requires_grad_(True)
                mx = max(lens)
                fa = lambda: flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, softmax_scale=scale, causal=True)
                with torch.no_grad():
                    rec(f"lib_flash_attn2_fwd_L{L}", time_op(fa, args.iters), fl)
                o = fa()
                do = d_out.view(T, Hq, Dh)
                rec(f"lib_flash_attn2_bwd_L{L}", time_op(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True), args.iters), 2.5 * fl)
                del o, q, k, v
            except Exception as e:  # noqa: BLE001
                print({"kernel": "lib_flash_attn2", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}, flush=True)
        T = args.tokens
    if not only or "elementwise" in only:
        x, r, w = bf(T, D), bf(T, D), bf(D)
        rec("rmsnorm_fwd_res", time_op(lambda: fused.rmsnorm_fwd(x, w, 1e-5, res=r), args.iters), bytes_=T * D * 2 * 4)
        y, h, rstd = fused.rmsnorm_fwd(x, w, 1e-5, res=r)
        dw = torch.zeros(D, device="cuda")
        rec("rmsnorm_bwd", time_op(lambda: fused.rmsnorm_bwd(h, w, rstd, y, r, dw), args.iters), bytes_=T * D * 2 * 4)
        gu = bf(T, 2 * F)
        rec("swiglu_fwd", time_op(lambda: fused.swiglu_fwd(gu), args.iters), bytes_=T * F * 2 * 3)
        da = bf(T, F)
        rec("swiglu_bwd", time_op(lambda: fused.swiglu_bwd_(gu, da), args.iters), bytes_=T * F * 2 * 5)
        qkv = bf(T, (Hq + 2 * Hkv) * Dh)
        pos = torch.arange(T, device="cuda", dtype=torch.int32)
        inv = torch.rand(Dh // 2, device="cuda")
        rec("rope", time_op(lambda: fused.rope_(qkv, pos, inv, Hq, Hkv, Dh), args.iters), bytes_=T * (Hq + Hkv) * Dh * 2 * 2)
        tab = fused.rope_table(pos, inv, Dh)
        rec("rope_from_table", time_op(lambda: fused.rope_(qkv, pos, inv, Hq, Hkv, Dh, table=tab), args.iters), bytes_=T * (Hq + Hkv) * Dh * 2 * 2)
        logits = bf(T, V)
        labels = torch.randint(0, V, (T,), device="cuda")
        rec("logprob_fwd", time_op(lambda: fused.logprob_fwd(logits, labels), args.iters), bytes_=T * V * 2)
        lp, lse, _ = fused.logprob_fwd(logits, labels)
        g = torch.ones(T, device="cuda")
        rec("logprob_bwd", time_op(lambda: fused.logprob_bwd_(logits, labels, lse, g), args.iters), bytes_=T * V * 2 * 2)
        if args.library:
            # lm_head GEMM + log-softmax + label gather, forward and backward, against liger's fused-linear-CE
            h = bf(T, D).requires_grad_(True)
            w = (bf(V, D) * 0.02).requires_grad_(True)
            lab2 = labels.clone()

            def ours_head():
                lg = fused.gemm(h.detach(), w.detach())
                lp2, lse2, _ = fused.logprob_fwd(lg, lab2)
                dl = fused.logprob_bwd_(lg, lab2, lse2, g)
                gw = torch.empty(V, D, device="cuda")
                fused.gemm(dl, h.detach(), gw, a_mn=True, b_mn=True, out_mode=fused.OUT_F32)
                return fused.gemm(dl, w.detach(), b_mn=True)

            fl_head = 3 * 2.0 * T * V * D
            rec("lm_head_logprob_fwd_bwd", time_op(ours_head, args.iters), fl_head)
            try:
                from liger_kernel.transformers.functional import liger_fused_linear_cross_entropy

                def liger_head():
                    loss = liger_fused_linear_cross_entropy(h, w, lab2)
                    return torch.autograd.grad(loss, (h, w))

                rec("lib_liger_flce_fwd_bwd", time_op(liger_head, args.iters), fl_head)
            except Exception as e:  # noqa: BLE001
                print({"kernel": "lib_liger_flce", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}, flush=True)

            def torch_head():
                lg = torch.matmul(h, w.t()).float()
                loss = torch.nn.functional.cross_entropy(lg, lab2)
                return torch.autograd.grad(loss, (h, w))

            rec("lib_torch_linear_ce_fwd_bwd", time_op(torch_head, args.iters), fl_head)
            del h, w
        del logits
        n = 1 << 28
        ma, m_, v_, gr = (torch.zeros(n, device="cuda") for _ in range(4))
        p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        rec("adamw", time_op(lambda: fused.adamw(ma, m_, v_, gr, p16, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1), args.iters),
            bytes_=n * (4 * 4 + 3 * 4 + 2 + 4))
        if args.library:
            st = torch.tensor(1.0, device="cuda")

            def torch_adamw():
                torch._fused_adamw_([ma], [gr], [m_], [v_], [], [st], lr=1e-3, beta1=0.9, beta2=0.999, weight_decay=0.0, eps=1e-8,
                                    amsgrad=False, maximize=False)
                p16.copy_(ma)  # the bf16 working copy the trainer refreshes after the fp32 update

            rec("lib_torch_fused_adamw_plus_bf16_copy", time_op(torch_adamw, args.iters), bytes_=n * (4 * 4 + 3 * 4 + 2 + 4))
    lib.check_status()
    if args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src}, "tokens": T, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
