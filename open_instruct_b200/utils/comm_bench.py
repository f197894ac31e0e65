"""Device-timed micro-benchmark of the fused compute + collective kernels (run under torchrun, one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29720 \
        -m open_instruct_b200.utils.comm_bench --params 8.03e9 --json comm_bench.json

For each kernel: CUDA-event time on the launching stream (max over ranks, after warm-up, inputs far larger than L2), the
bytes each GPU must move over NVLink, and the fraction of the link roofline (bytes / 770 GB/s measured peer-copy rate per
direction per GPU) or, where the kernel is bound by local HBM instead, of the measured copy bandwidth.

* ``zero_reduce_scatter``  owner sums its 1/N slice of every rank's fp32 gradient buffer (+ squared norm)
* ``zero_adamw_allgather`` AdamW on the fp32 shard, bf16 result stored into every rank's working copy
* ``nccl_reduce_scatter`` / ``nccl_all_gather``  the library collectives on the same buffers (baseline)
* ``tp_allreduce_norm``    one-shot all-reduce + residual + RMSNorm, decode- and prefill-sized
* ``ulysses_qkv_scatter``  QKV GEMM with the sequence -> head exchange in its epilogue, against the plain GEMM
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def timed(fn, iters: int = 5, warmup: int = 2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=8.03e9)
    ap.add_argument("--json", default="")
    ap.add_argument("--skip_zero", action="store_true")
    a = ap.parse_args()
    from open_instruct_b200.ops import lib
    from open_instruct_b200.parallel import dist as pdist
    from open_instruct_b200.parallel.symm import SymmetricState
    from open_instruct_b200.parallel.zero import padded_numel

    rank, world, device = pdist.init_distributed()
    hbm = 6551.0
    rows = []

    def rec(name, ms, link_bytes=None, hbm_bytes=None, note=""):
        r = {"kernel": name, "ms": round(ms, 4), "world": world, "note": note}
        if link_bytes:
            r["nvlink_gbs"] = round(link_bytes / ms / 1e6, 1)
            r["frac_of_link"] = round(link_bytes / ms / 1e6 / NVLINK_GBS, 3)
        if hbm_bytes:
            r["hbm_gbs"] = round(hbm_bytes / ms / 1e6, 1)
            r["frac_of_hbm"] = round(hbm_bytes / ms / 1e6 / hbm, 3)
        rows.append(r)
        if rank == 0:
            print(r, flush=True)

    if not a.skip_zero:
        n = padded_numel(int(a.params), world)
        st = SymmetricState(n, device)
        shard = n // world
        st.grads.normal_()
        out, nsq = torch.empty(shard, device=device), torch.zeros(1, device=device)
        master, m, v = torch.randn(shard, device=device), torch.zeros(shard, device=device), torch.zeros(shard, device=device)
        gs = torch.ones(1, device=device)

        def adam():
            st.adamw_allgather(master, m, v, out, rank * shard, gscale=gs, lr=1e-6, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1)
            st.finish_step()

        variants = [("p2p", False)] + ([("multimem", True)] if (st._mc_grads and st._mc_params) else [])
        for tag, mm in variants:
            st.use_multimem = mm
            # P2P: each owner pulls (world - 1) remote slices of 4-byte elements; multimem: the switch adds, the owner's ingress
            # carries one slice, every peer's egress still carries its copy of that slice
            rec(f"zero_reduce_scatter[{tag}]", timed(lambda: st.reduce_scatter_grad(out, nsq)), link_bytes=(world - 1) * shard * 4,
                hbm_bytes=world * shard * 4 + shard * 4, note="link bytes = egress per GPU (the bound for both variants)")
            # each owner pushes its bf16 shard to (world - 1) peers; locally it streams 16 B read + 12 B written per element
            rec(f"zero_adamw_allgather[{tag}]", timed(adam), link_bytes=(world - 1) * shard * 2, hbm_bytes=shard * 30)
        st.use_multimem = False
        g32 = st.grads
        rs_out = torch.empty(shard, device=device)
        rec("nccl_reduce_scatter", timed(lambda: dist.reduce_scatter_tensor(rs_out, g32)), link_bytes=(world - 1) * shard * 4)
        p16 = torch.empty(n, dtype=torch.bfloat16, device=device)
        my16 = torch.empty(shard, dtype=torch.bfloat16, device=device)
        rec("nccl_all_gather", timed(lambda: dist.all_gather_into_tensor(p16, my16)), link_bytes=(world - 1) * shard * 2)
        del st, out, master, m, v, rs_out, p16, my16
        torch.cuda.empty_cache()

    if world == 2:
        from open_instruct_b200.models.spec import get_spec
        from open_instruct_b200.ops import fused
        from open_instruct_b200.parallel.tp import TPContext
        from open_instruct_b200.parallel.ulysses import UlyssesContext

        D = 4096
        tp = TPContext(D, 8192, device)
        w = torch.ones(D, dtype=torch.bfloat16, device=device)
        for B in (64, 256, 4096, 8192):
            res = torch.randn(B, D, device=device).bfloat16()

            def ar():
                part = tp.out_buffer(B)
                tp.reduce_norm(part, w, 1e-5, res=res)

            # one peer slice read over NVLink; locally: own partial + residual read, two outputs written
            rec(f"tp_allreduce_norm_B{B}", timed(ar, iters=20), link_bytes=B * D * 2, hbm_bytes=B * D * 2 * 4)
        x = torch.randn(4096, 2048, device=device).bfloat16()
        wo = (torch.randn(D, 2048, device=device) * 0.02).bfloat16()

        def pushed():
            part = tp.row_gemm(x, wo)
            tp.reduce_norm(part, w, 1e-5, res=res[:4096])

        def plain():
            part = fused.gemm(x, wo, tp.out_buffer(4096))
            tp.reduce_norm(part, w, 1e-5, res=res[:4096])

        res = torch.randn(8192, D, device=device).bfloat16()
        rec("tp_rowgemm_push+reduce_T4096", timed(pushed, iters=20), link_bytes=4096 * D * 2, note="GEMM epilogue stores tiles to the peer; local reduce")
        rec("tp_rowgemm+pull_reduce_T4096", timed(plain, iters=20), link_bytes=4096 * D * 2, note="plain GEMM; reduce pulls the peer's slot")
        spec = get_spec("llama3.1-8b").replace(num_layers=1)
        sp = UlyssesContext(spec, 8192, device)
        n1 = torch.randn(4096, D, device=device).bfloat16()
        wqkv = (torch.randn(spec.qkv_dim, D, device=device) * 0.02).bfloat16()
        fl = 2.0 * 4096 * spec.qkv_dim * D
        t_sc = timed(lambda: sp.qkv_project(0, n1, wqkv, 8192), iters=20)
        t_pl = timed(lambda: fused.gemm(n1, wqkv), iters=20)
        rec("ulysses_qkv_scatter_T4096", t_sc, link_bytes=4096 * spec.qkv_dim, note=f"{fl / t_sc / 1e9:.0f} TFLOP/s incl. exchange + barrier; half the columns cross NVLink")
        rec("plain_qkv_gemm_T4096", t_pl, note=f"{fl / t_pl / 1e9:.0f} TFLOP/s, no exchange")
    torch.cuda.synchronize()
    lib.check_status()
    if a.json and rank == 0:
        json.dump({"nvlink_gbs_ref": NVLINK_GBS, "hbm_gbs_ref": hbm, "rows": rows}, open(a.json, "w"), indent=1)
    pdist.barrier()
    pdist.destroy()


if __name__ == "__main__":
    main()
