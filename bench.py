"""Headline benchmark: SFT training tokens/s at Llama-3.1-8B architecture.

    python bench.py --gpus N --steps K --warmup W        (N > 1: launched under torchrun, one rank per GPU)

One step = one optimizer step over ``packs_per_gpu`` packed rows of ``seq_len`` tokens per GPU
(weak scaling: 16 rows of 4096 per GPU, i.e. the 128-row global batch of the 8-GPU recipe),
synthetic data (example lengths log-uniform in [128, 4096], first 30 % of each example masked),
random-init bf16 weights, fp32 master + AdamW moments sharded over ranks, fp32 gradient
accumulation, full optimizer step inside the timed region.

Two timed phases of K steps each, both bracketed by barrier + synchronize and timed with CUDA
events on the launching stream, max over ranks:
  * ``value``  - device-timed with the step inputs already resident on the device;
  * ``e2e``    - through ``Learner.sft_step`` with every step's inputs copied from pinned host
                 memory inside the timed region and the step loss read back to the host.
Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# published context number: Olmo-3-7B SFT on 8xH100 derived from the reference's docs
# (1723 steps x 1,048,576 tokens in ~9.5 h = 52.8k tok/s = 6.6k tok/s per GPU)
BASELINE_TOK_S_PER_GPU = 6600.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "hf_stack"],
                    help="ours: this framework; reference: the unmodified reference (prints 'unavailable' where it cannot run); "
                         "hf_stack: transformers + FlashAttention-2 + liger + torch fused AdamW / FSDP2 over NCCL, the libraries the "
                         "reference trainer drives, without its accelerate/DeepSpeed wrapper (a same-box anchor, not the reference arm)")
    ap.add_argument("--hf_attn", default=None, help="hf_stack: attention implementation (default flash_attention_2 on CUDA)")
    ap.add_argument("--hf_grad_accum", default="fp32", choices=["fp32", "bf16"], help="hf_stack, one GPU: gradient accumulation dtype")
    ap.add_argument("--no_liger", action="store_true", help="hf_stack: plain transformers modules")
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--seq_len", type=int, default=4096)
    ap.add_argument("--packs_per_gpu", type=int, default=16)
    ap.add_argument("--packs_per_micro", type=int, default=1)
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"])
    ap.add_argument("--ops", default="fused", choices=["fused", "ref"])
    ap.add_argument("--gradient_checkpointing", action="store_true")
    ap.add_argument("--skip_e2e", action="store_true")
    ap.add_argument("--shard_parameters", action="store_true",
                    help="sft: ZeRO-3 style gather-on-use parameter sharding instead of the resident bf16 copy (for models that do not fit)")
    ap.add_argument("--task", default="sft", choices=["sft", "dpo", "grpo"],
                    help="sft: the headline metric; dpo: DPO train tokens/s with cached reference log-probs (same JSON shape); "
                         "grpo: RLVR step seconds (learner + rollout-engine processes, weight sync every step)")
    ap.add_argument("--grpo_response_length", type=int, default=2048)
    ap.add_argument("--grpo_prompts", type=int, default=64)
    ap.add_argument("--grpo_samples", type=int, default=8)
    ap.add_argument("--grpo_layout", default="", help="--task grpo: learners,engines,engine_tp overriding the default split of --gpus")
    ap.add_argument("--pairs_per_gpu", type=int, default=16)
    ap.add_argument("--pairs_per_micro", type=int, default=2)
    return ap.parse_args()


def reference_arm(args) -> None:
    """The unmodified reference cannot run here: its trainers import accelerate, deepspeed, ray
    and beaker at module load and none of them is installed or in the offline wheelhouse."""
    why = ("reference finetune.py needs accelerate+deepspeed (+ray, peft, beaker-py, olmo-core) which are not "
           "installed and not in the offline wheel folder; pip --no-deps install of the reference yields no importable module")
    try:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
        import importlib

        for mod in ("accelerate", "deepspeed"):
            importlib.import_module(mod)
        why = "reference dependencies import, but the reference package itself is not importable from baseline/_ref"
    except Exception as e:  # noqa: BLE001
        why = f"{why} ({type(e).__name__}: {e})"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why[:400]}))


def run_dpo(args) -> int:
    """DPO (length-normalised sigmoid loss, beta 5) on synthetic pairs: shared prompt of 64-512 tokens, independent
    responses of 64-1024 tokens, max length 2048, reference log-probs from a cache built before the timed region
    (``dpo_tune_cache`` path).  Tokens/s counts every chosen and rejected token that goes through the model."""
    import torch

    from open_instruct_b200.data.collate import TensorDataCollatorWithFlatteningDPO, pin, to_device
    from open_instruct_b200.data.synthetic import dpo_pairs
    from open_instruct_b200.dpo_utils import DPOConfig, compute_loss, concatenated_forward
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.ops import lib
    from open_instruct_b200.parallel import dist as pdist
    from open_instruct_b200.utils.clocks import ClockSampler

    rank, world, device = pdist.init_distributed()
    spec = get_spec(args.model)
    learner = Learner(spec, LearnerConfig(ops=args.ops, comm=args.comm, learning_rate=5e-7, lr_scheduler_type="linear", warmup_steps=30,
                                          total_steps=1000, max_grad_norm=1.0, gradient_checkpointing=args.gradient_checkpointing, seed=0),
                      device=device)
    dcfg = DPOConfig(loss_type="dpo_norm", beta=5.0)
    total_steps = args.warmup + 2 * args.steps
    collate = TensorDataCollatorWithFlatteningDPO()
    n = args.pairs_per_gpu
    host, index = [], 0
    for i in range(total_steps):
        rows = dpo_pairs(n, spec.vocab_size, seed=7000 * (rank + 1) + i, max_len=2048)
        for r in rows:
            r["index"] = index
            index += 1
        host.append([pin(collate(rows[j:j + args.pairs_per_micro])) for j in range(0, n, args.pairs_per_micro)])
    # reference cache: one forward-only pass of the initial policy over every pair (not timed, as in the cached trainer)
    cache = {"chosen_logps": torch.zeros(index, device=device), "rejected_logps": torch.zeros(index, device=device)}
    with torch.no_grad():
        for mbs in host:
            for mb in mbs:
                mb = to_device(mb, device)
                pc, pr, _ = concatenated_forward(learner, mb, average_log_prob=True)
                cache["chosen_logps"][mb["index"]] = pc
                cache["rejected_logps"][mb["index"]] = pr

    def step(mbs):
        ntok = 0
        for k, mb in enumerate(mbs):
            pc, pr, aux = concatenated_forward(learner, mb, average_log_prob=True)
            losses, _, _ = compute_loss(dcfg, mb, pc, pr, cache, (aux["chosen_tokens"], aux["rejected_tokens"]))
            learner.backward(losses.mean(), last=(k == len(mbs) - 1))
            ntok += mb["chosen_input_ids"].numel() + mb["rejected_input_ids"].numel()
        learner.optimizer_step()
        return losses.mean().detach(), ntok

    def sync():
        pdist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step([to_device(mb, device) for mb in host[i]])
    sync()
    lib.check_status()
    staged = [[to_device(mb, device) for mb in host[args.warmup + i]] for i in range(args.steps)]
    sync()
    sampler = ClockSampler(device.index or 0).start()
    l0 = lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    tok = 0
    for i in range(args.steps):
        loss, nt = step(staged[i])
        tok += nt
    e1.record()
    sync()
    ms = pdist.max_over_ranks(e0.elapsed_time(e1), device)
    launches = lib.launch_count - l0
    clocks = sampler.stop()
    t = torch.tensor([float(tok)], device=device)
    pdist.all_reduce_(t)
    tok_all = float(t.item())
    del staged
    sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    f0.record()
    tok2, h2d, lv = 0, 0, 0.0
    for i in range(args.steps):
        mbs = [to_device(mb, device, non_blocking=True) for mb in host[args.warmup + args.steps + i]]
        h2d = sum(v.numel() * v.element_size() for mb in host[args.warmup + args.steps + i] for v in mb.values() if torch.is_tensor(v))
        loss, nt = step(mbs)
        lv = float(loss.item())
        tok2 += nt
    f1.record()
    sync()
    ms2 = pdist.max_over_ranks(max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3), device)
    t = torch.tensor([float(tok2)], device=device)
    pdist.all_reduce_(t)
    lib.check_status()
    value = tok_all / (ms / 1e3)
    result = {"metric": "dpo_train_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
              "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
              "dtype": "bf16", "data": "synthetic preference pairs (shared random prompt 64-512, random responses 64-1024, random-init weights)",
              "config": {"model": args.model, "global_batch": world * n, "max_len": 2048, "pairs_per_micro_batch": args.pairs_per_micro,
                         "loss": "dpo_norm beta 5, cached reference log-probs (built before the timed region)",
                         "parallelism": (f"dp{world} zero-sharded optimizer ({learner.comm} comm), resident bf16 params" if learner.z3 is None else
                            f"dp{world} parameters, gradients and optimizer sharded, layers gathered on use ({learner.z3.comm} transport)"), "ops": learner.ops,
                         "l2": "per-step working set far exceeds the 126 MB L2; no explicit flush"},
              "clocks": clocks, "gpu_launches": launches, "loss": float(loss.item()), "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
              "e2e": {"value": float(t.item()) / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                      "ms_per_step": ms2 / args.steps, "last_loss": lv}}
    if rank == 0:
        print(json.dumps(result))
    pdist.barrier()
    pdist.destroy()
    return 0


def run_grpo(args) -> int:
    """GRPO step seconds with the GPUs of the node split between learner ranks and rollout engines the way the 8-GPU recipe
    does (4 learners + 2 engines of tensor-parallel size 2); fewer GPUs keep the learner : engine ratio at 1 : 1.  The GRPO
    driver starts its own actor processes (one per GPU), so under ``torchrun`` only rank 0 runs it and the others leave."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID", "GROUP_RANK", "ROLE_RANK", "LOCAL_WORLD_SIZE",
              "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS"):
        os.environ.pop(k, None)  # the actors rendezvous among themselves
    import bench_grpo

    n = max(1, args.gpus)
    layout = {1: ["--single_gpu_mode"], 2: ["--learners", "1", "--engines", "1"], 4: ["--learners", "2", "--engines", "2"],
              8: ["--learners", "4", "--engines", "2", "--engine_tp", "2"]}.get(n)
    if args.grpo_layout:  # "learners,engines,engine_tp", e.g. 2,1,2 = the 8-GPU recipe's shape on 4 GPUs
        nl, ne, tp = (int(x) for x in args.grpo_layout.split(","))
        if nl + ne * tp != n:
            raise SystemExit(f"--grpo_layout {args.grpo_layout} needs {nl + ne * tp} GPUs, --gpus says {n}")
        layout = ["--learners", str(nl), "--engines", str(ne), "--engine_tp", str(tp)]
    if layout is None:
        raise SystemExit("--task grpo runs on 1, 2, 4 or 8 GPUs")
    import torch

    layout = layout + ["--ops", "fused" if torch.cuda.is_available() else "ref"]
    return bench_grpo.main(layout + ["--steps", str(args.steps + args.warmup), "--warmup", str(args.warmup), "--model", args.model,
                                     "--prompts", str(args.grpo_prompts), "--samples", str(args.grpo_samples),
                                     "--response_length", str(args.grpo_response_length), "--pack_length", str(max(4096, args.grpo_response_length + 256))])


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return 0
    if args.impl == "hf_stack":
        from open_instruct_b200.utils.hf_stack_bench import run as run_hf_stack

        return run_hf_stack(args)
    if args.task == "dpo":
        return run_dpo(args)
    if args.task == "grpo":
        return run_grpo(args)
    import torch

    from open_instruct_b200.data.collate import pin, to_device
    from open_instruct_b200.data.synthetic import sft_step_batches
    from open_instruct_b200.learner import Learner, LearnerConfig
    from open_instruct_b200.models import get_spec
    from open_instruct_b200.ops import lib
    from open_instruct_b200.parallel import dist as pdist
    from open_instruct_b200.utils.clocks import ClockSampler

    rank, world, device = pdist.init_distributed()
    if world != args.gpus and rank == 0:
        print(f"[bench] note: WORLD_SIZE={world} but --gpus {args.gpus}; using WORLD_SIZE", file=sys.stderr)
    spec = get_spec(args.model)
    total_steps = args.warmup + 2 * args.steps
    cfg = LearnerConfig(ops=args.ops, comm=args.comm, learning_rate=5e-6, lr_scheduler_type="linear",
                        warmup_steps=max(1, int(0.03 * 1000)), total_steps=1000, max_grad_norm=1.0,
                        gradient_checkpointing=args.gradient_checkpointing, seed=0, shard_parameters=True if args.shard_parameters else None)
    learner = Learner(spec, cfg, device=device)

    def host_step(i):
        return [pin(b) for b in sft_step_batches(args.packs_per_gpu, args.seq_len, spec.vocab_size,
                                                 seed=1000 * (rank + 1) + i, packs_per_micro=args.packs_per_micro)]

    keys = ("input_ids", "position_ids", "cu_seq_lens_q", "labels_shifted")
    host = [[{k: mb[k] for k in keys} for mb in host_step(i)] for i in range(total_steps)]
    h2d_bytes = sum(t.numel() * t.element_size() for mb in host[0] for t in mb.values())

    def sync():
        pdist.barrier()
        torch.cuda.synchronize()

    # ---------------- warm-up (also allocates every buffer the steps need)
    for i in range(args.warmup):
        out = learner.sft_step([to_device(mb, device) for mb in host[i]])
    sync()
    lib.check_status()

    # ---------------- phase A: device-resident inputs
    staged = [[to_device(mb, device) for mb in host[args.warmup + i]] for i in range(args.steps)]
    # device time of the optimizer step alone (gradient exchange + clip + AdamW + bf16 refresh): events around the call,
    # read after the timed region
    opt_events = []
    plain_optimizer_step = learner.optimizer_step

    def timed_optimizer_step(*a, **k):
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
        r = plain_optimizer_step(*a, **k)
        ev[1].record()
        opt_events.append(ev)
        return r

    learner.optimizer_step = timed_optimizer_step
    sync()
    sampler = ClockSampler(device.index or 0).start()
    launches0 = lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        out = learner.sft_step(staged[i])
    e1.record()
    sync()
    ms_dev = pdist.max_over_ranks(e0.elapsed_time(e1), device)
    launches = lib.launch_count - launches0
    learner.optimizer_step = plain_optimizer_step
    opt_ms = pdist.max_over_ranks(sum(a.elapsed_time(b) for a, b in opt_events) / max(1, len(opt_events)), device)
    clocks = sampler.stop()
    del staged

    # ---------------- phase B: end to end (H2D of inputs from pinned memory + loss read-back per step)
    e2e = None
    if not args.skip_e2e:
        sync()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        f0.record()
        loss_val = 0.0
        for i in range(args.steps):
            mbs = [to_device(mb, device, non_blocking=True) for mb in host[args.warmup + args.steps + i]]
            out = learner.sft_step(mbs)
            loss_val = float(out["loss"].item())  # device -> host read of the step result
        f1.record()
        sync()
        wall_ms = (time.perf_counter() - t0) * 1e3
        ms_e2e = pdist.max_over_ranks(max(f0.elapsed_time(f1), wall_ms), device)
        tokens = world * args.packs_per_gpu * args.seq_len * args.steps
        e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps, "last_loss": loss_val}
    lib.check_status()

    tokens = world * args.packs_per_gpu * args.seq_len * args.steps
    value = tokens / (ms_dev / 1e3)
    result = {
        "metric": "sft_train_tokens_per_second",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps,
        "optimizer_step_ms": opt_ms,  # exchange + clip + AdamW + refresh; its growth with N is the exposed communication
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": value / (BASELINE_TOK_S_PER_GPU * world),
        "vs_baseline_note": "denominator = 6.6k tok/s/GPU derived from the reference's Olmo-3-7B 8xH100 SFT wall-clock "
                            "(different model/hardware; the reference publishes no 8B or B200 tokens/s)",
        "dtype": "bf16",
        "data": "synthetic (uniform-random token ids, log-uniform lengths, random-init weights)",
        "config": {
            "model": args.model,
            "global_batch": world * args.packs_per_gpu,
            "seq_len": args.seq_len,
            "micro_batch_tokens": args.seq_len * args.packs_per_micro,
            "parallelism": (f"dp{world} zero-sharded optimizer ({learner.comm} comm), resident bf16 params" if learner.z3 is None else
                            f"dp{world} parameters, gradients and optimizer sharded, layers gathered on use ({learner.z3.comm} transport)"),
            "ops": learner.ops,
            "optimizer": "AdamW fp32 master+moments, fp32 grad accumulation, clip 1.0, inside timed region",
            "gradient_checkpointing": bool(args.gradient_checkpointing),
            "l2": "per-step working set (>=16 GB weights + 32 GB grads) far exceeds the 126 MB L2; no explicit flush",
        },
        "clocks": clocks,
        "gpu_launches": launches,
        "loss": float(out["loss"].item()),
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
    }
    if e2e is not None:
        result["e2e"] = e2e
    if rank == 0:
        print(json.dumps(result))
    pdist.barrier()
    pdist.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
