"""Library-stack arm of the SFT benchmark: the same step, built from the libraries the reference's trainer is made of.

This is NOT the reference trainer (its ``finetune.py`` needs accelerate + DeepSpeed, which are not installable
offline).  It is the compute stack that trainer drives, minus the accelerate / DeepSpeed wrapper
(``open_instruct/finetune.py:571-598`` model load with liger or plain bf16 + FlashAttention-2, ``:680`` fused AdamW,
``:822-849`` step): Hugging Face ``LlamaForCausalLM`` built from the same architecture, bf16 compute,
``attn_implementation="flash_attention_2"`` on the padding-free batch (``cu_seq_lens_q/k`` + ``position_ids``), liger
kernels (RMSNorm, RoPE, SwiGLU, fused-linear-CE) where they import, cuBLAS GEMMs, ``torch.optim.AdamW(fused=True)`` on
fp32 master weights, gradient clipping, and for more than one GPU PyTorch ``fully_shard`` (FSDP2: fp32 sharded
parameters, bf16 all-gather, fp32 reduce-scatter after every micro-batch; the ZeRO-3 schedule) over NCCL.  None of
this repository's kernels, model or engine is on this path.

It consumes the same synthetic packs, warm-up, step count and timed regions as ``bench.py`` and prints the same JSON
shape with ``"impl": "hf_stack"``.
"""

from __future__ import annotations

import json
import os
import time

import torch


def _build_model(spec, device, attn: str, use_liger: bool, dtype):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=spec.vocab_size, hidden_size=spec.hidden_size, intermediate_size=spec.intermediate_size,
                      num_hidden_layers=spec.num_layers, num_attention_heads=spec.num_heads, num_key_value_heads=spec.num_kv_heads,
                      head_dim=spec.head_dim, rms_norm_eps=spec.rms_norm_eps, rope_theta=spec.rope_theta,
                      max_position_embeddings=max(8192, spec.max_position_embeddings if hasattr(spec, "max_position_embeddings") else 8192),
                      tie_word_embeddings=spec.tie_word_embeddings, attention_bias=False, use_cache=False)
    cfg._attn_implementation = attn
    liger = []
    if use_liger:
        try:
            from liger_kernel.transformers import apply_liger_kernel_to_llama

            apply_liger_kernel_to_llama(rope=True, swiglu=True, rms_norm=True, cross_entropy=False, fused_linear_cross_entropy=True)
            liger = ["rope", "swiglu", "rms_norm", "fused_linear_cross_entropy"]
        except Exception as e:  # noqa: BLE001 - any incompatibility of the installed liger with the installed transformers
            liger = [f"unavailable: {type(e).__name__}: {str(e)[:120]}"]
    torch.manual_seed(0)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).to(dtype)
    model.train()
    return model, liger


def _hf_batch(mb: dict, device, non_blocking=False) -> dict:
    """The reference collator's batch (``open_instruct/padding_free_collator.py:67-120``): batch dimension 1, labels with
    -100 on every document's first token (HF shifts inside the loss), FlashAttention varlen boundaries."""
    cu = mb["cu_seq_lens_q"].to(device, non_blocking=non_blocking)
    return {"input_ids": mb["input_ids"].to(device, non_blocking=non_blocking)[None],
            "labels": mb["labels"].to(device, non_blocking=non_blocking)[None],
            "position_ids": mb["position_ids"].to(device, non_blocking=non_blocking)[None],
            "cu_seq_lens_q": cu, "cu_seq_lens_k": cu, "max_length_q": int(mb["max_length_q"]), "max_length_k": int(mb["max_length_k"]),
            "use_cache": False}


class HFStackLearner:
    """bf16 model + fp32 master weights + fused AdamW (one GPU), or FSDP2 mixed precision (several GPUs)."""

    def __init__(self, spec, device, world: int, lr: float, max_grad_norm: float, attn: str = "flash_attention_2",
                 use_liger: bool = True, grad_accum_dtype: str = "fp32"):
        self.device, self.world, self.max_grad_norm = device, world, max_grad_norm
        self.fsdp = world > 1
        if self.fsdp:
            from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

            self.model, self.liger = _build_model(spec, device, attn, use_liger, torch.float32)
            mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            for layer in self.model.model.layers:
                fully_shard(layer, mp_policy=mp)
            fully_shard(self.model, mp_policy=mp)
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=0.0, fused=True)
            self.master = None
        else:
            self.model, self.liger = _build_model(spec, device, attn, use_liger, torch.bfloat16)
            self.params = [p for p in self.model.parameters() if p.requires_grad]
            self.master = [p.detach().float() for p in self.params]
            self.accum32 = grad_accum_dtype == "fp32"
            for m in self.master:
                m.grad = torch.zeros_like(m)
            self.opt = torch.optim.AdamW(self.master, lr=lr, weight_decay=0.0, fused=True)
        self.sched = torch.optim.lr_scheduler.LambdaLR(self.opt, lambda s: min(1.0, (s + 1) / 30.0))

    def step(self, micro_batches: list[dict]) -> torch.Tensor:
        n = len(micro_batches)
        total = None
        for mb in micro_batches:
            out = self.model(**mb)
            loss = out.loss / n
            loss.backward()
            if not self.fsdp and self.accum32:  # DeepSpeed bf16 mode accumulates in fp32 (grad_accum_dtype fp32)
                grads = [p.grad for p in self.params]
                torch._foreach_add_([m.grad for m in self.master], grads)
                for p in self.params:
                    p.grad = None
            total = loss.detach() if total is None else total + loss.detach()
        if self.fsdp:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
        else:
            if not self.accum32:
                with torch.no_grad():
                    torch._foreach_copy_([m.grad for m in self.master], [p.grad for p in self.params])
                for p in self.params:
                    p.grad = None
            torch.nn.utils.clip_grad_norm_(self.master, self.max_grad_norm, foreach=True)
            self.opt.step()
            torch._foreach_zero_([m.grad for m in self.master])
            with torch.no_grad():
                torch._foreach_copy_(self.params, self.master)  # bf16 working copy refreshed from the master
        self.sched.step()
        return total


def run(args) -> int:
    from ..data.collate import pin
    from ..data.synthetic import sft_step_batches
    from ..models import get_spec
    from ..parallel import dist as pdist
    from .clocks import ClockSampler

    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    rank, world, device = pdist.init_distributed()
    spec = get_spec(args.model)
    attn = getattr(args, "hf_attn", None) or ("flash_attention_2" if device.type == "cuda" else "sdpa")
    learner = HFStackLearner(spec, device, world, lr=5e-6, max_grad_norm=1.0, attn=attn, use_liger=not getattr(args, "no_liger", False),
                             grad_accum_dtype=getattr(args, "hf_grad_accum", "fp32"))
    total_steps = args.warmup + 2 * args.steps
    keys = ("input_ids", "labels", "position_ids", "cu_seq_lens_q")
    host = []
    for i in range(total_steps):
        mbs = sft_step_batches(args.packs_per_gpu, args.seq_len, spec.vocab_size, seed=1000 * (rank + 1) + i, packs_per_micro=args.packs_per_micro)
        host.append([dict(pin({k: mb[k] for k in keys}), max_length_q=mb["max_length_q"], max_length_k=mb["max_length_k"]) for mb in mbs])
    h2d_bytes = sum(t.numel() * t.element_size() for mb in host[0] for t in mb.values() if torch.is_tensor(t))
    cuda = device.type == "cuda"

    def sync():
        pdist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(fn):
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            t0 = time.perf_counter()
            fn()
            e1.record()
            sync()
            return e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3
        t0 = time.perf_counter()
        fn()
        ms = (time.perf_counter() - t0) * 1e3
        return ms, ms

    for i in range(args.warmup):
        loss = learner.step([_hf_batch(mb, device) for mb in host[i]])
    sync()
    staged = [[_hf_batch(mb, device) for mb in host[args.warmup + i]] for i in range(args.steps)]
    sync()
    sampler = ClockSampler(device.index or 0).start() if cuda else None
    box = {}

    def phase_a():
        for i in range(args.steps):
            box["loss"] = learner.step(staged[i])

    ms_dev, _ = timed(phase_a)
    ms_dev = pdist.max_over_ranks(ms_dev, device)
    clocks = sampler.stop() if sampler is not None else None
    del staged
    sync()

    def phase_b():
        for i in range(args.steps):
            mbs = [_hf_batch(mb, device, non_blocking=True) for mb in host[args.warmup + args.steps + i]]
            box["loss"] = learner.step(mbs)
            box["last"] = float(box["loss"].item())

    ms_b, wall_b = timed(phase_b)
    ms_e2e = pdist.max_over_ranks(max(ms_b, wall_b), device)
    tokens = world * args.packs_per_gpu * args.seq_len * args.steps
    value = tokens / (ms_dev / 1e3)
    result = {
        "impl": "hf_stack", "metric": "sft_train_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (same packs as the default arm; random-init weights)",
        "config": {"model": args.model, "global_batch": world * args.packs_per_gpu, "seq_len": args.seq_len,
                   "micro_batch_tokens": args.seq_len * args.packs_per_micro,
                   "stack": f"transformers LlamaForCausalLM, attn={attn}, liger={learner.liger}, torch fused AdamW on fp32 master, "
                            + ("FSDP2 fully_shard (fp32 shards, bf16 all-gather, fp32 reduce-scatter) over NCCL" if world > 1
                               else f"single GPU, {getattr(args, 'hf_grad_accum', 'fp32')} gradient accumulation"),
                   "note": "library stack of the reference trainer without accelerate/DeepSpeed; not the reference arm",
                   "l2": "per-step working set far exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks, "gpu_launches": 0, "loss": float(box["loss"].item()),
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30 if cuda else 0.0,
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
                "ms_per_step": ms_e2e / args.steps, "last_loss": box.get("last")},
    }
    if rank == 0:
        print(json.dumps(result))
    pdist.barrier()
    pdist.destroy()
    return 0
